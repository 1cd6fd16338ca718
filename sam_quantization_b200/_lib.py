"""ctypes binding of libsamq.so (declarations: include/samq.h).

The library is the only compute path of this package: if it is missing or does not load,
importing a compute function raises — there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int8, c_int32, c_int64, c_size_t, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libsamq.so")

# enums of include/samq.h
F16, BF16, F32, I32 = 0, 1, 2, 3
GRAN_ROW, GRAN_TENSOR, GRAN_GROUP = 0, 1, 2
ACT_NONE, ACT_GELU = 0, 1
HAD_NONE, HAD_FULL, HAD_PARTIAL = 0, 1, 2

EXPORTED_SYMBOLS = (
    "samq_version",
    "samq_last_error_string",
    "samq_quant_workspace_bytes",
    "samq_act_quant_i8",
    "samq_act_quant_i8_ex",
    "samq_weight_quant_i8",
    "samq_act_quant_per_tensor_static",
    "samq_gemm_i8",
    "samq_gemm_set_pair_mode",
    "samq_gemm_i8_stall_selftest",
    "samq_sym_quant_i4",
    "samq_pack_i4",
    "samq_unpack_i4",
    "samq_matmul_i4",
    "samq_sym_dequant_i32",
    "samq_attn_window_prep",
    "samq_attn_rel_bias",
    "samq_attn_windowed",
    "samq_attn_transpose_v",
    "samq_attn_global",
    "samq_attn_window14",
)


class HadamardSpec(Structure):
    """Mirror of ``samq_hadamard_spec``."""

    _fields_ = [
        ("mode", c_int32),
        ("had_k", c_int32),
        ("hadk", c_void_p),
        ("had_dim", c_int32),
        ("signs", c_void_p),
    ]


class QuantPrologue(Structure):
    """Mirror of ``samq_quant_prologue``."""

    _fields_ = [
        ("row_map", c_void_p),
        ("ln_weight", c_void_p),
        ("ln_bias", c_void_p),
        ("ln_eps", c_float),
        ("src_dtype", c_int32),
    ]


class SamqError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference's bindings raise RuntimeError
    from torch::check*/TORCH_CHECK, quant/qgemm/kernels/bindings.cpp:9-17,87)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"samq error {code}: {message}")
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    """Load libsamq.so once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m sam_quantization_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.samq_version.restype = c_int
    lib.samq_version.argtypes = []
    lib.samq_last_error_string.restype = c_char_p
    lib.samq_last_error_string.argtypes = []
    lib.samq_quant_workspace_bytes.restype = c_size_t
    lib.samq_quant_workspace_bytes.argtypes = [c_int]
    lib.samq_act_quant_i8.restype = c_int
    lib.samq_act_quant_i8.argtypes = [
        c_void_p, c_int, c_int64, c_int64, c_int64,      # x, dtype, M, K, ldx
        c_void_p, POINTER(HadamardSpec),                 # divisor, had
        c_int, c_int, c_int,                             # granularity, group_size, n_bits
        c_void_p, c_void_p, c_void_p, c_void_p,          # q, scale, fq, tx
        c_void_p, c_size_t, c_void_p,                    # workspace, bytes, stream
    ]
    lib.samq_act_quant_i8_ex.restype = c_int
    lib.samq_act_quant_i8_ex.argtypes = [
        c_void_p, c_int, c_int64, c_int64, c_int64,      # x, dtype, M (output rows), K, ldx
        POINTER(QuantPrologue),                          # prologue
        c_void_p, POINTER(HadamardSpec),                 # divisor, had
        c_int, c_int, c_int,                             # granularity, group_size, n_bits
        c_void_p, c_void_p, c_void_p, c_void_p,          # q, scale, fq, tx
        c_void_p, c_size_t, c_void_p,                    # workspace, bytes, stream
    ]
    lib.samq_weight_quant_i8.restype = c_int
    lib.samq_weight_quant_i8.argtypes = [
        c_void_p, c_int, c_int64, c_int64, c_int64,
        c_int, c_int, c_int,
        c_void_p, c_void_p, c_void_p,
        c_void_p, c_size_t, c_void_p,
    ]
    lib.samq_act_quant_per_tensor_static.restype = c_int
    lib.samq_act_quant_per_tensor_static.argtypes = [
        c_void_p, c_int, c_int64, c_int64, c_int64, c_int,   # x, dtype, M, K, ldx, n_bits
        c_void_p, c_void_p, c_void_p, c_void_p,              # q, scale, fq, stream
    ]
    lib.samq_gemm_i8.restype = c_int
    lib.samq_gemm_i8.argtypes = [
        c_void_p, c_int64, c_void_p, c_int64,            # A, lda, W, ldw
        c_int64, c_int64, c_int64,                       # M, N, K
        c_void_p, c_int, c_void_p, c_int, c_int,         # a_scale, a_gran, w_scale, w_gran, group
        c_void_p, c_void_p, c_int64,                     # bias, residual, ldr
        c_int, c_void_p, c_int, c_int64,                 # activation, out, out_dtype, ldo
        c_void_p, c_void_p,                              # status, stream
    ]
    lib.samq_gemm_i8_stall_selftest.restype = c_int
    lib.samq_gemm_i8_stall_selftest.argtypes = [
        c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64,   # A, lda, W, ldw, M, N, K
        c_void_p, c_int64, c_int, ctypes.c_longlong, c_void_p, c_void_p,   # out, ldo, skip_kblock, wait_limit_cycles, status, stream
    ]
    lib.samq_sym_quant_i4.restype = c_int
    lib.samq_sym_quant_i4.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]
    lib.samq_pack_i4.restype = c_int
    lib.samq_pack_i4.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p]
    lib.samq_unpack_i4.restype = c_int
    lib.samq_unpack_i4.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p]
    lib.samq_matmul_i4.restype = c_int
    lib.samq_matmul_i4.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]
    lib.samq_sym_dequant_i32.restype = c_int
    lib.samq_sym_dequant_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]
    lib.samq_gemm_set_pair_mode.restype = c_int
    lib.samq_gemm_set_pair_mode.argtypes = [c_int]
    lib.samq_attn_transpose_v.restype = c_int
    lib.samq_attn_transpose_v.argtypes = [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.samq_attn_global.restype = c_int
    lib.samq_attn_global.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int,     # qkv, vt, rel_all, dtype, images, rel_pitch
        c_int, c_int, c_int, c_int, c_float,                     # H, W, heads, head_dim, scale
        c_void_p, c_void_p, c_void_p,                            # out, status, stream
    ]
    lib.samq_attn_window_prep.restype = c_int
    lib.samq_attn_window_prep.argtypes = [
        c_void_p, c_void_p, c_int, c_int64, c_int,              # qkv, rel_all, dtype, tokens, rel_pitch
        c_int, c_int, c_int, c_int, c_float, c_int,             # H, W, heads, head_dim, scale, width
        c_void_p, c_void_p, c_void_p,                           # q_aug, k_aug, stream
    ]
    lib.samq_attn_rel_bias.restype = c_int
    lib.samq_attn_rel_bias.argtypes = [
        c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,   # rel_all, dtype, images, rel_pitch, H, W, heads
        c_void_p, c_void_p,                                     # bias, stream
    ]
    lib.samq_attn_windowed.restype = c_int
    lib.samq_attn_windowed.argtypes = [
        c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,   # qkv, dtype, windows, H, W, heads, head_dim
        c_void_p, c_int, c_float, c_void_p, c_void_p,           # rel_table, table_rows, scale, out, stream
    ]
    lib.samq_attn_window14.restype = c_int
    lib.samq_attn_window14.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int64,              # qkv, rel_table, table_rows, dtype, windows
        c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,    # heads, head_dim, scale, out, status, stream
    ]
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        msg = load().samq_last_error_string()
        raise SamqError(code, msg.decode("utf-8", "replace") if msg else "")
