"""The call surface of the reference's native extension ``qgemm``
(quant/qgemm/kernels/bindings.cpp:98-134): ``sym_quant``, ``matmul``, ``sym_dequant`` on the packed
int4 format, so that ``quant/qgemm/bench_int4.py`` runs against this library with
``import sam_quantization_b200.qgemm as qgemm``.

Same tensor conventions: ``x`` fp16 [M, K] and ``scale`` fp16 [M, 1] -> packed uint8 [M, ceil(K/2)]
(two 4-bit two's-complement codes per byte, low nibble first); ``matmul(A, B)`` takes both operands
packed, [M, K/2] and [N, K/2], and returns int32 [M, N]; ``sym_dequant(q, scale_row, scale_col, 32)``
returns fp16.  Preconditions raise ``RuntimeError`` like the reference's ``torch::check*`` calls.
Plus ``pack_int4`` / ``unpack_int4`` for weights quantized with ``n_bits = 4``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .ops import _ptr, _stream, status_word


def _check(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")


@torch.no_grad()
def sym_quant(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """bindings.cpp:29-48 -> quant.cu:11-61."""
    _check(x, "x", torch.float16)
    _check(scale, "scale", torch.float16)
    if x.dim() != 2 or scale.shape[0] != x.shape[0] or scale.numel() != x.shape[0] or scale.device != x.device:
        raise RuntimeError("sym_quant expects x [rows, cols] and scale [rows, 1] on the same GPU")
    rows, cols = x.shape
    q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().samq_sym_quant_i4(_ptr(x), _ptr(scale), rows, cols, cols, _ptr(q), _stream()))
    return q


@torch.no_grad()
def matmul(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """bindings.cpp:7-26 -> gemm.cu:6-45: int32 [M, N] from packed [M, K/2] and [N, K/2]."""
    _check(A, "A", torch.uint8)
    _check(B, "B", torch.uint8)
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[1] or A.device != B.device:
        raise RuntimeError("matmul expects packed A [M, K/2] and B [N, K/2] on the same GPU")
    M, N, K = A.shape[0], B.shape[0], 2 * A.shape[1]
    Kp = (K + 15) // 16 * 16
    ws = torch.empty(((M + N) * Kp,), dtype=torch.int8, device=A.device)
    C = torch.empty((M, N), dtype=torch.int32, device=A.device)
    with torch.cuda.device(A.device):
        _lib.check(_lib.load().samq_matmul_i4(_ptr(A), _ptr(B), M, N, K, _ptr(ws), ctypes.c_size_t(ws.numel()), _ptr(C),
                                              _ptr(status_word(A.device)), _stream()))
    return C


@torch.no_grad()
def sym_dequant(q: torch.Tensor, scale_row: torch.Tensor, scale_col: torch.Tensor, bits: int) -> torch.Tensor:
    """bindings.cpp:51-91 -> quant.cu:64-97; only ``bits == 32`` exists there."""
    _check(q, "q")
    _check(scale_row, "scale_row", torch.float16)
    _check(scale_col, "scale_col", torch.float16)
    if bits != 32 or q.dtype != torch.int32:
        raise RuntimeError("Unsupported data type")
    rows, cols = q.shape
    if scale_row.shape[0] != rows or scale_col.shape[0] != cols:
        raise RuntimeError("sym_dequant expects scale_row [rows, ...] and scale_col [cols, ...]")
    out = torch.empty((rows, cols), dtype=torch.float16, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().samq_sym_dequant_i32(_ptr(q), _ptr(scale_row), _ptr(scale_col), rows, cols, _ptr(out), _stream()))
    return out


@torch.no_grad()
def pack_int4(codes: torch.Tensor) -> torch.Tensor:
    """int8 codes in [-8, 7], [rows, cols] -> packed uint8 [rows, ceil(cols / 2)]."""
    _check(codes, "codes", torch.int8)
    rows, cols = codes.shape
    q = torch.empty((rows, (cols + 1) // 2), dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        _lib.check(_lib.load().samq_pack_i4(_ptr(codes), rows, cols, cols, _ptr(q), q.shape[1], _stream()))
    return q


@torch.no_grad()
def unpack_int4(q: torch.Tensor, cols: int) -> torch.Tensor:
    """packed uint8 [rows, ceil(cols / 2)] -> int8 codes [rows, cols]."""
    _check(q, "q", torch.uint8)
    rows = q.shape[0]
    if q.shape[1] != (cols + 1) // 2:
        raise RuntimeError("packed width does not match cols")
    out = torch.empty((rows, cols), dtype=torch.int8, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().samq_unpack_i4(_ptr(q), rows, cols, q.shape[1], _ptr(out), cols, _stream()))
    return out
