"""Tensor-level wrappers over the C ABI (include/samq.h).

Each function takes CUDA tensors, allocates the outputs with torch (the library itself never
allocates), passes raw pointers plus the current CUDA stream through ctypes and returns the
outputs.  CPU tensors are rejected: this package has no CPU compute path.
"""
from __future__ import annotations

import ctypes
import weakref
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (ACT_GELU, ACT_NONE, BF16, F16, F32, GRAN_GROUP, GRAN_ROW, GRAN_TENSOR, HAD_FULL,
                   HAD_NONE, HAD_PARTIAL, I32, HadamardSpec, QuantPrologue)

_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}
_OUT_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.int32: I32}

# reference strings (RTN_quantization/per_tensor_channel_group.py:130-140,178-192) -> enum
ACT_GRANULARITY = {"per_token": GRAN_ROW, "per_tensor": GRAN_TENSOR, "per_group_token": GRAN_GROUP}
WEIGHT_GRANULARITY = {"per_channel": GRAN_ROW, "per_tensor": GRAN_TENSOR, "per_group": GRAN_GROUP}


@dataclass
class Hadamard:
    """Online transform applied before quantization (see ``samq_hadamard_spec``).

    mode: "full" (quarot/utils.py:257-261) or "partial" (:263-289)
    had_k / hadk: the explicit Hadamard factor of ``get_hadK`` (1 / None for powers of two)
    had_dim: head width for the partial transform
    signs: optional int8 [K] of +-1 multiplied in before the transform
    """

    mode: str
    had_k: int = 1
    hadk: Optional[torch.Tensor] = None
    had_dim: int = 0
    signs: Optional[torch.Tensor] = None


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: sam_quantization_b200 has no CPU compute path")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_status_words = {}

# ---- launch accounting and optional per-kernel timing (used by bench.py) -----------------------
_launches = 0
_timing_on = False
_timing_records = []          # (kind, start_event, end_event, work, detail)
_valid_rows = {}              # (data_ptr, numel) of a row map -> rows that are not padding


def reset_counters() -> None:
    global _launches
    _launches = 0


def launch_count() -> int:
    """CUDA kernels of this library launched since ``reset_counters()``."""
    return _launches


def enable_kernel_timing(on: bool) -> None:
    """Bracket every C-ABI launch with CUDA events on the launching stream."""
    global _timing_on
    _timing_on = bool(on)
    _timing_records.clear()


def kernel_timing_summary() -> dict:
    """{kind: {"ms", "launches", "ops" | "bytes"}} summed over the bracketed launches
    (synchronises).  ``ops`` = 2*M*N*K per GEMM, ``bytes`` = the algorithmic bytes of K1 (source rows
    actually read x element size + codes + scales).  The GEMM entry also carries ``bytes_alg`` (the
    algorithmic M*K + N*K + out_bytes*M*N) and ``"gemm_shapes"`` maps "KxN" to launches and total rows."""
    torch.cuda.synchronize()
    out = {}
    shapes = {}
    for kind, e0, e1, work, detail in _timing_records:
        d = out.setdefault(kind, {"ms": 0.0, "launches": 0, "ops": 0.0, "bytes": 0.0})
        ms = e0.elapsed_time(e1)
        d["ms"] += ms
        d["launches"] += 1
        d["ops" if kind == "gemm_i8" else "bytes"] += work
        if kind == "gemm_i8" and detail is not None:
            M, N, K, out_bytes = detail
            d["bytes_alg"] = d.get("bytes_alg", 0.0) + M * K + N * K + out_bytes * M * N
            sh = shapes.setdefault(f"{K}x{N}", {"launches": 0, "rows": 0, "ms": 0.0, "ops": 0.0})
            sh["launches"] += 1
            sh["rows"] += M
            sh["ms"] += ms
            sh["ops"] += work
    if shapes:
        out["gemm_shapes"] = shapes
    return out


class _Timed:
    def __init__(self, kind, work, kernels=1, detail=None):
        self.kind, self.work, self.kernels, self.detail = kind, work, kernels, detail

    def __enter__(self):
        global _launches
        _launches += self.kernels
        if _timing_on:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _timing_on:
            self.e1.record()
            _timing_records.append((self.kind, self.e0, self.e1, self.work, self.detail))
        return False


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 that GEMM kernels raise when one of their bounded waits ran out."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status_words[key]


def check_status(device=None) -> None:
    """Synchronise and raise if any GEMM kernel on ``device`` reported a timed-out wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = status_word(dev)
    if int(word.item()) != 0:
        word.zero_()
        raise RuntimeError("samq GEMM kernel gave up on a bounded wait (pipeline stalled)")


def _as_rows(x: torch.Tensor) -> Tuple[torch.Tensor, int, int, int]:
    """View x as [M, K] with a row stride; copies only if the last dim is not contiguous."""
    K = x.shape[-1]
    if x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= K:
        return x, x.shape[0], K, x.stride(0)
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) != K):
        x2 = x2.contiguous()
    return x2, x2.shape[0], K, K


def _spec(had: Optional[Hadamard], keep: list) -> Optional[HadamardSpec]:
    if had is None:
        return None
    mode = {"full": HAD_FULL, "partial": HAD_PARTIAL, "none": HAD_NONE}[had.mode]
    hadk = None
    if had.had_k > 1:
        if had.hadk is None:
            raise ValueError("had_k > 1 needs the hadk matrix")
        hadk = had.hadk.to(dtype=torch.float32).contiguous()
        _require_cuda(hadk, "hadk")
        keep.append(hadk)
    signs = None
    if had.signs is not None:
        signs = had.signs.to(dtype=torch.int8).contiguous()
        _require_cuda(signs, "signs")
        keep.append(signs)
    return HadamardSpec(mode, int(had.had_k), 0 if hadk is None else hadk.data_ptr(), int(had.had_dim),
                        0 if signs is None else signs.data_ptr())


def hadamard_layer_norm_fused(x: torch.Tensor, hadamard: "Hadamard", as_dtype: Optional[torch.dtype] = None) -> bool:
    """True when ``quantize(x, GRAN_ROW, hadamard=..., layer_norm=...)`` runs as one kernel: a full
    power-of-two transform over fp16 rows of 1024 elements (codes and scales only)."""
    return (hadamard is not None and hadamard.mode == "full" and int(hadamard.had_k) == 1 and x.dtype == torch.float16 and
            (as_dtype is None or as_dtype == torch.float16) and x.shape[-1] == 1024)


def quantize(x: torch.Tensor, granularity: int = GRAN_ROW, group_size: Optional[int] = None,
             divisor: Optional[torch.Tensor] = None, hadamard: Optional[Hadamard] = None,
             codes: bool = True, fake_quant: bool = False, transformed: bool = False, n_bits: int = 8,
             row_map: Optional[torch.Tensor] = None, layer_norm=None, as_dtype: Optional[torch.dtype] = None):
    """Run K1 on ``x`` ([..., K]; fp16 / bf16 / fp32).

    Returns a dict with the requested outputs: ``q`` int8 [..., K], ``scale`` fp32
    ([...] | [1] | [..., K/group]), ``fq`` (fake-quantized) and ``tx`` (input after the
    prologue / divisor / Hadamard), both in the tensor dtype.

    Prologue fused into the same kernel (see ``samq_quant_prologue``): ``row_map`` int32 [M_out]
    gathers source rows (negative = a zero row) and makes the outputs ``[M_out, ...]``;
    ``layer_norm=(weight, bias, eps)`` normalises each source row first; ``as_dtype=torch.float16``
    reads a bf16 ``x`` as the fp16 tensor the model would cast it to.
    """
    _require_cuda(x, "x")
    if x.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {x.dtype}")
    lib = _lib.load()
    lead = x.shape[:-1]
    x2, M, K, ldx = _as_rows(x)
    tdtype = x.dtype
    pro = None
    keep_pro = []
    if row_map is not None or layer_norm is not None or (as_dtype is not None and as_dtype != x.dtype):
        pro = QuantPrologue(0, 0, 0, 0.0, -1)
        if row_map is not None:
            _require_cuda(row_map, "row_map")
            if row_map.dtype != torch.int32 or not row_map.is_contiguous():
                raise TypeError("row_map must be a contiguous int32 tensor")
            pro.row_map = row_map.data_ptr()
            M = row_map.numel()
            lead = (M,)
        if as_dtype is not None and as_dtype != x.dtype:
            if not (x.dtype == torch.bfloat16 and as_dtype == torch.float16):
                raise TypeError("as_dtype only reads bf16 storage as an fp16 tensor")
            pro.src_dtype = _DTYPE_CODE[x.dtype]
            tdtype = as_dtype
        if layer_norm is not None:
            ln_w, ln_b, ln_eps = layer_norm
            ln_w = ln_w.detach().to(device=x.device, dtype=tdtype).contiguous()
            ln_b = ln_b.detach().to(device=x.device, dtype=tdtype).contiguous()
            keep_pro += [ln_w, ln_b]
            pro.ln_weight, pro.ln_bias, pro.ln_eps = ln_w.data_ptr(), ln_b.data_ptr(), float(ln_eps)
    g = int(group_size) if granularity == GRAN_GROUP else 0
    if granularity == GRAN_GROUP:
        if not isinstance(group_size, int):
            raise AssertionError("group_size must be an integer")
        if K % g != 0:
            raise AssertionError(f"Last dimension ({K}) must be divisible by group_size ({g})")
    out = {}
    dev = x.device
    q = torch.empty((M, K), dtype=torch.int8, device=dev) if codes else None
    if granularity == GRAN_ROW:
        scale = torch.empty((M,), dtype=torch.float32, device=dev)
    elif granularity == GRAN_TENSOR:
        scale = torch.empty((1,), dtype=torch.float32, device=dev)
    else:
        scale = torch.empty((M, K // g), dtype=torch.float32, device=dev)
    fq = torch.empty((M, K), dtype=tdtype, device=dev) if fake_quant else None
    tx = torch.empty((M, K), dtype=tdtype, device=dev) if transformed else None
    ws_bytes = int(lib.samq_quant_workspace_bytes(granularity))
    ws = torch.empty((max(ws_bytes, 4) // 4,), dtype=torch.int32, device=dev) if ws_bytes else None
    keep = []
    if divisor is not None:
        divisor = divisor.to(device=dev, dtype=tdtype).contiguous()
        if divisor.numel() != K:
            raise ValueError("divisor must have K elements")
    spec = _spec(hadamard, keep)
    rows_read = M
    if _timing_on and row_map is not None:                # padding rows (negative map entries) read nothing
        key = (row_map.data_ptr(), row_map.numel())
        if key not in _valid_rows:
            _valid_rows[key] = int((row_map >= 0).sum().item())
        rows_read = _valid_rows[key]
    nbytes = rows_read * K * x.element_size() + M * ((K if codes else 0) + (K * x.element_size() if fake_quant else 0)
                                                     + (K * x.element_size() if transformed else 0)) + scale.numel() * 4
    with torch.cuda.device(dev), _Timed("act_quant", nbytes, 3 if granularity == GRAN_TENSOR else 1):
        _lib.check(lib.samq_act_quant_i8_ex(
            _ptr(x2), _DTYPE_CODE[tdtype], M, K, ldx,
            ctypes.byref(pro) if pro is not None else None, _ptr(divisor),
            ctypes.byref(spec) if spec is not None else None,
            granularity, g, int(n_bits), _ptr(q), _ptr(scale), _ptr(fq), _ptr(tx),
            _ptr(ws), ws_bytes, _stream()))
    if codes:
        out["q"] = q.view(*lead, K)
    if granularity == GRAN_ROW:
        out["scale"] = scale.view(*lead)
    elif granularity == GRAN_TENSOR:
        out["scale"] = scale
    else:
        out["scale"] = scale.view(*lead, K // g)
    if fake_quant:
        out["fq"] = fq.view(*lead, K)
    if transformed:
        out["tx"] = tx.view(*lead, K)
    return out


def quantize_weight(w: torch.Tensor, granularity: int = GRAN_ROW, group_size: Optional[int] = None,
                    codes: bool = True, fake_quant: bool = False, n_bits: int = 8):
    """Run K3 (weight quantization) on ``w`` [N, K] through ``samq_weight_quant_i8``."""
    _require_cuda(w, "w")
    if w.dim() != 2:
        raise AssertionError("weight must be 2-D")
    if w.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {w.dtype}")
    lib = _lib.load()
    w2, N, K, ldw = _as_rows(w)
    g = int(group_size) if granularity == GRAN_GROUP else 0
    if granularity == GRAN_GROUP:
        if not isinstance(group_size, int):
            raise AssertionError("group_size must be an integer")
        if K % g != 0:
            raise AssertionError(f"in_features ({K}) must be divisible by group_size ({g})")
    dev = w.device
    q = torch.empty((N, K), dtype=torch.int8, device=dev) if codes else None
    shape = {GRAN_ROW: (N,), GRAN_TENSOR: (1,), GRAN_GROUP: (N, K // g if g else 1)}[granularity]
    scale = torch.empty(shape, dtype=torch.float32, device=dev)
    fq = torch.empty((N, K), dtype=w.dtype, device=dev) if fake_quant else None
    ws_bytes = int(lib.samq_quant_workspace_bytes(granularity))
    ws = torch.empty((max(ws_bytes, 4) // 4,), dtype=torch.int32, device=dev) if ws_bytes else None
    with torch.cuda.device(dev), _Timed("weight_quant", N * K * (w.element_size() + 1), 3 if granularity == GRAN_TENSOR else 1):
        _lib.check(lib.samq_weight_quant_i8(
            _ptr(w2), _DTYPE_CODE[w.dtype], N, K, ldw, granularity, g, int(n_bits),
            _ptr(q), _ptr(scale), _ptr(fq), _ptr(ws), ws_bytes, _stream()))
    out = {"scale": scale}
    if codes:
        out["q"] = q
    if fake_quant:
        out["fq"] = fq
    return out


GEMM_GROUP_MULTIPLE = 32        # one tcgen05.mma covers 32 columns of K
GEMM_MAX_GROUPS = 160


def check_gemm_group_size(in_features: int, group_size) -> None:
    """Raise early (at module construction) for a group size the grouped int8 GEMM cannot run: the
    reference's float path accepts any divisor of the width; the tensor-core path needs groups of a
    multiple of 32 columns and at most 160 groups per row."""
    assert type(group_size) == int, "group_size must be an integer"
    assert in_features % group_size == 0, f"in_features ({in_features}) must be divisible by group_size ({group_size})"
    if group_size % GEMM_GROUP_MULTIPLE != 0 or in_features // group_size > GEMM_MAX_GROUPS:
        raise ValueError(f"group_size={group_size} with in_features={in_features}: the int8 GEMM needs group sizes that are "
                         f"multiples of {GEMM_GROUP_MULTIPLE} and at most {GEMM_MAX_GROUPS} groups per row")


GEMM_PAIR_NEVER, GEMM_PAIR_AUTO, GEMM_PAIR_ALWAYS = 0, 1, 2


def set_gemm_pair_mode(mode: int) -> int:
    """Choose the K2 implementation: single CTAs, CTA pairs (tcgen05 cta_group::2), or by size.

    Returns the previous mode.  Both implementations give bit-identical results.
    """
    prev = _lib.load().samq_gemm_set_pair_mode(int(mode))
    if prev < 0:
        raise ValueError(f"unknown GEMM pair mode {mode}")
    return prev


_bias_cache = {}


def _bias_as(bias: torch.Tensor, dtype: torch.dtype, dev) -> torch.Tensor:
    """``bias`` flattened in the epilogue's parameter dtype.  A layer whose output dtype differs from its
    bias dtype (qkv storing bf16 for the attention) would otherwise launch a conversion kernel on every
    call; the converted copy is cached until the bias changes (new storage or an in-place update)."""
    if bias.dtype == dtype and bias.device == dev and bias.dim() == 1 and bias.is_contiguous():
        return bias
    key = (id(bias), bias.data_ptr(), bias._version, dtype, str(dev))
    hit = _bias_cache.get(key)
    if hit is None or hit[0]() is not bias:              # the weak reference guards against a recycled id / address
        if len(_bias_cache) > 4096:
            _bias_cache.clear()
        hit = (weakref.ref(bias), bias.detach().reshape(-1).to(device=dev, dtype=dtype).contiguous())
        _bias_cache[key] = hit
    return hit[1]


def gemm_i8(a_q: torch.Tensor, w_q: torch.Tensor,
            a_scale: Optional[torch.Tensor] = None, w_scale: Optional[torch.Tensor] = None,
            a_gran: int = GRAN_ROW, w_gran: int = GRAN_ROW, group_size: int = 0,
            bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
            activation: int = ACT_NONE, out_dtype: torch.dtype = torch.float16,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Run K2: ``act(dequant(a_q @ w_q.T) + bias) + residual`` -> [..., N] of ``out_dtype``.

    ``out_dtype=torch.int32`` returns the raw accumulators (no scales / bias allowed).
    """
    _require_cuda(a_q, "a_q")
    _require_cuda(w_q, "w_q")
    if a_q.dtype != torch.int8 or w_q.dtype != torch.int8:
        raise TypeError("a_q and w_q must be int8")
    lib = _lib.load()
    lead = a_q.shape[:-1]
    a2, M, K, lda = _as_rows(a_q)
    if w_q.dim() != 2 or w_q.shape[1] != K:
        raise ValueError(f"w_q must be [N, {K}]")
    w2, N, _, ldw = _as_rows(w_q)
    dev = a_q.device
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    else:
        if out.dtype != out_dtype or out.shape[-1] != N or out.numel() != M * N or not out.is_contiguous():
            raise ValueError("out has the wrong dtype, shape or layout")
    param_dtype = torch.float32 if out_dtype in (torch.float32, torch.int32) else out_dtype
    if bias is not None:
        bias = _bias_as(bias, param_dtype, dev)
        if bias.numel() != N:
            raise ValueError("bias must have N elements")
    ldr = 0
    if residual is not None:
        _require_cuda(residual, "residual")
        if residual.dtype != out_dtype:
            raise TypeError("residual must have the output dtype")
        residual, rm, rn, ldr = _as_rows(residual)
        if rm != M or rn != N:
            raise ValueError("residual must be [..., N] with the rows of a_q")
    if a_scale is not None:
        a_scale = a_scale.to(device=dev, dtype=torch.float32).contiguous()
    if w_scale is not None:
        w_scale = w_scale.to(device=dev, dtype=torch.float32).contiguous()
    with torch.cuda.device(dev), _Timed("gemm_i8", 2.0 * M * N * K, detail=(M, N, K, out.element_size())):
        _lib.check(lib.samq_gemm_i8(
            _ptr(a2), lda, _ptr(w2), ldw, M, N, K,
            _ptr(a_scale), a_gran, _ptr(w_scale), w_gran, int(group_size or 0),
            _ptr(bias), _ptr(residual), ldr, activation,
            _ptr(out), _OUT_CODE[out_dtype], N, _ptr(status_word(dev)), _stream()))
    return out.view(*lead, N)


def gemm_stall_selftest(a_q: torch.Tensor, w_q: torch.Tensor, skip_kblock: int = 0, wait_limit_cycles: int = 2_000_000) -> torch.Tensor:
    """Run ``samq_gemm_i8_stall_selftest``: the raw-int32 GEMM with one operand stage that the
    producer never fills, so that a bounded wait inside the kernel runs out.  The kernel returns on
    its own and raises the device status word (``check_status`` then raises); the returned tensor
    is incomplete."""
    _require_cuda(a_q, "a_q")
    lib = _lib.load()
    M, K = a_q.shape
    N = w_q.shape[0]
    out = torch.zeros((M, N), dtype=torch.int32, device=a_q.device)
    with torch.cuda.device(a_q.device):
        _lib.check(lib.samq_gemm_i8_stall_selftest(_ptr(a_q), a_q.stride(0), _ptr(w_q), w_q.stride(0), M, N, K, _ptr(out), N,
                                                   int(skip_kblock), int(wait_limit_cycles), _ptr(status_word(a_q.device)), _stream()))
    return out


def rel_pos_table(rel_pos_h: torch.Tensor, rel_pos_w: torch.Tensor, dtype, device) -> torch.Tensor:
    """The rows of ``rel_pos_h`` followed by those of ``rel_pos_w`` as one [J, d] matrix of
    ``dtype`` (J rounded up to a multiple of 8, zero rows at the end)."""
    rows = rel_pos_h.shape[0] + rel_pos_w.shape[0]
    J = (rows + 7) // 8 * 8
    tab = torch.zeros((J, rel_pos_h.shape[1]), dtype=dtype, device=device)
    tab[:rel_pos_h.shape[0]] = rel_pos_h.detach().to(device=device, dtype=dtype)
    tab[rel_pos_h.shape[0]:rows] = rel_pos_w.detach().to(device=device, dtype=dtype)
    return tab


def rel_pos_products(qkv: torch.Tensor, num_heads: int, table: torch.Tensor) -> torch.Tensor:
    """rel_all[head, token, j] = q[token, head, :] . table[j, :]: one batched tensor-core GEMM on
    strided views of ``qkv`` [tokens, 3C], no copy of q."""
    tokens, three_c = qkv.shape
    d = three_c // 3 // num_heads
    q_heads = qkv.view(tokens, 3, num_heads, d)[:, 0].permute(1, 0, 2)          # [heads, tokens, d], strides (d, 3C, 1)
    return torch.matmul(q_heads, table.t())                                      # [heads, tokens, J]


def attn_window_prep(qkv: torch.Tensor, H: int, W: int, num_heads: int, rel_pos_h: torch.Tensor,
                     rel_pos_w: torch.Tensor, scale: float, width: int, table: Optional[torch.Tensor] = None):
    """Augmented attention inputs for windows (``samq_attn_window_prep``): from ``qkv``
    [tokens, 3C] returns ``(q_aug, k_aug)``, each [tokens, heads, width].  ``table`` is an
    optional cached ``rel_pos_table`` of the two tables."""
    _require_cuda(qkv, "qkv")
    lib = _lib.load()
    tokens, three_c = qkv.shape
    d = three_c // 3 // num_heads
    if not qkv.is_contiguous():
        raise ValueError("qkv must be contiguous")
    if rel_pos_h.shape != (2 * H - 1, d) or rel_pos_w.shape != (2 * W - 1, d):
        raise ValueError("relative position tables must be [2H-1, d] and [2W-1, d]")
    if table is None:
        table = rel_pos_table(rel_pos_h, rel_pos_w, qkv.dtype, qkv.device)
    rel_all = rel_pos_products(qkv, num_heads, table)
    if not rel_all.is_contiguous():
        rel_all = rel_all.contiguous()
    qa = torch.empty((tokens, num_heads, width), dtype=qkv.dtype, device=qkv.device)
    ka = torch.empty((tokens, num_heads, width), dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(qkv.device), _Timed("attn_prep", tokens * num_heads * (2 * d + 2 * width) * qkv.element_size()):
        _lib.check(lib.samq_attn_window_prep(_ptr(qkv), _ptr(rel_all), _DTYPE_CODE[qkv.dtype], tokens, rel_all.shape[-1],
                                             H, W, num_heads, d, float(scale), width, _ptr(qa), _ptr(ka), _stream()))
    return qa, ka


def attn_rel_bias(qkv: torch.Tensor, images: int, H: int, W: int, num_heads: int, rel_pos_h: torch.Tensor,
                  rel_pos_w: torch.Tensor, table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Explicit relative-position bias [images, heads, H*W, H*W] for global attention
    (``samq_attn_rel_bias``) from ``qkv`` [images*H*W, 3C]."""
    _require_cuda(qkv, "qkv")
    lib = _lib.load()
    tokens, three_c = qkv.shape
    L = H * W
    if tokens != images * L or not qkv.is_contiguous():
        raise ValueError("qkv must be a contiguous [images*H*W, 3C] tensor")
    if table is None:
        table = rel_pos_table(rel_pos_h, rel_pos_w, qkv.dtype, qkv.device)
    rel_all = rel_pos_products(qkv, num_heads, table)
    if not rel_all.is_contiguous():
        rel_all = rel_all.contiguous()
    bias = torch.empty((images, num_heads, L, L), dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(qkv.device), _Timed("attn_bias", bias.numel() * bias.element_size()):
        _lib.check(lib.samq_attn_rel_bias(_ptr(rel_all), _DTYPE_CODE[qkv.dtype], images, rel_all.shape[-1], H, W, num_heads,
                                          _ptr(bias), _stream()))
    return bias


def attn_global_supported(H: int, W: int, head_dim: int, dtype) -> bool:
    """Shapes ``samq_attn_global`` is built for: images of H x 64 tokens or windows up to 16 x 16."""
    shape_ok = (W == 64 and (H * W) % 128 == 0) or (W <= 16 and H <= 16)
    return shape_ok and head_dim in (64, 80) and dtype in (torch.float16, torch.bfloat16)


def attn_global(qkv: torch.Tensor, units: int, H: int, W: int, num_heads: int, rel_pos_h: torch.Tensor,
                rel_pos_w: torch.Tensor, scale: float, table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention with the decomposed relative-position bias on the tensor cores (``samq_attn_global``):
    ``qkv`` [units*H*W, 3C] -> [units*H*W, C], heads side by side; a unit is an image (W = 64) or a
    window (H, W <= 16).  Scores and bias stay on chip."""
    _require_cuda(qkv, "qkv")
    lib = _lib.load()
    tokens, three_c = qkv.shape
    C = three_c // 3
    d = C // num_heads
    L = H * W
    if tokens != units * L or not qkv.is_contiguous():
        raise ValueError("qkv must be a contiguous [units*H*W, 3C] tensor")
    if rel_pos_h.shape != (2 * H - 1, d) or rel_pos_w.shape != (2 * W - 1, d):
        raise ValueError("relative position tables must be [2H-1, d] and [2W-1, d]")
    if table is None:
        table = rel_pos_table(rel_pos_h, rel_pos_w, qkv.dtype, qkv.device)
    rel_all = rel_pos_products(qkv, num_heads, table)
    if not rel_all.is_contiguous():
        rel_all = rel_all.contiguous()
    out = torch.empty((tokens, C), dtype=qkv.dtype, device=qkv.device)
    esz = qkv.element_size()
    with torch.cuda.device(qkv.device):
        with _Timed("attn_global", 4 * tokens * C * esz):
            _lib.check(lib.samq_attn_global(_ptr(qkv), None, _ptr(rel_all), _DTYPE_CODE[qkv.dtype], units, rel_all.shape[-1],
                                            H, W, num_heads, d, float(scale), _ptr(out), _ptr(status_word(qkv.device)), _stream()))
    return out


def attn_window14_supported(H: int, W: int, head_dim: int, dtype) -> bool:
    """Shapes ``samq_attn_window14`` is built for: SAM's 14 x 14 windows, head width 64 or 80."""
    return H == 14 and W == 14 and head_dim in (64, 80) and dtype in (torch.float16, torch.bfloat16)


def attn_window14(qkv: torch.Tensor, windows: int, num_heads: int, rel_pos_h: torch.Tensor, rel_pos_w: torch.Tensor,
                  scale: float, table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of 14 x 14 windows with the decomposed relative-position bias in one tensor-core
    kernel (``samq_attn_window14``): ``qkv`` [windows*196, 3C] -> [windows*196, C], same dtype.
    ``table`` is an optional cached ``rel_pos_table`` of the two [27, d] tables (56 rows)."""
    _require_cuda(qkv, "qkv")
    lib = _lib.load()
    tokens, three_c = qkv.shape
    C = three_c // 3
    d = C // num_heads
    if tokens != windows * 196 or not qkv.is_contiguous():
        raise ValueError("qkv must be a contiguous [windows*196, 3C] tensor")
    if rel_pos_h.shape != (27, d) or rel_pos_w.shape != (27, d):
        raise ValueError("relative position tables must be [27, d]")
    if table is None:
        table = rel_pos_table(rel_pos_h, rel_pos_w, qkv.dtype, qkv.device)
    out = torch.empty((tokens, C), dtype=qkv.dtype, device=qkv.device)
    esz = qkv.element_size()
    with torch.cuda.device(qkv.device), _Timed("attn_window14", 4 * tokens * C * esz):
        _lib.check(lib.samq_attn_window14(_ptr(qkv), _ptr(table), table.shape[0], _DTYPE_CODE[qkv.dtype], windows, num_heads, d,
                                          float(scale), _ptr(out), _ptr(status_word(qkv.device)), _stream()))
    return out


def attn_windowed_supported(H: int, W: int, head_dim: int) -> bool:
    """Shapes ``samq_attn_windowed`` has a variant for."""
    L, J = H * W, 2 * H - 1 + 2 * W - 1
    return (L <= 16 and J <= 16 and head_dim in (16, 32, 64)) or (L <= 208 and J <= 56 and head_dim in (64, 80))


def attn_windowed(qkv: torch.Tensor, windows: int, H: int, W: int, num_heads: int, rel_pos_h: torch.Tensor,
                  rel_pos_w: torch.Tensor, scale: float, table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Windowed attention with decomposed relative position bias in one kernel
    (``samq_attn_windowed``): ``qkv`` [windows*H*W, 3C] -> [windows*H*W, C], same dtype.
    ``table`` is an optional cached ``rel_pos_table`` of the two tables."""
    _require_cuda(qkv, "qkv")
    lib = _lib.load()
    tokens, three_c = qkv.shape
    C = three_c // 3
    d = C // num_heads
    if tokens != windows * H * W or not qkv.is_contiguous():
        raise ValueError("qkv must be a contiguous [windows*H*W, 3C] tensor")
    if rel_pos_h.shape != (2 * H - 1, d) or rel_pos_w.shape != (2 * W - 1, d):
        raise ValueError("relative position tables must be [2H-1, d] and [2W-1, d]")
    if table is None:
        table = rel_pos_table(rel_pos_h, rel_pos_w, qkv.dtype, qkv.device)
    out = torch.empty((tokens, C), dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(qkv.device), _Timed("attn_window", tokens * 4 * C * qkv.element_size()):
        _lib.check(lib.samq_attn_windowed(_ptr(qkv), _DTYPE_CODE[qkv.dtype], windows, H, W, num_heads, d,
                                          _ptr(table), table.shape[0], float(scale), _ptr(out), _stream()))
    return out
