"""CPU oracle for the W8A8 quantized-linear path — TEST INFRASTRUCTURE, NOT PRODUCT.

A numpy restatement of the arithmetic of hchautran/SAM_Quantization's quantize -> dequantize
path.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import it; the
package ``sam_quantization_b200`` never does.  Each function cites the reference lines it
follows.  Parity is pinned: tests/test_oracle_golden.py checks every function here against
tests/golden/*.npz, which tests/golden/make_golden.py produced by running the reference's own
Python functions (the one third-party kernel it calls, Dao-AILab fast_hadamard_transform, is
absent from the reference checkout; for it the oracle is the reference's own pure-torch
``matmul_hadU`` and that boundary is documented as toleranced).

dtype handling: tensors are numpy float32 arrays that hold values representable in the
emulated dtype ("f16", "bf16" or "f32"); ``rnd`` rounds to that dtype with round-to-nearest-even
exactly as torch does after computing each elementwise op in fp32.
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------------
# dtype emulation
# ----------------------------------------------------------------------------------------

def rnd(x, dtype: str):
    """Round fp32/fp64 values to ``dtype`` (RNE) and return them widened to float32."""
    x = np.asarray(x)
    if dtype == "f32":
        return x.astype(np.float32)
    if dtype == "f16":
        return x.astype(np.float32).astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        f = np.ascontiguousarray(x.astype(np.float32))
        u = f.view(np.uint32).astype(np.uint64)
        lsb = (u >> 16) & 1
        r = ((u + 0x7FFF + lsb) >> 16) << 16
        out = r.astype(np.uint32).view(np.float32).reshape(f.shape)
        nan = np.isnan(f)
        if nan.any():
            out = np.where(nan, f, out)
        return out
    raise ValueError(dtype)


def _div(a, b, dtype):
    """a / b computed in fp32 and rounded once to dtype (torch's half/bfloat16 opmath)."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        return rnd(np.asarray(a, np.float32) / np.asarray(b, np.float32), dtype)


# ----------------------------------------------------------------------------------------
# absmax quantizers: RTN_quantization/per_tensor_channel_group.py
# ----------------------------------------------------------------------------------------

def _scale_from_absmax(absmax, dtype, n_bits=8):
    """``scales.clamp_(min=1e-5).div_(q_max)`` in the tensor dtype (:10,:19,:59,:70)."""
    q_max = np.float32(2 ** (n_bits - 1) - 1)
    floor = rnd(np.float32(1e-5), dtype)
    return _div(np.maximum(np.asarray(absmax, np.float32), floor), q_max, dtype)


def quantize_rows(x, dtype="f16", n_bits=8):
    """per_token (:53-61) == per_channel (:5-12): one scale per last-dim row.

    Returns (q, scale, fq): q = round(x / s) as float32 integers (NOT saturated — the reference
    never clamps), scale [..., 1] and the fake-quantized tensor q * s, all in ``dtype``.
    """
    x = rnd(x, dtype)
    absmax = np.abs(x).max(axis=-1, keepdims=True)
    s = _scale_from_absmax(absmax, dtype, n_bits)
    q = np.rint(_div(x, s, dtype)).astype(np.float32)          # .div_().round_() : RNE twice
    fq = rnd(q * s, dtype)                                     # .mul_(scales)
    return q, s, fq


def quantize_tensor(x, dtype="f16", n_bits=8):
    """per_tensor for weights (:14-21) and activations (:64-72): one scalar scale."""
    x = rnd(x, dtype)
    s = _scale_from_absmax(np.abs(x).max() if x.size else np.float32(0), dtype, n_bits)
    q = np.rint(_div(x, s, dtype)).astype(np.float32)
    fq = rnd(q * s, dtype)
    return q, np.asarray(s, np.float32).reshape(1), fq


def quantize_groups(x, group_size, dtype="f16", n_bits=8):
    """per_group weights (:23-50) and per_group_token activations (:74-93): the last dim is
    cut into groups of ``group_size`` and each group is a row of ``quantize_rows``."""
    x = np.asarray(x)
    K = x.shape[-1]
    assert isinstance(group_size, int), "group_size must be an integer"
    assert K % group_size == 0
    xg = x.reshape(x.shape[:-1] + (K // group_size, group_size))
    q, s, fq = quantize_rows(xg, dtype, n_bits)
    return q.reshape(x.shape), s.reshape(x.shape[:-1] + (K // group_size,)), fq.reshape(x.shape)


def quantize(x, granularity, dtype="f16", group_size=None, n_bits=8):
    """Dispatch on the reference's strings; returns (q, scale, fq) with scale squeezed to
    [...] (rows), [1] (tensor) or [..., K/g] (groups)."""
    if granularity in ("per_token", "per_channel"):
        q, s, fq = quantize_rows(x, dtype, n_bits)
        return q, s[..., 0], fq
    if granularity == "per_tensor":
        return quantize_tensor(x, dtype, n_bits)
    if granularity in ("per_group_token", "per_group"):
        return quantize_groups(x, group_size, dtype, n_bits)
    raise ValueError(f"Invalid quantization granularity: {granularity}")


def saturate_codes(q):
    """int8 codes as the CUDA path stores them: q clamped to [-127, 127].  The clamp only acts
    on rows whose fp16 scale is subnormal (row absmax below about 7.8e-3), where the
    reference's unclamped quotient can exceed 127."""
    return np.clip(q, -127, 127).astype(np.int8)


# ----------------------------------------------------------------------------------------
# integer GEMM and the W8A8 linear layer
# ----------------------------------------------------------------------------------------

def int32_accumulators(qa, qw):
    """acc[m, n] = sum_k qa[m, k] * qw[n, k], exact.  The reference never forms this tensor; it
    is defined by stopping ``W8A8Linear.forward`` (:157-162) before dequantization.  float64
    BLAS is exact here: |acc| <= 127^2 * K < 2^53."""
    acc = np.asarray(qa, np.float64) @ np.asarray(qw, np.float64).T
    return acc.astype(np.int64).astype(np.int32)


def int32_group_accumulators(qa, qw, group_size):
    """Per-group partial sums [M, N, K/g] for grouped scales."""
    M, K = qa.shape
    N = qw.shape[0]
    G = K // group_size
    a = np.asarray(qa, np.float64).reshape(M, G, group_size)
    w = np.asarray(qw, np.float64).reshape(N, G, group_size)
    return np.einsum("mgk,ngk->mng", a, w).astype(np.int64).astype(np.int32)


def gelu_erf(x):
    """torch.nn.GELU() default (erf form), fp64 inside."""
    from math import sqrt
    try:
        from scipy.special import erf
    except Exception:                                           # pragma: no cover
        erf = np.vectorize(__import__("math").erf)
    x64 = np.asarray(x, np.float64)
    return (0.5 * x64 * (1.0 + erf(x64 / sqrt(2.0)))).astype(np.float32)


def dequant_epilogue(acc, a_scale, w_scale, bias=None, activation=None, residual=None, out_dtype="f16"):
    """What the CUDA epilogue computes: act(float(acc) * a_s[m] * w_s[n] + bias[n]) + residual,
    fp32 arithmetic, one rounding to out_dtype.  (The reference's own ``sym_dequant`` forms the
    product in fp16, quant/qgemm/kernels/quant.cu:79-80, which overflows past 65504.)"""
    y = np.asarray(acc, np.float32)
    if a_scale is not None:
        y = y * np.asarray(a_scale, np.float32).reshape(-1, 1) if np.size(a_scale) > 1 else y * np.float32(np.asarray(a_scale).reshape(-1)[0])
    if w_scale is not None:
        y = y * np.asarray(w_scale, np.float32).reshape(1, -1) if np.size(w_scale) > 1 else y * np.float32(np.asarray(w_scale).reshape(-1)[0])
    if bias is not None:
        y = y + np.asarray(bias, np.float32).reshape(1, -1)
    if activation == "gelu":
        y = gelu_erf(y)
    if residual is not None:
        y = y + np.asarray(residual, np.float32)
    return rnd(y, out_dtype)


def w8a8_linear_reference(x, w, bias, dtype="f16", weight_quant="per_channel", act_quant="per_token",
                          group_size=None, quantize_output=False):
    """``W8A8Linear.from_float(lin, 8, weight_quant, act_quant, quantize_output, group_size)(x)``
    (:157-196): float GEMM of the fake-quantized operands with fp32 accumulation, bias added in
    fp32, rounded to dtype; then the activation quantizer again if ``quantize_output``."""
    _, _, fw = quantize(w, weight_quant, dtype, group_size)
    lead = x.shape[:-1]
    x2 = np.asarray(x).reshape(-1, x.shape[-1])
    _, _, fx = quantize(x2, act_quant, dtype, group_size)
    y = fx.astype(np.float32) @ fw.astype(np.float32).T
    if bias is not None:
        y = y + rnd(bias, dtype).reshape(1, -1)
    y = rnd(y, dtype)
    if quantize_output:
        _, _, y = quantize(y, act_quant, dtype, group_size)
    return y.reshape(lead + (w.shape[0],))


def w8a8_linear_int8(x, w, bias, dtype="f16", weight_quant="per_channel", act_quant="per_token",
                     group_size=None, activation=None, residual=None):
    """The same layer evaluated the way the CUDA path does: int8 codes -> int32 accumulators ->
    fp32 dequant epilogue.  Returns (y, qa, sa, qw, sw, acc) for bit-exact comparisons."""
    qw, sw, _ = quantize(w, weight_quant, dtype, group_size)
    x2 = np.asarray(x).reshape(-1, x.shape[-1])
    qa, sa, _ = quantize(x2, act_quant, dtype, group_size)
    qa8, qw8 = saturate_codes(qa), saturate_codes(qw)
    grouped = weight_quant == "per_group" or act_quant == "per_group_token"
    if not grouped:
        acc = int32_accumulators(qa8, qw8)
        y = dequant_epilogue(acc, sa, sw, bias, activation, residual, dtype)
    else:
        acc = int32_group_accumulators(qa8, qw8, group_size)            # [M, N, G]
        M, N, G = acc.shape
        if act_quant == "per_group_token":
            sa_g = sa.reshape(M, 1, -1)
        elif np.size(sa) == 1:
            sa_g = np.asarray(sa, np.float32).reshape(1, 1, 1)
        else:
            sa_g = np.asarray(sa, np.float32).reshape(-1, 1, 1)
        sw_g = sw.reshape(1, N, -1) if weight_quant == "per_group" else np.broadcast_to(np.asarray(sw, np.float32).reshape(1, -1, 1), (1, N if np.size(sw) > 1 else 1, 1))
        y = (acc.astype(np.float32) * sa_g.astype(np.float32) * sw_g.astype(np.float32)).sum(axis=2, dtype=np.float32)
        if bias is not None:
            y = y + np.asarray(bias, np.float32).reshape(1, -1)
        if activation == "gelu":
            y = gelu_erf(y)
        if residual is not None:
            y = y + np.asarray(residual, np.float32)
        y = rnd(y, dtype)
    return y, qa8, sa, qw8, sw, acc


# ----------------------------------------------------------------------------------------
# SmoothQuant folding: RTN_quantization/Smooth.py:5-43, calibration.py:35-49
# ----------------------------------------------------------------------------------------

def act_scales_running_max(batches):
    """``stat_tensor`` (calibration.py:35-49): per-channel max |x| over all tokens of all
    batches, fp32."""
    cur = None
    for b in batches:
        b = np.abs(np.asarray(b, np.float32).reshape(-1, b.shape[-1])).max(axis=0)
        cur = b if cur is None else np.maximum(cur, b)
    return cur


def smooth_ln_fcs(ln_weight, ln_bias, fc_weights, act_scales, alpha=0.5, dtype="f16"):
    """Returns (scales, new_ln_weight, new_ln_bias, [new_fc_weights]) following Smooth.py:25-43:
    everything is computed in the weights' dtype, op by op."""
    act = rnd(act_scales, dtype)
    w_abs_max = np.stack([np.abs(rnd(w, dtype)).max(axis=0) for w in fc_weights], 0).max(axis=0)
    w_scales = np.maximum(w_abs_max, rnd(np.float32(1e-5), dtype))
    num = rnd(np.power(act.astype(np.float32), np.float32(alpha)), dtype)
    den = rnd(np.power(w_scales.astype(np.float32), np.float32(1 - alpha)), dtype)
    s = np.maximum(_div(num, den, dtype), rnd(np.float32(1e-5), dtype))
    new_w = _div(rnd(ln_weight, dtype), s, dtype)
    new_b = _div(rnd(ln_bias, dtype), s, dtype)
    new_fcs = [rnd(rnd(w, dtype) * s.reshape(1, -1), dtype) for w in fc_weights]
    return s, new_w, new_b, new_fcs


# ----------------------------------------------------------------------------------------
# Hadamard: quarot/hadamard_utils.py
# ----------------------------------------------------------------------------------------

def is_pow2(n):
    return n > 0 and (n & (n - 1)) == 0


def _legendre_is_residue(p):
    res = np.zeros(p, bool)
    for i in range(1, p):
        res[(i * i) % p] = True
    return res


def paley1(p):
    """Hadamard matrix of order p+1 (p prime, p = 3 mod 4) in the normal form the reference's
    table had12 uses (hadamard_utils.py:179-194): first column +1, rest of the first row -1, and
    a circulant core whose row i is the generator shifted right by i, generator[j] = +1 for
    j = 0 and for quadratic non-residues j, -1 for residues."""
    res = _legendre_is_residue(p)
    gen = np.array([1 if (j == 0 or not res[j]) else -1 for j in range(p)], np.float32)
    H = np.ones((p + 1, p + 1), np.float32)
    H[0, 1:] = -1
    for i in range(p):
        H[i + 1, 1:] = np.roll(gen, i)
    return H


_HADK_TABLES = {}


def register_hadk(k, table):
    _HADK_TABLES[int(k)] = np.asarray(table, np.float32)


def hadk_table(k):
    if k in _HADK_TABLES:
        return _HADK_TABLES[k]
    if k == 12:
        return paley1(11)
    if k == 20:
        return paley1(19)
    raise KeyError(f"no Hadamard table of order {k} registered in the oracle")


def get_hadK(n):
    """Divisor search order of hadamard_utils.py:6-56.  Returns (hadK or None, K)."""
    for k in (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12):
        if n % k == 0:
            assert is_pow2(n // k)
            return hadk_table(k), k
    assert is_pow2(n)
    return None, 1


def matmul_hadU(x, hadk=None, k=None, np_dtype=np.float32):
    """hadamard_utils.py:59-80 on the last dim: butterflies with strides 1, 2, 4, ... over each
    contiguous chunk of n/K, then hadK mixes the K chunks, then a division by fp32 sqrt(n).
    Arithmetic in ``np_dtype`` (the reference runs in the input's dtype: fp32 for the
    ``fp32_had`` path, fp64 for ``random_hadamard_matrix``)."""
    x = np.asarray(x, np_dtype)
    n = x.shape[-1]
    if k is None:
        hadk, k = get_hadK(n)
    y = x.reshape(-1, n).copy()
    chunk = n // k
    stride = 1
    while stride < chunk:
        v = y.reshape(-1, n // (2 * stride), 2, stride)
        a = v[:, :, 0, :].copy()
        b = v[:, :, 1, :].copy()
        v[:, :, 0, :] = a + b
        v[:, :, 1, :] = a - b
        stride *= 2
    if k > 1:
        y = np.einsum("kj,bjc->bkc", np.asarray(hadk, np_dtype), y.reshape(-1, k, chunk)).reshape(-1, n)
    root = np.sqrt(np.float32(n)).astype(np_dtype)
    return (y / root).reshape(x.shape).astype(np_dtype)


def hadamard_full_online(x, dtype="f16", signs=None):
    """``ActQuantWrapper.forward`` with online_full_had and fp32_had=True
    (quarot/utils.py:257-259): transform in fp32 on the up-cast input, one rounding to dtype.
    ``signs`` folds the diagonal of ``random_hadamard_matrix`` in first (x @ Q == hadU(x * signs),
    hadamard_utils.py:86-94)."""
    x = rnd(x, dtype)
    if signs is not None:
        x = x * np.asarray(signs, np.float32)
    return rnd(matmul_hadU(x, np_dtype=np.float32), dtype)


def hadamard_partial_online(x, had_dim, dtype="f16"):
    """online_partial_had (quarot/utils.py:263-289): the last dim C is viewed as
    [heads = C / had_dim, had_dim] and the size-``heads`` transform runs across heads."""
    x = rnd(x, dtype)
    C = x.shape[-1]
    heads = C // had_dim
    v = x.reshape(-1, heads, had_dim).transpose(0, 2, 1)          # [..., had_dim, heads]
    t = matmul_hadU(v, np_dtype=np.float32)                       # scaled by 1/sqrt(heads)
    return rnd(t.transpose(0, 2, 1).reshape(x.shape), dtype)


def random_hadamard_signs(size, seed):
    """The +-1 diagonal drawn by ``random_hadamard_matrix`` (hadamard_utils.py:86-91) needs
    torch's generator; tests pass the signs in from a fixture or from torch directly."""
    import torch
    torch.manual_seed(seed)
    q = torch.randint(low=0, high=2, size=(size,)).to(torch.float64)
    return (q * 2 - 1).numpy()


def random_hadamard_matrix(size, seed, signs=None):
    """Q = hadU(diag(signs)) in fp64 (hadamard_utils.py:86-94)."""
    s = random_hadamard_signs(size, seed) if signs is None else np.asarray(signs, np.float64)
    return matmul_hadU(np.diag(s), np_dtype=np.float64)


# ----------------------------------------------------------------------------------------
# The packed int4 path of the native extension: quant/qgemm/kernels/quant.cu, bindings.cpp
# ----------------------------------------------------------------------------------------

def sym_quant_int4(x, scale):
    """``sym_quant`` (quant.cu:11-46): codes = clamp(round_half_even(fp16(x / scale[row])), -8, 7)
    from fp16 ``x`` [rows, cols] and fp16 ``scale`` [rows]; returns (codes int8 [rows, cols],
    packed uint8 [rows, ceil(cols / 2)]) with element 2j in the low nibble of byte j.  The fp16
    quotient formed in fp32 and rounded once equals the correctly rounded half division."""
    x = rnd(x, "f16")
    s = rnd(np.asarray(scale, np.float32).reshape(-1, 1), "f16")
    q = np.clip(np.rint(_div(x, s, "f16")), -8, 7).astype(np.int8)
    return q, pack_int4(q)


def pack_int4(codes):
    codes = np.asarray(codes, np.int8)
    rows, cols = codes.shape
    padded = np.zeros((rows, (cols + 1) // 2 * 2), np.uint8)
    padded[:, :cols] = codes.astype(np.uint8) & 0xF
    return (padded[:, 0::2] | (padded[:, 1::2] << 4)).astype(np.uint8)


def unpack_int4(packed, cols):
    packed = np.asarray(packed, np.uint8)
    out = np.empty((packed.shape[0], packed.shape[1] * 2), np.int8)
    out[:, 0::2] = ((packed & 0xF).astype(np.int8) ^ 8) - 8
    out[:, 1::2] = ((packed >> 4).astype(np.int8) ^ 8) - 8
    return out[:, :cols]


def matmul_int4(a_packed, b_packed):
    """``matmul`` (bindings.cpp:7-26): int32 [M, N] = A [M, K] x B [N, K]^T from the packed operands."""
    K = 2 * np.asarray(a_packed).shape[1]
    return int32_accumulators(unpack_int4(a_packed, K), unpack_int4(b_packed, K))


def sym_dequant_int32(q, scale_row, scale_col):
    """``sym_dequant`` (quant.cu:64-80): (scale_row[m] * scale_col[n]) * half(q[m, n]), each product
    rounded to fp16; int -> half rounds to nearest even and overflows to inf beyond 65504."""
    sr = rnd(np.asarray(scale_row, np.float32).reshape(-1, 1), "f16")
    sc = rnd(np.asarray(scale_col, np.float32).reshape(1, -1), "f16")
    with np.errstate(over="ignore"):
        xe = np.asarray(q, np.float64).astype(np.float16).astype(np.float32)
        return rnd(rnd(sr * sc, "f16") * xe, "f16")
