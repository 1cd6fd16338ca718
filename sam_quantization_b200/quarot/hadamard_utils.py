"""Hadamard helpers with the interface of quarot/hadamard_utils.py.

``matmul_hadU`` is the offline (weight-side, any dtype incl. fp64) transform written with torch
ops; ``matmul_hadU_cuda`` is the online transform and runs the fused CUDA kernel K1 (fp32
butterflies, one rounding to the input dtype).  The +-1 tables the reference stores as literals
(:179-4218) are generated: had12 and had20 are Paley type-I matrices in the same normal form,
had40 is their Sylvester doubling; tests compare them entry by entry with fixtures taken from
the reference.  The larger tables (28 ... 172) serve LLM widths, none of SAM's, and are not
provided.
"""
from __future__ import annotations

import math

import torch

from .. import ops


def is_pow2(n):
    return (n & (n - 1) == 0) and (n > 0)


def _paley1(p: int) -> torch.Tensor:
    """Order p+1 Hadamard matrix (p prime, p = 3 mod 4): first column +1, rest of row 0 is -1,
    circulant core with generator +1 at 0 and at the quadratic non-residues."""
    residue = [False] * p
    for i in range(1, p):
        residue[(i * i) % p] = True
    gen = torch.tensor([1.0 if (j == 0 or not residue[j]) else -1.0 for j in range(p)])
    H = torch.ones(p + 1, p + 1)
    H[0, 1:] = -1
    for i in range(p):
        H[i + 1, 1:] = torch.roll(gen, i)
    return H


def get_had12():
    return _paley1(11)


def get_had20():
    return _paley1(19)


def get_had40():
    h20 = _paley1(19)
    return torch.cat([torch.cat([h20, h20], 1), torch.cat([h20, -h20], 1)], 0)


_TABLES = ((40, get_had40), (20, get_had20), (12, get_had12))
_UNSUPPORTED = (172, 156, 140, 108, 60, 52, 36, 28)


def get_hadK(n, transpose=False):
    """(hadK, K) with the divisor search order of quarot/hadamard_utils.py:6-56
    (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12, else a power of two -> (None, 1))."""
    for k in _UNSUPPORTED:
        if n % k == 0:
            raise NotImplementedError(f"the order-{k} Hadamard table (n={n}) is not provided; SAM widths need 12, 20 and 40 only")
    for k, fn in _TABLES:
        if n % k == 0:
            assert is_pow2(n // k)
            h = fn()
            return (h.T if transpose else h), k
    assert is_pow2(n)
    return None, 1


def matmul_hadU(X, transpose=False):
    """X @ H_n / sqrt(n) over the last dim, any device and dtype, the arithmetic of
    quarot/hadamard_utils.py:59-80: stride-1,2,4,... butterflies over chunks of n/K, then the
    K x K table across chunks, then a division by fp32 sqrt(n)."""
    n = X.shape[-1]
    hadK, K = get_hadK(n, transpose)
    y = X.reshape(-1, n).clone()
    chunk, stride = n // K, 1
    while stride < chunk:
        v = y.view(-1, n // (2 * stride), 2, stride)
        a, b = v[:, :, 0, :].clone(), v[:, :, 1, :].clone()
        v[:, :, 0, :] = a + b
        v[:, :, 1, :] = a - b
        stride *= 2
    if K > 1:
        y = (hadK.view(1, K, K).to(y) @ y.view(-1, K, chunk)).reshape(-1, n)
    return y.view(X.shape) / torch.tensor(n).sqrt()


def matmul_hadUt(X):
    return matmul_hadU(X, transpose=True)


def random_hadamard_matrix(size, device, seed):
    """Q = diag(+-1) H / sqrt(n) in fp64 (quarot/hadamard_utils.py:86-94), same generator calls
    so a given seed yields the reference's matrix."""
    if seed is not None:
        torch.manual_seed(seed)
        torch.cuda.manual_seed_all(seed)
    signs = torch.randint(low=0, high=2, size=(size,)).to(torch.float64) * 2 - 1
    return matmul_hadU(torch.diag(signs)).to(device)


def random_hadamard_signs(size, seed):
    """The diagonal of ``random_hadamard_matrix``: x @ Q == hadU(x * signs)."""
    if seed is not None:
        torch.manual_seed(seed)
        torch.cuda.manual_seed_all(seed)
    return (torch.randint(low=0, high=2, size=(size,)) * 2 - 1).to(torch.int8)


def matmul_hadU_cuda(X, hadK, K):
    """Online transform of quarot/hadamard_utils.py:96-105 on the GPU: one fused kernel (K1 with
    only the transformed output requested) instead of the fast_hadamard_transform library call
    plus a K x K matmul."""
    spec = ops.Hadamard("full", had_k=int(K), hadk=None if K == 1 else hadK.to(X.device))
    x = X if X.dtype in (torch.float16, torch.bfloat16, torch.float32) else X.float()
    out = ops.quantize(x.contiguous(), ops.GRAN_ROW, hadamard=spec, codes=False, transformed=True)["tx"]
    return out.to(X.dtype).reshape(X.shape)


def hadamard_transform_last_dim(x, scale_len=None):
    """Power-of-two transform over the last dim scaled by 1/sqrt(len): the role of
    ``fast_hadamard_transform.hadamard_transform(x, scale)`` at
    quarot/hadamard_utils.py:140,148 and quarot/utils.py:275."""
    n = x.shape[-1]
    assert is_pow2(n), "Hadamard dimension must be a power of 2!"
    xf = x if x.dtype in (torch.float16, torch.bfloat16, torch.float32) else x.float()
    out = ops.quantize(xf.contiguous(), ops.GRAN_ROW, hadamard=ops.Hadamard("full"), codes=False, transformed=True)["tx"]
    return out.to(x.dtype)


def apply_exact_had_to_linear(module, had_dim=-1, output=False):
    """quarot/hadamard_utils.py:112-166: fold a Hadamard into a Linear's weight, on the input
    side (``output=False``, whole in_features) or on the output side per head of width
    ``had_dim`` (weight rows and bias)."""
    assert isinstance(module, torch.nn.Linear)
    in_features, out_features = module.in_features, module.out_features
    if had_dim != -1:
        assert is_pow2(had_dim), "Hadamard dimension must be a power of 2!"
    W_ = module.weight.data
    dtype, dev = W_.dtype, W_.device
    W_ = W_.float().cuda()
    if had_dim == -1:
        if output:
            had_K, K = get_hadK(out_features)
            W_ = matmul_hadU_cuda(W_.t().contiguous(), had_K, K).t()
            if module.bias is not None:
                raise ValueError("Bias has not been implemented")
        else:
            had_K, K = get_hadK(in_features)
            W_ = matmul_hadU_cuda(W_, had_K, K)
    else:
        if not output:
            raise NotImplementedError("Not implemented (or tested) yet!")
        Wt = W_.t().contiguous()
        shape_t = Wt.shape
        Wt = hadamard_transform_last_dim(Wt.reshape(-1, shape_t[-1] // had_dim, had_dim)).reshape(shape_t)
        W_ = Wt.t()
        if module.bias is not None:
            b = module.bias.data.float().cuda().reshape(-1, had_dim)
            module.bias.data = hadamard_transform_last_dim(b).reshape(module.bias.data.shape).to(device=dev, dtype=dtype)
    module.weight.data = W_.contiguous().to(device=dev, dtype=dtype)
