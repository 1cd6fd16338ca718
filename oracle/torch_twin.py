"""Float / fake-quant twins of the quantized layers — TEST INFRASTRUCTURE, NOT PRODUCT.

Torch restatements of the reference's modules, used to drive the float twin of the encoder
through the reference's quantize -> dequantize arithmetic on the same weights:

* ``RefW8A8Linear``      RTN_quantization/per_tensor_channel_group.py:95-199
* ``RefActQuantWrapper`` quarot/utils.py:202-298 (Hadamard through the pure-torch ``matmul_hadU``,
                         the designated stand-in for the absent fast_hadamard_transform kernel)

They run wherever their tensors live (CPU in the no-GPU tests, cuda in the GPU tests) with plain
torch ops, op for op in the tensor's dtype like the reference.  tests/test_oracle_golden.py pins
``RefW8A8Linear`` to outputs of the reference's own class (tests/golden/w8a8_linear.npz).
Only tests/, __graft_entry__.smoke() and bench.py's reference leg may import this file.
"""
from __future__ import annotations

import math

import torch
from torch import nn


@torch.no_grad()
def fq_rows(t, n_bits=8):
    """quantize_*_per_token/per_channel_absmax (:5-12,:53-61), in place."""
    scales = t.abs().max(dim=-1, keepdim=True)[0]
    scales.clamp_(min=1e-5).div_(2 ** (n_bits - 1) - 1)
    t.div_(scales).round_().mul_(scales)
    return t


@torch.no_grad()
def fq_tensor(t, n_bits=8):
    """quantize_*_per_tensor_absmax (:14-21,:64-72), in place."""
    scales = t.abs().max()
    scales.clamp_(min=1e-5).div_(2 ** (n_bits - 1) - 1)
    t.div_(scales).round_().mul_(scales)
    return t


@torch.no_grad()
def fq_groups(t, group_size, n_bits=8):
    """per-group variants (:23-50,:74-93): groups of the last dim are rows."""
    shape = t.shape
    assert shape[-1] % group_size == 0
    fq_rows(t.view(-1, group_size), n_bits)
    return t.view(shape)


def fake_quant(t, granularity, group_size=None, n_bits=8):
    if granularity in ("per_token", "per_channel"):
        return fq_rows(t, n_bits)
    if granularity == "per_tensor":
        return fq_tensor(t, n_bits)
    if granularity in ("per_group_token", "per_group"):
        return fq_groups(t, group_size, n_bits)
    raise ValueError(granularity)


class RefW8A8Linear(nn.Module):
    def __init__(self, weight, bias, act_quant="per_token", quantize_output=False, group_size=None, n_bits=8):
        super().__init__()
        self.weight, self.bias = weight, bias
        self.act_quant_name, self.quantize_output = act_quant, quantize_output
        self.group_size, self.n_bits = group_size, n_bits

    @staticmethod
    def from_float(module, n_bits, weight_quant="per_channel", act_quant="per_token", quantize_output=False, group_size=None):
        assert isinstance(module, nn.Linear)
        w = fake_quant(module.weight.data, weight_quant, group_size, n_bits)
        return RefW8A8Linear(w, None if module.bias is None else module.bias.data, act_quant, quantize_output, group_size, n_bits)

    @torch.no_grad()
    def forward(self, x):
        q_x = fake_quant(x.contiguous().clone(), self.act_quant_name, self.group_size, self.n_bits)
        y = torch.nn.functional.linear(q_x, self.weight, self.bias)
        if self.quantize_output:
            y = fake_quant(y, self.act_quant_name, self.group_size, self.n_bits)
        return y


def is_pow2(n):
    return n > 0 and (n & (n - 1)) == 0


def matmul_hadU(X, hadK=None, K=1):
    """quarot/hadamard_utils.py:59-80 with the table passed in."""
    n = X.shape[-1]
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


class RefActQuantWrapper(nn.Module):
    """quarot/utils.py:202-298 with ``fp32_had`` semantics for the transforms."""

    def __init__(self, module, act_quant="per_token", weight_quant="per_channel", n_bit=8, group_size=None):
        super().__init__()
        self.module = module
        self.act_quant_name, self.group_size, self.n_bits = act_quant, group_size, n_bit
        self.had_K, self.K, self.had_dim = None, 1, 0
        self.online_full_had = self.online_partial_had = False
        self.quantize_input = self.quantize_output = False
        # optional: the online x @ Q of quarot/model_utils.py:146-152 evaluated as
        # hadU(x * signs) in fp32 (Q = diag(signs) H / sqrt(n), hadamard_utils.py:86-94) and rounded once
        self.pre_signs, self.pre_hadK, self.pre_K = None, None, 1
        # optional: evaluate the float linear in another dtype (fp64) and round once to the tensor dtype: the same
        # arithmetic as the reference up to the summation order / accumulator width of its float GEMM
        self.linear_dtype = None
        if weight_quant is not None:                      # None: transforms only (change-of-basis checks)
            fake_quant(module.weight.data, weight_quant, group_size, n_bit)

    @torch.no_grad()
    def forward(self, x):
        dt = x.dtype
        if self.pre_signs is not None:
            x = matmul_hadU(x.float() * self.pre_signs.to(x.device).float(), self.pre_hadK, self.pre_K).to(dt)
        if self.online_full_had:
            x = matmul_hadU(x.float(), self.had_K, self.K).to(dt)
        elif self.online_partial_had:
            shape = x.shape
            heads = shape[-1] // self.had_dim
            v = x.float().reshape(-1, heads, self.had_dim).transpose(1, 2)
            if self.K == 1:
                v = matmul_hadU(v.contiguous())
            else:
                v = (self.had_K.to(v) @ v.transpose(1, 2)).transpose(1, 2) / math.sqrt(heads)
            x = v.transpose(1, 2).reshape(shape).to(dt)
        if self.quantize_input:
            x = fake_quant(x.contiguous().clone(), self.act_quant_name, self.group_size, self.n_bits)
        if self.linear_dtype is None:
            x = self.module(x).to(dt)
        else:
            ld = self.linear_dtype
            x = torch.nn.functional.linear(x.to(ld), self.module.weight.to(ld),
                                           None if self.module.bias is None else self.module.bias.to(ld)).to(dt)
        if self.quantize_output:
            x = fake_quant(x, self.act_quant_name, self.group_size, self.n_bits)
        return x


def replace_linears(module, factory, exclude=()):
    """Swap every nn.Linear below ``module`` for ``factory(linear)`` (walk of
    RTN_quantization/utils.py:33-61)."""
    for name, child in module.named_children():
        if isinstance(child, nn.Linear) and name not in exclude:
            setattr(module, name, factory(child))
        else:
            replace_linears(child, factory, exclude)
    return module


# ----------------------------------------------------------------------------------------
# QuaRot weight rotation of the image encoder, restated with the pure-torch transform above
# ----------------------------------------------------------------------------------------

def exact_had_input_side(lin, hadK=None, K=1):
    """``apply_exact_had_to_linear(lin, had_dim=-1, output=False)`` (quarot/hadamard_utils.py:112-134):
    the weight's input side takes the full transform, computed in fp32 and cast back."""
    W = lin.weight.data
    lin.weight.data = matmul_hadU(W.float(), hadK, K).to(W.dtype)


def exact_had_output_side_per_head(weight, bias, had_dim):
    """``apply_exact_had_to_linear(v, had_dim=head_dim, output=True)`` (quarot/hadamard_utils.py:135-151):
    every group of ``had_dim`` consecutive output features takes the power-of-two transform scaled
    by 1/sqrt(had_dim), weight rows and bias alike; fp32, cast back.  Returns (weight, bias)."""
    Wt = weight.float().t().contiguous()                                   # [in, out]
    shape = Wt.shape
    Wt = matmul_hadU(Wt.reshape(-1, shape[-1] // had_dim, had_dim)).reshape(shape)
    b = matmul_hadU(bias.float().reshape(-1, had_dim)).reshape(bias.shape)
    return Wt.t().contiguous().to(weight.dtype), b.to(bias.dtype)


@torch.no_grad()
def rotate_encoder_weights(model, Q, hidden, heads, hadK_of=None):
    """``rotate_model_sam`` for the image encoder (quarot/rotation_utils.py:137-195): qkv and lin1
    take ``W @ Q`` in fp64; lin2 and proj take the exact transform on their input side; the V
    slice of qkv takes the per-head transform on its output side, bias included.
    ``hadK_of(n) -> (table or None, K)`` supplies the explicit factor for widths that are not a
    power of two."""
    hadK_of = hadK_of or (lambda n: (None, 1))
    Q64 = Q.to(torch.float64)
    blocks = model.image_encoder.blocks
    for blk in blocks:
        for lin in (blk.attn.qkv, blk.mlp.lin1):
            W = lin.weight.data
            lin.weight.data = (W.to(torch.float64) @ Q64.to(W.device)).to(W.dtype)
    for blk in blocks:
        exact_had_input_side(blk.mlp.lin2, *hadK_of(blk.mlp.lin2.in_features))
    head_dim = hidden // heads
    for blk in blocks:
        qkv = blk.attn.qkv
        w, b = exact_had_output_side_per_head(qkv.weight.data[2 * hidden:3 * hidden].clone(),
                                              qkv.bias.data[2 * hidden:3 * hidden].clone(), head_dim)
        qkv.weight.data[2 * hidden:3 * hidden] = w
        qkv.bias.data[2 * hidden:3 * hidden] = b
        exact_had_input_side(blk.attn.proj, *hadK_of(blk.attn.proj.in_features))


def random_hadamard_Q(size, seed):
    """``random_hadamard_matrix`` (quarot/hadamard_utils.py:86-94): (signs, Q) with
    Q = hadU(diag(signs)) in fp64, so that x @ Q == hadU(x * signs)."""
    torch.manual_seed(seed)
    signs = (torch.randint(low=0, high=2, size=(size,)).to(torch.float64) * 2 - 1)
    return signs, matmul_hadU(torch.diag(signs))
