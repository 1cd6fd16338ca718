"""The six absmax quantizers and the W8A8Linear module of the reference, on the CUDA kernels.

Same names, arguments and in-place behaviour as
RTN_quantization/per_tensor_channel_group.py:5-93: each function overwrites its argument with the
fake-quantized tensor (quantize -> dequantize in the tensor's dtype) and returns it.  The
``*_codes`` twins return what the reference never materialises: ``(int8 codes, fp32 scale)``.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from .._lib import ACT_GELU, ACT_NONE, GRAN_GROUP, GRAN_ROW, GRAN_TENSOR


def _fake_quant_(t: torch.Tensor, gran: int, group_size, n_bits: int, weight: bool) -> torch.Tensor:
    if weight:
        fq = ops.quantize_weight(t, gran, group_size, codes=False, fake_quant=True, n_bits=n_bits)["fq"]
    else:
        fq = ops.quantize(t, gran, group_size, codes=False, fake_quant=True, n_bits=n_bits)["fq"]
    t.copy_(fq.view(t.shape))
    return t


@torch.no_grad()
def quantize_weight_per_channel_absmax(w, n_bits=8):
    """per_tensor_channel_group.py:5-12 — one scale per output row, in place."""
    return _fake_quant_(w, GRAN_ROW, None, n_bits, weight=w.dim() == 2)


@torch.no_grad()
def quantize_weight_per_tensor_absmax(w, n_bits=8):
    """per_tensor_channel_group.py:14-21 — one scalar scale, in place."""
    return _fake_quant_(w, GRAN_TENSOR, None, n_bits, weight=w.dim() == 2)


@torch.no_grad()
def quantize_weight_per_group_absmax_input_features(w, group_size, n_bits=8):
    """per_tensor_channel_group.py:23-50 — groups of ``group_size`` along the input features."""
    out_features, in_features = w.shape
    assert in_features % group_size == 0, f"in_features ({in_features}) must be divisible by group_size ({group_size})"
    assert w.dim() == 2
    assert type(group_size) == int, "group_size must be an integer"
    return _fake_quant_(w, GRAN_GROUP, group_size, n_bits, weight=True)


@torch.no_grad()
def quantize_activation_per_token_absmax(t, n_bits=8):
    """per_tensor_channel_group.py:53-61 — one scale per last-dim row, in place."""
    return _fake_quant_(t, GRAN_ROW, None, n_bits, weight=False)


@torch.no_grad()
def quantize_activation_per_tensor_absmax(t, n_bits=8):
    """per_tensor_channel_group.py:64-72 — one scalar scale, in place."""
    return _fake_quant_(t, GRAN_TENSOR, None, n_bits, weight=False)


@torch.no_grad()
def quantize_activation_per_group_absmax_token_dim(t, group_size, n_bits=8):
    """per_tensor_channel_group.py:74-93 — groups of ``group_size`` along the last dim."""
    last_dim = t.shape[-1]
    assert type(group_size) == int, "group_size must be an integer"
    assert last_dim % group_size == 0, f"Last dimension ({last_dim}) must be divisible by group_size ({group_size})"
    return _fake_quant_(t, GRAN_GROUP, group_size, n_bits, weight=False)


# ---- what the int8 GEMM consumes -------------------------------------------------------------

@torch.no_grad()
def quantize_activation_codes(t, act_quant="per_token", group_size=None, n_bits=8, divisor=None, hadamard=None):
    """(int8 codes [..., K], fp32 scale) for "per_token" | "per_tensor" | "per_group_token"."""
    if act_quant not in ops.ACT_GRANULARITY:
        raise ValueError(f"Invalid act_quant: {act_quant}")
    out = ops.quantize(t, ops.ACT_GRANULARITY[act_quant], group_size, divisor=divisor, hadamard=hadamard, n_bits=n_bits)
    return out["q"], out["scale"]


@torch.no_grad()
def quantize_weight_codes(w, weight_quant="per_channel", group_size=None, n_bits=8):
    """(int8 codes [N, K], fp32 scale) for "per_channel" | "per_tensor" | "per_group"."""
    if weight_quant not in ops.WEIGHT_GRANULARITY:
        raise ValueError(f"Invalid weight_quant: {weight_quant}")
    out = ops.quantize_weight(w, ops.WEIGHT_GRANULARITY[weight_quant], group_size, n_bits=n_bits)
    return out["q"], out["scale"]


# ---- the module ------------------------------------------------------------------------------
#
# W8A8Linear — the drop-in module for the reference's class of the same name
# (RTN_quantization/per_tensor_channel_group.py:95-199).
#
# The reference keeps a fake-quantized float weight and runs ``F.linear`` on a fake-quantized
# activation.  This module keeps the int8 weight codes and their scales and runs K1 (dynamic
# activation quantization) followed by K2 (tcgen05 int8 GEMM with the dequant / bias epilogue),
# i.e. the same layer in real integer arithmetic.  ``weight`` is still exposed (dequantized on
# demand, bit-identical to the reference's fake-quantized weight).

class W8A8Linear(nn.Module):
    def __init__(self, in_features, out_features, bias=True, act_quant="per_token",
                 quantize_output=False, group_size=None, n_bit=8):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self.n_bits = n_bit
        if act_quant not in ops.ACT_GRANULARITY:
            raise ValueError(f"Invalid act_quant: {act_quant}")
        self.act_quant_name = act_quant
        self.weight_quant_name = "per_channel"
        self.output_quant_name = act_quant if quantize_output else "None"
        self.quantize_output = bool(quantize_output)
        self.register_buffer("qweight", torch.zeros(out_features, in_features, dtype=torch.int8))
        self.register_buffer("w_scale", torch.ones(out_features, dtype=torch.float32))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16))
        else:
            self.register_buffer("bias", None)
        self.compute_dtype = torch.float16
        # optional transforms folded into the activation quantizer (not part of the reference API)
        self.smooth_divisor = None
        self.hadamard = None

    # callers that know this module may fuse the following GELU / residual add into the GEMM
    supports_fused_epilogue = True

    # -- reference surface ------------------------------------------------------------------
    @property
    def weight(self) -> torch.Tensor:
        """Dequantized weight, ``codes * scale`` rounded to the layer dtype — the tensor the
        reference stores after ``quantize_weight_*_absmax`` (:179-190), bit for bit in fp16 and
        fp32; in bf16 the reference's rounded quotient can reach 128, which the int8 code
        saturates to 127."""
        q = self.qweight.to(self.compute_dtype)
        s = self.w_scale.to(self.compute_dtype)
        if self.weight_quant_name == "per_channel":
            return q * s.view(-1, 1)
        if self.weight_quant_name == "per_tensor":
            return q * s
        g = self.group_size
        return (q.view(self.out_features, -1, g) * s.view(self.out_features, -1, 1)).view(self.out_features, -1)

    @weight.setter
    def weight(self, value: torch.Tensor) -> None:
        """Assigning a float weight (what reference-style code does with ``module.weight = ...``)
        re-quantizes it with this layer's weight granularity."""
        out = ops.quantize_weight(value.detach().to(self.qweight.device if self.qweight.is_cuda else value.device),
                                  ops.WEIGHT_GRANULARITY[self.weight_quant_name], self.group_size, n_bits=self.n_bits)
        self.qweight, self.w_scale = out["q"], out["scale"]
        self.compute_dtype = value.dtype

    # -- checkpoints ---------------------------------------------------------------------------
    def get_extra_state(self):
        """What a checkpoint needs besides the tensors (int8 codes ``qweight``, fp32 ``w_scale``,
        ``bias``) to rebuild the layer."""
        return {"kind": "W8A8Linear", "in_features": self.in_features, "out_features": self.out_features,
                "act_quant": self.act_quant_name, "weight_quant": self.weight_quant_name,
                "quantize_output": self.quantize_output, "group_size": self.group_size, "n_bits": self.n_bits,
                "compute_dtype": str(self.compute_dtype).split(".")[-1]}

    def set_extra_state(self, state):
        self.act_quant_name, self.weight_quant_name = state["act_quant"], state["weight_quant"]
        self.quantize_output = bool(state["quantize_output"])
        self.output_quant_name = self.act_quant_name if self.quantize_output else "None"
        self.group_size, self.n_bits = state["group_size"], state["n_bits"]
        self.compute_dtype = getattr(torch, state["compute_dtype"])

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        """Accepts this module's own format and the reference's (RTN_quantization/per_tensor_channel_group.py:111-128:
        a float ``weight`` [N, K], already fake-quantized or not, and a ``bias`` of shape [1, N] or [N]): a float
        weight is quantized on the way in."""
        wkey, bkey = prefix + "weight", prefix + "bias"
        if wkey in state_dict and prefix + "qweight" not in state_dict:
            w = state_dict.pop(wkey)
            dev = self.qweight.device if self.qweight.is_cuda else w.device
            if dev.type != "cuda":
                raise RuntimeError("loading a float weight into W8A8Linear quantizes it on the GPU: move the module to a CUDA device first")
            out = ops.quantize_weight(w.detach().to(dev), ops.WEIGHT_GRANULARITY[self.weight_quant_name], self.group_size,
                                      n_bits=self.n_bits)
            state_dict[prefix + "qweight"], state_dict[prefix + "w_scale"] = out["q"], out["scale"]
            self.compute_dtype = w.dtype
            if prefix + "_extra_state" not in state_dict:
                state_dict[prefix + "_extra_state"] = self.get_extra_state()
        if bkey in state_dict and state_dict[bkey] is not None and self._buffers.get("bias") is not None:
            b = state_dict[bkey].reshape(-1)
            state_dict[bkey] = b
            if self.bias.dtype != b.dtype:                          # the bias keeps the checkpoint's dtype
                self._buffers["bias"] = torch.empty_like(self.bias, dtype=b.dtype)
        skey = prefix + "w_scale"
        if skey in state_dict and state_dict[skey].shape != self.w_scale.shape:   # [N] | [1] | [N, K/g] by granularity
            self._buffers["w_scale"] = torch.empty(state_dict[skey].shape, dtype=torch.float32, device=self.w_scale.device)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

    def act_quant(self, x):
        """Fake-quantize like the reference's ``self.act_quant`` partial (:130-140)."""
        out = ops.quantize(x, ops.ACT_GRANULARITY[self.act_quant_name], self.group_size, codes=False,
                           fake_quant=True, n_bits=self.n_bits)
        return out["fq"]

    def output_quant(self, y):
        return self.act_quant(y) if self.quantize_output else y

    @torch.no_grad()
    def forward(self, x, residual=None, activation=None, out_dtype=None):
        """``y = x_q @ W_q^T`` dequantized, plus bias (:157-162).  Extras beyond the reference:
        ``activation="gelu"`` and ``residual`` are applied inside the GEMM epilogue, ``out_dtype``
        selects the stored type.  With ``quantize_output`` the result is fake-quantized again."""
        a_gran = ops.ACT_GRANULARITY[self.act_quant_name]
        w_gran = ops.WEIGHT_GRANULARITY[self.weight_quant_name]
        xa = ops.quantize(x, a_gran, self.group_size, divisor=self.smooth_divisor, hadamard=self.hadamard,
                          n_bits=self.n_bits)
        y = ops.gemm_i8(xa["q"], self.qweight, xa["scale"], self.w_scale, a_gran, w_gran,
                        self.group_size or 0, bias=self.bias, residual=residual,
                        activation=ACT_GELU if activation == "gelu" else ACT_NONE,
                        out_dtype=out_dtype or x.dtype)
        if self.quantize_output:
            y = self.output_quant(y)
        return y

    def can_fuse_prologue(self) -> bool:
        """True when LayerNorm / row gather may be folded into this layer's quantization kernel
        (per-token and per-group activations; a per-tensor scale needs a separate reduction)."""
        return self.act_quant_name in ("per_token", "per_group_token")

    @torch.no_grad()
    def forward_fused(self, x, row_map=None, layer_norm=None, as_dtype=None, residual=None,
                      activation=None, out_dtype=None):
        """The layer with its neighbours folded in: ``x`` is [rows, K]; ``row_map`` gathers rows
        (window partition / unpartition), ``layer_norm=(w, b, eps)`` normalises them, ``as_dtype``
        reads bf16 storage as fp16, all inside K1; ``activation`` / ``residual`` / ``out_dtype``
        act in K2's epilogue.  Returns [rows_out, N]."""
        a_gran = ops.ACT_GRANULARITY[self.act_quant_name]
        w_gran = ops.WEIGHT_GRANULARITY[self.weight_quant_name]
        tdtype = as_dtype or x.dtype
        xa = ops.quantize(x, a_gran, self.group_size, divisor=self.smooth_divisor, hadamard=self.hadamard,
                          n_bits=self.n_bits, row_map=row_map, layer_norm=layer_norm, as_dtype=as_dtype)
        y = ops.gemm_i8(xa["q"], self.qweight, xa["scale"], self.w_scale, a_gran, w_gran,
                        self.group_size or 0, bias=self.bias, residual=residual,
                        activation=ACT_GELU if activation == "gelu" else ACT_NONE,
                        out_dtype=out_dtype or tdtype)
        if self.quantize_output:
            y = self.output_quant(y)
        return y

    @staticmethod
    def from_float(module, n_bits, weight_quant="per_channel", act_quant="per_token",
                   quantize_output=False, group_size=None):
        """Same signature as the reference (:164-196).  The source weight must live on a CUDA
        device; like the reference, the source module's weight is overwritten with its
        fake-quantized value."""
        assert isinstance(module, torch.nn.Linear)
        if weight_quant not in ops.WEIGHT_GRANULARITY:
            raise ValueError(f"Invalid weight_quant: {weight_quant}")
        new_module = W8A8Linear(module.in_features, module.out_features, module.bias is not None,
                                act_quant=act_quant, quantize_output=quantize_output,
                                group_size=group_size, n_bit=n_bits)
        w = module.weight.data
        if weight_quant == "per_group" or act_quant == "per_group_token":
            ops.check_gemm_group_size(module.in_features, group_size)
        out = ops.quantize_weight(w, ops.WEIGHT_GRANULARITY[weight_quant], group_size, codes=True,
                                  fake_quant=True, n_bits=n_bits)
        w.copy_(out["fq"])                               # the reference quantizes the source in place
        new_module.qweight = out["q"]
        new_module.w_scale = out["scale"]
        new_module.weight_quant_name = weight_quant
        new_module.compute_dtype = w.dtype
        if module.bias is not None:
            new_module.bias = module.bias.data
        return new_module

    def __repr__(self):
        return (f"W8A8Linear({self.in_features}, {self.out_features}, bias={self.bias is not None}, "
                f"weight_quant={self.weight_quant_name}, act_quant={self.act_quant_name}, "
                f"output_quant={self.output_quant_name})")
