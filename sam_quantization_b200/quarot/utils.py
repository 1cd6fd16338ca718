"""QuaRot wrappers with the interface of quarot/utils.py: ``ActQuantWrapper`` (online Hadamard
+ activation quantization around a Linear), ``add_actquant`` / ``find_qlayers`` and the small
numpy Hadamard builders.  The wrapper's forward runs the fused CUDA kernels: the Hadamard
transform, the absmax and the int8 rounding are one pass of K1, the Linear is K2."""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch

from .. import ops
from .._lib import ACT_GELU, ACT_NONE
from ..RTN_quantization.per_tensor_channel_group import (quantize_activation_per_group_absmax_token_dim,
                                                          quantize_activation_per_tensor_absmax,
                                                          quantize_activation_per_token_absmax)
from .hadamard_utils import matmul_hadU_cuda


def parser_gen(argv=None):
    """Arguments of quarot/utils.py:29-96 that the SAM rotation recipe reads."""
    p = argparse.ArgumentParser()
    p.add_argument("--seed", type=int, default=123)
    p.add_argument("--device", type=str, default="cuda:0")
    p.add_argument("--algo", type=str, default="quarot")
    p.add_argument("--hidden_size_image_en", type=int, default=1024)
    p.add_argument("--num_attention_head_image_en", type=int, default=64)
    p.add_argument("--hidden_size_mask_de", type=int, default=256)
    p.add_argument("--num_attention_head_mask_de", type=int, default=8)
    p.add_argument("--rotate_mode", type=str, default="hadamard", choices=["hadamard", "random"])
    p.add_argument("--fp32_had", action="store_true", default=False)
    return p.parse_args(argv)


def _sylvester(n):
    H = np.array([[1]])
    while H.shape[0] < n:
        H = np.block([[H, H], [H, -H]])
    return H


def hadamard_matrix(nh, dh):
    """kron(H_nh, I_dh) (quarot/utils.py:98-116)."""
    return np.kron(_sylvester(nh), np.eye(dh))


def hadamard_matrix_transposed(nh, dh):
    """kron(I_nh, H_dh) (quarot/utils.py:117-137)."""
    return np.kron(np.eye(nh), _sylvester(dh))


_ACT_FUNCS = {
    "per_token": lambda x, bits, g: quantize_activation_per_token_absmax(x, n_bits=bits),
    "per_tensor": lambda x, bits, g: quantize_activation_per_tensor_absmax(x, n_bits=bits),
    "per_group_token": lambda x, bits, g: quantize_activation_per_group_absmax_token_dim(x, group_size=g, n_bits=bits),
}


class ActQuantizer(torch.nn.Module):
    """Stand-alone activation fake-quantizer (quarot/utils.py:138-199)."""

    def __init__(self, act_quant="per_token", group_size=None, n_bits=8):
        super().__init__()
        self.configure(n_bits, act_quant, group_size)

    def configure(self, bits, act_quant="per_token", group_size=None):
        if act_quant not in _ACT_FUNCS:
            raise ValueError(f"Invalid act_quant: {act_quant}")
        if act_quant == "per_group_token":
            assert group_size is not None, "group_size must be provided for per_group_token quantization"
        self.bits, self.group_size, self.act_quant_name = bits, group_size, act_quant

    def act_quant(self, x):
        return _ACT_FUNCS[self.act_quant_name](x, self.bits, self.group_size)

    def forward(self, x):
        return x if self.bits == 16 else self.act_quant(x)

    quantize = forward


class ActQuantWrapper(torch.nn.Module):
    """Wraps an ``nn.Linear`` (quarot/utils.py:202-298).  State the rotation recipe sets after
    construction: ``online_full_had``, ``online_partial_had``, ``had_K``, ``K``, ``had_dim``,
    ``fp32_had``, ``quantize_input``, ``quantize_output``; ``pre_signs`` (not in the reference)
    folds the online ``x @ Q`` of a randomized-Hadamard Q into the same kernel.

    ``fp32_had``: the kernel always computes the transform in fp32 and rounds once to the tensor
    dtype.  For power-of-two lengths (``K == 1``) that is also what the reference's library call
    does internally for half inputs, so both settings run the same code; for lengths with an
    explicit factor (``K > 1``: 768, 1280, 3072, 5120, 12 heads) ``fp32_had=False`` raises
    ``NotImplementedError`` at the first forward instead of returning values rounded differently
    from the reference's two-rounding half path.

    forward: [full | partial Hadamard] -> [int8 activation quantization] -> Linear ->
    [output fake-quant].  With ``quantize_input`` the Linear is the int8 GEMM on the stored weight
    codes; without it the transformed fp16 activation meets the fake-quantized float weight in a
    plain ``F.linear``, as in the reference."""

    supports_fused_epilogue = True

    def __init__(self, module: torch.nn.Linear, act_quant="per_token", weight_quant="per_channel", n_bit=8, group_size=None):
        super().__init__()
        assert isinstance(module, torch.nn.Linear)
        if act_quant not in ops.ACT_GRANULARITY:
            raise ValueError(f"Invalid act_quant: {act_quant}")
        if act_quant == "per_group_token" or weight_quant == "per_group":
            ops.check_gemm_group_size(module.in_features, group_size)
        self.module = module
        self.bias = module.bias
        self.group_size = group_size
        self.n_bits = n_bit
        self.act_quant_name = act_quant
        self.weight_quant_name = weight_quant
        self.register_buffer("had_K", torch.tensor(0))
        self._buffers["had_K"] = None
        self.K = 1
        self.online_full_had = False
        self.online_partial_had = False
        self.had_dim = 0
        self.fp32_had = False
        self.quantize_output = False
        self.quantize_input = False
        self.pre_signs = None
        self._pre_k, self._pre_hadk = 1, None
        self.register_buffer("qweight", None)            # int8 codes and fp32 scales of the weight: saved in checkpoints
        self.register_buffer("w_scale", None)
        if weight_quant in ops.WEIGHT_GRANULARITY:
            out = ops.quantize_weight(module.weight.data, ops.WEIGHT_GRANULARITY[weight_quant], group_size,
                                      codes=True, fake_quant=True, n_bits=n_bit)
            module.weight.data.copy_(out["fq"])          # the wrapped Linear keeps the fake-quantized weight
            self.qweight, self.w_scale = out["q"], out["scale"]
        self.weight = module.weight

    # -- checkpoints ---------------------------------------------------------------------------
    _FLAGS = ("K", "online_full_had", "online_partial_had", "had_dim", "fp32_had", "quantize_output", "quantize_input",
              "group_size", "n_bits", "act_quant_name", "weight_quant_name", "_pre_k")

    def get_extra_state(self):
        """The rotation flags a checkpoint must carry next to the tensors (weight codes and scales,
        the wrapped Linear, ``had_K``): which online transform runs, its factor order and head width,
        and the sign vector / factor of a folded ``x @ Q``."""
        state = {"kind": "ActQuantWrapper"}
        state.update({k: getattr(self, k) for k in self._FLAGS})
        state["pre_signs"] = None if self.pre_signs is None else self.pre_signs.detach().cpu()
        state["pre_hadk"] = None if self._pre_hadk is None else self._pre_hadk.detach().cpu()
        return state

    def set_extra_state(self, state):
        for k in self._FLAGS:
            setattr(self, k, state[k])
        dev = self.module.weight.device
        self.pre_signs = None if state["pre_signs"] is None else state["pre_signs"].to(dev)
        self._pre_hadk = None if state["pre_hadk"] is None else state["pre_hadk"].to(dev)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        dev = self.module.weight.device
        for name, dtype in (("qweight", torch.int8), ("w_scale", torch.float32), ("had_K", None)):
            t = state_dict.get(prefix + name)
            cur = self._buffers.get(name)
            if t is not None and (cur is None or cur.shape != t.shape or cur.dtype != t.dtype):
                self._buffers[name] = torch.empty(t.shape, dtype=t.dtype if dtype is None else dtype, device=dev)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

    def extra_repr(self) -> str:
        return f"Activation Quantization: {self.act_quant_name}"

    def act_quant(self, x):
        return _ACT_FUNCS[self.act_quant_name](x, self.n_bits, self.group_size)

    def _hadamard_spec(self, x):
        signs = self.pre_signs
        if (self.online_full_had or self.online_partial_had) and not self.fp32_had and int(self.K) > 1:
            # quarot/utils.py:260-261,280-288: without fp32_had the reference runs the power-of-two part in the
            # fast_hadamard_transform library, rounds to the tensor dtype, and mixes the K chunks with a matmul in
            # that dtype (a second rounding).  The kernel here evaluates the whole transform in fp32 and rounds
            # once; rather than silently returning differently rounded values it asks for the mode it implements.
            raise NotImplementedError(
                f"online Hadamard with an explicit order-{int(self.K)} factor is implemented in fp32 with one rounding: "
                "construct the rotation with fp32_had=True")
        if self.online_full_had or signs is not None:
            hk = None if self.K == 1 or self.had_K is None else self.had_K.to(x.device)
            if not self.online_full_had:
                # only the sign flip + transform of the folded x @ Q
                return ops.Hadamard("full", had_k=self._pre_k, hadk=self._pre_hadk, signs=signs)
            return ops.Hadamard("full", had_k=int(self.K), hadk=hk, signs=signs)
        if self.online_partial_had:
            hk = None if self.K == 1 or self.had_K is None else self.had_K.to(x.device)
            return ops.Hadamard("partial", had_k=int(self.K), hadk=hk, had_dim=int(self.had_dim))
        return None

    def set_pre_rotation(self, signs, hadK=None, K=1):
        """Fold ``x @ Q`` with ``Q = random_hadamard_matrix`` (diag(signs) H / sqrt(n)) into the
        quantization kernel of this layer (quarot/model_utils.py:146-152,235-240 does it as a
        dense matmul before the Linear)."""
        self.pre_signs = signs
        self._pre_k = int(K)
        self._pre_hadk = hadK

    def can_fuse_prologue(self) -> bool:
        return bool(self.quantize_input) and self.qweight is not None and \
            self.act_quant_name in ("per_token", "per_group_token")

    @torch.no_grad()
    def forward_fused(self, x, row_map=None, layer_norm=None, as_dtype=None, residual=None,
                      activation=None, out_dtype=None):
        """Same contract as ``W8A8Linear.forward_fused``.  An online Hadamard and a LayerNorm are one
        pass of K1 for fp16 rows of 1024 or 4096 elements (power-of-two transform, per-token codes) and
        two passes otherwise (normalise + gather, then transform + quantize)."""
        spec = self._hadamard_spec(x)
        tdtype = as_dtype or x.dtype
        if spec is not None and (layer_norm is not None) and not (
                self.act_quant_name == "per_token" and ops.hadamard_layer_norm_fused(x, spec, as_dtype)):
            x = ops.quantize(x, ops.GRAN_ROW, codes=False, transformed=True, row_map=row_map,
                             layer_norm=layer_norm, as_dtype=as_dtype)["tx"]
            row_map, layer_norm, as_dtype = None, None, None
        a_gran = ops.ACT_GRANULARITY[self.act_quant_name]
        xa = ops.quantize(x, a_gran, self.group_size, hadamard=spec, n_bits=self.n_bits, row_map=row_map,
                          layer_norm=layer_norm, as_dtype=as_dtype)
        y = ops.gemm_i8(xa["q"], self.qweight, xa["scale"], self.w_scale, a_gran,
                        ops.WEIGHT_GRANULARITY[self.weight_quant_name], self.group_size or 0,
                        bias=self.bias, residual=residual,
                        activation=ACT_GELU if activation == "gelu" else ACT_NONE, out_dtype=out_dtype or tdtype)
        if self.quantize_output:
            y = self.act_quant(y)
        return y

    @torch.no_grad()
    def forward(self, x, residual=None, activation=None, out_dtype=None):
        x_dtype = x.dtype
        spec = self._hadamard_spec(x)
        act = ACT_GELU if activation == "gelu" else ACT_NONE
        if self.quantize_input and self.qweight is not None:
            a_gran = ops.ACT_GRANULARITY[self.act_quant_name]
            xa = ops.quantize(x, a_gran, self.group_size, hadamard=spec, n_bits=self.n_bits)
            y = ops.gemm_i8(xa["q"], self.qweight, xa["scale"], self.w_scale, a_gran,
                            ops.WEIGHT_GRANULARITY[self.weight_quant_name], self.group_size or 0,
                            bias=self.bias, residual=residual, activation=act, out_dtype=out_dtype or x_dtype)
        else:
            if spec is not None:
                x = ops.quantize(x, ops.GRAN_ROW, hadamard=spec, codes=False, transformed=True)["tx"]
            if self.quantize_input:
                x = self.act_quant(x)
            y = self.module(x).to(x_dtype)
            if activation == "gelu":
                y = torch.nn.functional.gelu(y)
            if residual is not None:
                y = y + residual
            if out_dtype is not None:
                y = y.to(out_dtype)
        if self.quantize_output:
            y = self.act_quant(y)
        return y


def add_actquant(module, name="", layers=(torch.nn.Linear,), rtn_ro_config=None):
    """Wrap every ``nn.Linear`` below ``module`` in an ``ActQuantWrapper`` (quarot/utils.py:301-395),
    configured from ``rtn_ro_config.{n_bits, weight_quant, act_quant, group_size, quantize_output,
    quantize_input}`` when given.  Children that are already wrappers are left alone."""
    if isinstance(module, ActQuantWrapper):
        return
    layers = tuple(layers)

    def wrap(lin):
        if rtn_ro_config is None:
            return ActQuantWrapper(lin)
        w = ActQuantWrapper(lin, act_quant=rtn_ro_config.act_quant, weight_quant=rtn_ro_config.weight_quant,
                            n_bit=rtn_ro_config.n_bits, group_size=rtn_ro_config.group_size)
        w.quantize_output = bool(rtn_ro_config.quantize_output)
        w.quantize_input = bool(rtn_ro_config.quantize_input)
        return w

    for child_name, child in list(module.named_children()):
        if type(child) in layers:
            setattr(module, child_name, wrap(child))
        elif type(child) in (torch.nn.Sequential, torch.nn.ModuleList):
            members = [wrap(m) if type(m) in layers else m for m in child.children()]
            setattr(module, child_name, type(child)(members) if isinstance(child, torch.nn.ModuleList)
                    else torch.nn.Sequential(*members))
    for child_name, child in module.named_children():
        add_actquant(child, name + "." + child_name if name != "" else child_name, layers, rtn_ro_config)


def find_qlayers(module, layers=(torch.nn.Linear, ActQuantWrapper), name=""):
    """{qualified name: module} of every Linear / wrapper below ``module`` (quarot/utils.py:397-406)."""
    if type(module) in tuple(layers):
        return {name: module}
    res = {}
    for child_name, child in module.named_children():
        res.update(find_qlayers(child, layers=layers, name=name + "." + child_name if name != "" else child_name))
    return res


def cleanup_memory(verbos=True) -> None:
    """Run the garbage collector and release cached GPU blocks (quarot/utils.py:408-437)."""
    import gc
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
