"""Packed checkpoints of a quantized encoder: int8 weight codes, fp32 scales, biases and the
rotation flags, instead of the reference's fake-quantized float weights.

The reference saves the whole ``state_dict`` of the model it has just quantized
(quant/e2e_quant.py:10-14, RTN_quantization/Smooth_sam.py:126-142) and rebuilds the quantized
structure in code before loading it.  Here the structure travels with the tensors: every
``W8A8Linear`` / ``ActQuantWrapper`` stores its configuration as extra state, so
``load_quantized`` can turn the float skeleton's ``nn.Linear`` children into the right quantized
modules before ``load_state_dict`` fills them.  Nothing is re-quantized on load.
"""
from __future__ import annotations

from typing import Union

import torch
from torch import nn

FORMAT = 1


def quantized_state_dict(model: nn.Module) -> dict:
    """``model.state_dict()`` plus a format tag; tensors stay on their device."""
    return {"format": FORMAT, "state_dict": model.state_dict()}


def save_quantized(model: nn.Module, path: str) -> None:
    torch.save(quantized_state_dict(model), path)


def _child(root: nn.Module, dotted: str):
    parent = root
    parts = dotted.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    return parent, parts[-1]


def restore_quantized_modules(model: nn.Module, state_dict: dict) -> int:
    """Replace every ``nn.Linear`` of ``model`` whose checkpoint entry is a quantized layer by an
    empty ``W8A8Linear`` / ``ActQuantWrapper`` of the recorded configuration (on the Linear's
    device).  Returns how many were replaced."""
    from .RTN_quantization.per_tensor_channel_group import W8A8Linear
    from .quarot.utils import ActQuantWrapper
    replaced = 0
    for key in [k for k in state_dict if k.endswith("._extra_state") or k == "_extra_state"]:
        state = state_dict[key]
        if not isinstance(state, dict) or state.get("kind") not in ("W8A8Linear", "ActQuantWrapper"):
            continue
        name = key[: -len("._extra_state")]
        parent, attr = _child(model, name)
        cur = getattr(parent, attr)
        if not isinstance(cur, nn.Linear):
            continue                                        # already a quantized module
        dev = cur.weight.device
        if state["kind"] == "W8A8Linear":
            new = W8A8Linear(cur.in_features, cur.out_features, cur.bias is not None, act_quant=state["act_quant"],
                             quantize_output=state["quantize_output"], group_size=state["group_size"], n_bit=state["n_bits"])
            new = new.to(dev)
        else:
            new = ActQuantWrapper(cur, act_quant=state["act_quant_name"], weight_quant=None, n_bit=state["n_bits"],
                                  group_size=state["group_size"])
        setattr(parent, attr, new)
        replaced += 1
    return replaced


def load_quantized(model: nn.Module, source: Union[str, dict], strict: bool = True) -> nn.Module:
    """Load a packed checkpoint into a float skeleton of the same architecture (already on its
    CUDA device): quantized layers are re-created from the recorded configuration, then all tensors
    are loaded.  ``source`` is a path or the dictionary ``quantized_state_dict`` returned."""
    blob = torch.load(source, map_location="cpu") if isinstance(source, str) else source
    if blob.get("format") != FORMAT:
        raise ValueError(f"unknown checkpoint format {blob.get('format')!r}")
    sd = blob["state_dict"]
    restore_quantized_modules(model, sd)
    model.load_state_dict(sd, strict=strict)
    return model
