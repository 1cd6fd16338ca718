"""Activation-scale calibration (RTN_quantization/calibration.py:16-69 of the reference)."""
import functools

import torch
from torch import nn


@torch.no_grad()
def get_act_scales_sam(model, batched_input, num_samples=512):
    """Per-channel running max |x| of the input of every ``attn.qkv | attn.proj | mlp.lin1 |
    mlp.lin2`` Linear of ``model.image_encoder`` (RTN_quantization/calibration.py:16-69; the
    statistic is ``stat_tensor``, :35-49: fp32, kept on the CPU).  ``batched_input`` is an
    iterable of image batches ``[B, 3, H, W]`` already normalised; the reference's version feeds
    SAM prompt dictionaries through the whole model, which needs its mask decoder."""
    model.eval()
    act_scales = {}

    def stat_tensor(name, tensor):
        if tensor is None or not isinstance(tensor, torch.Tensor) or tensor.dim() < 2:
            return
        hidden_dim = tensor.shape[-1]
        tensor = tensor.reshape(-1, hidden_dim).abs().detach()
        current_max = torch.max(tensor, dim=0)[0].float().cpu()
        act_scales[name] = torch.max(act_scales[name], current_max) if name in act_scales else current_max

    def stat_input_hook(m, x, y, name):
        if x is None:
            return
        if isinstance(x, tuple):
            x = x[0]
        stat_tensor(name, x)

    hooks = []
    for name, module in model.image_encoder.named_modules():
        if isinstance(module, nn.Linear) and any(p in name for p in ["attn.qkv", "attn.proj", "mlp.lin1", "mlp.lin2"]):
            hooks.append(module.register_forward_hook(functools.partial(stat_input_hook, name=f"image_encoder.{name}")))
    try:
        for i, images in enumerate(batched_input):
            if i >= num_samples:
                break
            model.image_encoder(images)
    finally:
        for h in hooks:
            h.remove()
    return act_scales
