"""Attention / MLP variants that rotate their input online (quarot/model_utils.py:134-172,227-241)
and the window helpers (:15-59).  ``Q`` is applied as a dense matmul exactly like the reference
unless the first Linear is a wrapper that has the rotation folded into its quantization kernel
(``ActQuantWrapper.set_pre_rotation``), in which case nothing is done here."""
from __future__ import annotations

from typing import Optional

import torch

from ..sam_encoder import Attention, MLPBlock, window_partition, window_unpartition  # noqa: F401


def get_rope_function_name(model):
    """SAM has no rotary embedding (quarot/model_utils.py:10-14)."""
    return None


def _rotate(x: torch.Tensor, Q: Optional[torch.Tensor], first_linear) -> torch.Tensor:
    if Q is None or getattr(first_linear, "pre_signs", None) is not None:
        return x
    B, H, W, C = x.shape
    return torch.matmul(x.reshape(B, H * W, C), Q.to(device=x.device, dtype=x.dtype)).reshape(B, H, W, C)


class CustomAttention(Attention):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.Q = None

    def _take_Q(self, Q: Optional[torch.Tensor] = None):
        if Q is not None:
            self.Q = Q

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return super().forward(_rotate(x, self.Q, self.qkv))


class custom_MLPBlock(MLPBlock):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.Q = None

    def _take_Q(self, Q: Optional[torch.Tensor] = None):
        if Q is not None:
            self.Q = Q

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return super().forward(_rotate(x, self.Q, self.lin1), residual=residual)
