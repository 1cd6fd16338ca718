"""Batch runner for a quantized image encoder: fixed-shape forward captured in a CUDA graph.

The reference runs its encoder eagerly, one Python-dispatched kernel at a time
(quant/hq44k_engine_quan.py:190-211 -> predictor(inputs)).  With the layer kernels fused, a block
is ~13 short launches and the host becomes the bottleneck; capturing the whole forward once and
replaying it removes the per-launch host cost.  All kernels of this package take their stream
explicitly and allocate nothing, so they are capturable as they are.
"""
from __future__ import annotations

from typing import Optional

import torch


class EncoderRunner:
    """``runner(images)`` == ``model.image_encoder(images)`` for batches of exactly ``batch`` images.

    ``images`` may live on the host (pinned memory makes the copy asynchronous) or on the device;
    they are copied into the graph's static input.  The returned tensor is the graph's static
    output: it is overwritten by the next call, so copy it if it must outlive that call.

    The GEMM and attention kernels give up on a stalled pipeline after a bounded wait and raise a
    device status word instead of hanging; their output is then incomplete.  ``check_status=True``
    makes every call synchronise and raise ``RuntimeError`` in that case; otherwise call
    ``runner.check()`` (or ``ops.check_status``) wherever the caller synchronises anyway."""

    def __init__(self, model: torch.nn.Module, batch: int, img_size: int = 1024, dtype: torch.dtype = torch.float16,
                 device: Optional[torch.device] = None, use_graph: bool = True, warmup: int = 3, check_status: bool = False):
        self.check_status = bool(check_status)
        self.encoder = getattr(model, "image_encoder", model)
        self.device = torch.device(device) if device is not None else next(self.encoder.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("EncoderRunner needs a CUDA device")
        self.batch = batch
        self.static_in = torch.zeros((batch, 3, img_size, img_size), dtype=dtype, device=self.device)
        self.graph = None
        with torch.no_grad(), torch.cuda.device(self.device):
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(max(1, warmup)):                 # first calls build caches and cuDNN plans
                    self.static_out = self.encoder(self.static_in)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            if use_graph:
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    self.static_out = self.encoder(self.static_in)

    @torch.no_grad()
    def __call__(self, images: torch.Tensor) -> torch.Tensor:
        if images.shape != self.static_in.shape:
            raise ValueError(f"expected a batch of shape {tuple(self.static_in.shape)}, got {tuple(images.shape)}")
        if images.data_ptr() != self.static_in.data_ptr():
            self.static_in.copy_(images, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.static_out = self.encoder(self.static_in)
        if self.check_status:
            self.check()
        return self.static_out

    def check(self) -> None:
        """Synchronise and raise if a kernel of this device reported a timed-out wait."""
        from . import ops
        ops.check_status(self.device)
