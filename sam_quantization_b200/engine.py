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
    device status word instead of hanging; their output is then incomplete.  ``lanes`` > 1 (graph mode
    only) encodes the batch as that many independent sub-batches on concurrent streams inside the one
    graph; results are identical, image by image.  ``check_status=True``
    makes every call synchronise and raise ``RuntimeError`` in that case; otherwise call
    ``runner.check()`` (or ``ops.check_status``) wherever the caller synchronises anyway."""

    def __init__(self, model: torch.nn.Module, batch: int, img_size: int = 1024, dtype: torch.dtype = torch.float16,
                 device: Optional[torch.device] = None, use_graph: bool = True, warmup: int = 3, check_status: bool = False,
                 lanes: int = 1):
        self.check_status = bool(check_status)
        self.encoder = getattr(model, "image_encoder", model)
        self.device = torch.device(device) if device is not None else next(self.encoder.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("EncoderRunner needs a CUDA device")
        self.lanes = int(lanes) if use_graph else 1
        if self.lanes < 1 or batch % self.lanes:
            raise ValueError(f"batch {batch} is not a multiple of lanes {lanes}")
        self.batch = batch
        self._copy_stream = None
        self.static_in = torch.zeros((batch, 3, img_size, img_size), dtype=dtype, device=self.device)
        self.graph = None
        per_lane = batch // self.lanes
        with torch.no_grad(), torch.cuda.device(self.device):
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(max(1, warmup)):                 # first calls build caches and cuDNN plans
                    self.static_out = self.encoder(self.static_in)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            lane_streams = []
            if self.lanes > 1:
                # every lane once outside the capture: per-stream library workspaces and the caches keyed
                # by the lane's batch size exist before the graph is recorded
                lane_streams = [torch.cuda.Stream(device=self.device) for _ in range(self.lanes)]
                for k, st in enumerate(lane_streams):
                    with torch.cuda.stream(st):
                        self.static_out[k * per_lane:(k + 1) * per_lane].copy_(
                            self.encoder(self.static_in[k * per_lane:(k + 1) * per_lane]))
                torch.cuda.synchronize(self.device)
            if use_graph:
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    if self.lanes == 1:
                        self.static_out = self.encoder(self.static_in)
                    else:
                        # The batch is split over `lanes` streams that fork from and join the capturing
                        # stream.  The lanes run the same kernel sequence on different images; a
                        # persistent GEMM fills every SM, so two GEMMs take turns, and the memory-bound
                        # kernels of one lane (quantization, LayerNorm) find room beside the GEMM of the
                        # other instead of leaving the tensor cores idle while they run.
                        main = torch.cuda.current_stream(self.device)
                        self.static_out = torch.empty_like(self.static_out)
                        for k, st in enumerate(lane_streams):
                            st.wait_stream(main)
                            with torch.cuda.stream(st):
                                self.static_out[k * per_lane:(k + 1) * per_lane].copy_(
                                    self.encoder(self.static_in[k * per_lane:(k + 1) * per_lane]))
                        for st in lane_streams:
                            main.wait_stream(st)

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

    @torch.no_grad()
    def encode(self, images: torch.Tensor, out: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """Encode ``images`` [n * batch, 3, S, S] into ``out`` [n * batch, C, h, w], ``batch`` images per
        forward.  With host tensors (pinned memory) the copy of chunk i + 1 to the device runs on a
        second stream while chunk i is being encoded, and the embeddings of chunk i leave for the host on a
        third while chunk i + 1 is encoded; the first copy of a call may already run under the last
        forward of the call before it.  Device tensors are encoded in place.  Returns ``out``; the work is
        ordered on the current stream (synchronise it before reading a host ``out``).  ``wait=False`` leaves
        the last copies back to the host unordered with the current stream, so that the next call's forward
        does not wait for them: call ``runner.synchronize()`` before reading ``out``."""
        n, b = images.shape[0], self.batch
        if n % b or out.shape[0] != n:
            raise ValueError(f"images and out must hold a multiple of {b} images")
        cur = torch.cuda.current_stream(self.device)
        if images.is_cuda:
            for i in range(0, n, b):
                out[i:i + b].copy_(self(images[i:i + b]), non_blocking=True)
            return out
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)      # host -> device
            self._back_stream = torch.cuda.Stream(device=self.device)      # device -> host (its own stream: a copy back that
            #                                                                waits for a forward must not hold up the next copy in)
            self._stage = [torch.empty_like(self.static_in) for _ in range(2)]
            self._stage_free = [torch.cuda.Event() for _ in range(2)]
            self._stage_used = [False, False]
            self._out_stage = [torch.empty_like(self.static_out) for _ in range(2)]
            self._out_free = [torch.cuda.Event() for _ in range(2)]
            self._out_used = [False, False]
        side, back = self._copy_stream, self._back_stream
        # The staging buffers are guarded by events of their own, not by the whole current stream: the
        # first copy of this call may therefore run while the last forward of the previous call is
        # still in flight (calls in a row pipeline across their boundaries).

        def stage_in(slot, lo):                                 # host -> staging buffer `slot`, on the copy stream
            with torch.cuda.stream(side):
                if self._stage_used[slot]:
                    side.wait_event(self._stage_free[slot])     # the forward that last read this slot has taken its copy
                self._stage[slot].copy_(images[lo:lo + b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
            return ev

        ready = [stage_in(0, 0)]
        for k, i in enumerate(range(0, n, b)):
            slot = k & 1
            if i + b < n:                                       # prefetch the next chunk while this one runs
                ready.append(stage_in(slot ^ 1, i + b))
            cur.wait_event(ready[k])
            self.static_in.copy_(self._stage[slot], non_blocking=True)
            self._stage_free[slot].record(cur)
            self._stage_used[slot] = True
            if self.graph is not None:
                self.graph.replay()
            else:
                self.static_out = self.encoder(self.static_in)
            if out.is_cuda:
                out[i:i + b].copy_(self.static_out, non_blocking=True)
            else:
                if self._out_used[slot]:
                    cur.wait_event(self._out_free[slot])        # the copy that last read this slot has finished
                self._out_stage[slot].copy_(self.static_out, non_blocking=True)
                done = torch.cuda.Event(); done.record(cur)
                with torch.cuda.stream(back):
                    back.wait_event(done)
                    out[i:i + b].copy_(self._out_stage[slot], non_blocking=True)
                    self._out_free[slot].record(back)
                self._out_used[slot] = True
        if wait:
            cur.wait_stream(back)
        if self.check_status:
            self.check()
        return out

    def synchronize(self) -> None:
        """Block until everything ``encode`` has queued, the copies back to the host included, is done."""
        torch.cuda.current_stream(self.device).synchronize()
        if self._copy_stream is not None:
            self._back_stream.synchronize()

    def check(self) -> None:
        """Synchronise and raise if a kernel of this device reported a timed-out wait."""
        from . import ops
        ops.check_status(self.device)
