"""Data-parallel sharding of an image batch over the GPUs of one node.

The only parallelism in the reference is torch DDP around its evaluation loop with a metric
all-reduce (quant/hq44k_engine_quan.py:312-319,404).  Encoding is embarrassingly parallel over
images, so here each rank (one process per GPU) encodes a contiguous slice of the global batch
with replicated int8 weights and no collective on the data path; one gather of the embeddings
after the timed region serves verification only.
"""
from __future__ import annotations

import datetime
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(rank: int, world_size: int, total: int) -> Tuple[int, int]:
    """[start, stop) of the items rank ``rank`` owns: contiguous, sizes differ by at most one,
    earlier ranks take the larger shards."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def init_process_group(backend: Optional[str] = None, timeout_s: float = 600.0, device: Optional[torch.device] = None) -> Tuple[int, int]:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun's
    environment). Returns (rank, world_size); a single process needs no group."""
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        kwargs = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world


def gather_shards(local: torch.Tensor, total: int, dst: int = 0) -> Optional[torch.Tensor]:
    """Reassemble per-rank shards (rows of ``shard_range``) on rank ``dst`` in global order.
    Returns the [total, ...] tensor there and None elsewhere.  Raises RuntimeError if a rank does
    not arrive within the process group's timeout."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    sizes = [shard_range(r, world, total) for r in range(world)]
    if local.shape[0] != sizes[rank][1] - sizes[rank][0]:
        raise ValueError("local shard has the wrong number of rows")
    bufs: Optional[List[torch.Tensor]] = None
    if rank == dst:
        bufs = [torch.empty((b - a,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device) for a, b in sizes]
    if len({b - a for a, b in sizes}) == 1:
        dist.gather(local.contiguous(), bufs, dst=dst)
    else:                                            # ragged shards: point-to-point
        if rank == dst:
            reqs = [dist.irecv(bufs[r], src=r) for r in range(world) if r != dst]
            bufs[dst].copy_(local)
            for q in reqs:
                q.wait()
        else:
            dist.send(local.contiguous(), dst=dst)
    return torch.cat(bufs, 0) if rank == dst else None
