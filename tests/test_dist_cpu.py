"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2 and 3): shard
arithmetic, gather order, and detection of a rank that never arrives."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from sam_quantization_b200.dist import shard_range


def test_shard_ranges_partition_exactly():
    for total in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(r, world, total) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        shard_range(2, 2, 8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, total, absent_rank, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    from sam_quantization_b200.dist import gather_shards, init_process_group, shard_range as sr
    init_process_group("gloo", timeout_s=4.0)
    a, b = sr(rank, world, total)
    local = torch.arange(a, b, dtype=torch.float32).view(-1, 1).repeat(1, 3)       # row i holds value i
    try:
        if rank == absent_rank:
            # this rank "fails" between steps: it leaves without joining the collective
            result[rank] = "left"
            return
        out = gather_shards(local, total, dst=0)
        if rank == 0:
            ok = out.shape == (total, 3) and torch.equal(out[:, 0], torch.arange(total, dtype=torch.float32))
            result[rank] = "ok" if ok else "wrong order"
        else:
            result[rank] = "ok"
    except Exception as e:                                     # the survivors see an error, not a hang
        result[rank] = "error: " + type(e).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(world, total, absent_rank=-1):
    port = _free_port()
    with mp.Manager() as mgr:
        result = mgr.dict()
        procs = [mp.get_context("spawn").Process(target=_worker, args=(r, world, port, total, absent_rank, result))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(60)
            if p.is_alive():
                p.kill()
        return dict(result)


@pytest.mark.timeout(120)
def test_gather_reassembles_global_order_world2_and_ragged_world3():
    assert _run(2, 8) == {0: "ok", 1: "ok"}
    assert _run(3, 7) == {0: "ok", 1: "ok", 2: "ok"}            # shards of 3, 2, 2


@pytest.mark.timeout(120)
def test_missing_rank_is_detected_not_hung():
    res = _run(2, 8, absent_rank=1)
    assert res[1] == "left"
    assert res[0].startswith("error")
