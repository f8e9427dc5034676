"""CPU tests (gloo, world size 2) of the batch-sharding plumbing: shard ranges, the logits
all-gather with equal and unequal shards, and what the other ranks see when one rank fails on
the host."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vtpack_b200 import parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    r, w, _ = parallel.init_from_env("gloo")
    assert (r, w) == (rank, world)
    lo, hi = parallel.shard_range(total, rank, world)
    full = torch.arange(total * 5, dtype=torch.float32).reshape(total, 5)
    local = full[lo:hi].clone()                      # this rank's logits
    gathered = parallel.gather_logits(local)
    ok = torch.equal(gathered, full)
    if (hi - lo) * world == total:                   # equal shards: the preallocated fast path too
        out = torch.empty(total, 5)
        parallel.gather_logits_equal(local, out)
        ok = ok and torch.equal(out, full)
    q.put((rank, ok, lo, hi))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total", [8, 7])
def test_gather_logits_gloo(total):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in res)
    assert res[0][2] == 0 and res[0][3] == res[1][2] and res[1][3] == total


def test_shard_range_covers_everything():
    for total in (0, 1, 5, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [parallel.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _failing_worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    dist.barrier()
    def report(msg, code):
        q.put((rank, msg))
        q.close()
        q.join_thread()                              # flush before leaving without cleanup
        os._exit(code)

    if rank == 1:
        report("left", 3)                            # host-side failure between steps, nothing in flight
    try:
        parallel.gather_logits(torch.zeros(2, 3))
        report("no error", 0)
    except Exception as e:                           # noqa: BLE001 - the surviving rank must see an error
        report("error:" + type(e).__name__, 0)


def test_rank_failure_is_reported_to_survivor():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert got[1] == "left"
    assert got[0].startswith("error:")
