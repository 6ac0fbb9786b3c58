"""Host-side failure detection: a rank that leaves (or stops answering) between steps is noticed by the others before
their next launch. Ranks are CPU processes sharing a file store; no GPU and no collective is involved."""

import multiprocessing as mp
import time

import pytest


def _rank(rank, world, path, leave_at, silent_at, q):
    import torch.distributed as dist

    from lyra_b200.parallel.health import Heartbeat, PeerLost

    store = dist.FileStore(path, world)
    hb = Heartbeat(store, rank, world)
    try:
        for step in range(6):
            if rank == 1 and step == leave_at:
                hb.leave()
                q.put((rank, "left", step))
                return
            if rank == 1 and step == silent_at:
                time.sleep(3.0)            # alive but stuck: never announces the step
                q.put((rank, "stuck", step))
                return
            hb.beat(step)
            hb.check(step, timeout=1.0)
            time.sleep(0.01)               # the "training step"
        hb.leave()
        q.put((rank, "done", 6))
    except PeerLost as e:
        q.put((rank, f"lost:{e.rank}", step))


@pytest.mark.parametrize("mode", ["leave", "silent", "healthy"])
def test_heartbeat_detects_a_lost_rank(tmp_path, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    leave_at = 3 if mode == "leave" else -1
    silent_at = 2 if mode == "silent" else -1
    world = 3
    procs = [ctx.Process(target=_rank, args=(r, world, str(tmp_path / "store"), leave_at, silent_at, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict()
    for _ in range(world):
        r, what, step = q.get(timeout=60)
        results[r] = (what, step)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    if mode == "healthy":
        assert all(v == ("done", 6) for v in results.values()), results
    elif mode == "leave":
        assert results[1] == ("left", 3)
        assert results[0] == ("lost:1", 3) and results[2] == ("lost:1", 3), results     # noticed before running step 3
    else:
        assert results[0] == ("lost:1", 2) and results[2] == ("lost:1", 2), results
