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
    step = 0
    try:
        hb.beat(0)
        hb.check(0, timeout=120.0)         # start-up (importing torch in three fresh processes) is not what the test times
        for step in range(6):
            if rank == 1 and step == leave_at:
                hb.leave()
                q.put((rank, "left", step))
                return
            if rank == 1 and step == silent_at:
                time.sleep(9.0)            # alive but stuck: never announces the step
                q.put((rank, "stuck", step))
                return
            hb.beat(step)
            hb.check(step, timeout=4.0)       # generous: on a loaded machine a healthy peer can be a second late
            time.sleep(0.01)               # the "training step"
        hb.done()
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


def _train_rank(rank, world, port, tmp, fail):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LYRA_SMALL_LEAF="2048")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pathlib import Path

        from lyra_b200.data import DataLoaderConfig
        from lyra_b200.model import ModelWeights
        from lyra_b200.parallel.health import PeerLost
        from lyra_b200.parallel.runtime import Runtime
        from lyra_b200.training.train import TrainHooks, TrainingConfig, train
        from tests.helpers import small_config

        c = small_config(n_routed_experts=7, n_shared_experts=1, n_active_experts=3, seq_len=16)
        out = Path(tmp) / "run"
        resuming = not fail
        tcfg = TrainingConfig(steps=4, batch_size=4, accumulation_steps=1, data_path=Path(tmp) / "tok.npy", eval_every=None, checkpoint_every=2,
                              checkpoint_path=out, log_every=1, peer_timeout_seconds=20.0, data_loader=DataLoaderConfig(worker_count=1),
                              resume_from=out if resuming else None)

        class DieAfterTheCheckpoint(TrainHooks):
            def on_checkpoint(self, step, *a):
                if fail and rank == 1 and step == 2:
                    raise RuntimeError("this rank's node went away")

        rt = Runtime.create(world_size=world, rank=rank, device="cpu", implementation="nccl", mcfg=c)
        model = None if resuming else ModelWeights.init(0, c, shard_fn=rt.shard_info)
        outcome = "finished"
        try:
            train(model, c, tcfg, rt=rt, device="cpu", hooks=DieAfterTheCheckpoint())
        except PeerLost as e:
            outcome = f"peer lost: {e}"
        except RuntimeError as e:
            outcome = f"failed: {e}"
        (Path(tmp) / f"outcome{int(fail)}_{rank}.txt").write_text(outcome)
    finally:
        dist.destroy_process_group()


def test_training_loop_notices_a_lost_rank_and_the_restart_resumes(tmp_path):
    """A rank fails between two steps (after the step-2 checkpoint): the other rank learns it on the host at the next step
    boundary, before launching anything that would wait for the dead rank, and stops; the relaunched job resumes from step 2."""
    import json

    import torch.multiprocessing as mp

    from tests.helpers import free_port, token_file

    token_file(tmp_path / "tok.npy", n=4 * 17 * 8, vocab=500)
    mp.spawn(_train_rank, args=(2, free_port(), str(tmp_path), True), nprocs=2, join=True)
    assert (tmp_path / "outcome1_1.txt").read_text() == "failed: this rank's node went away"
    assert (tmp_path / "outcome1_0.txt").read_text() == "peer lost: rank 1 left the job"
    mp.spawn(_train_rank, args=(2, free_port(), str(tmp_path), False), nprocs=2, join=True)
    assert (tmp_path / "outcome0_0.txt").read_text() == (tmp_path / "outcome0_1.txt").read_text() == "finished"
    rows = [json.loads(l) for l in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines() if json.loads(l)["kind"] == "train"]
    assert [r["step"] for r in rows] == [1, 2, 3, 4]
