"""Expert re-placement by measured load: the planner, the relabelling symmetry of a MoE layer, and two gloo ranks that move
experts (masters and optimizer moments) in the middle of a run without changing the training trajectory."""

import os
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
os.environ["LYRA_SMALL_LEAF"] = "2048"

from lyra_b200.parallel.placement import ExpertLoadMeter, apply_slot_permutation, plan_slots, rank_loads  # noqa: E402
from tests.helpers import free_port  # noqa: E402


def test_planner_balances_within_capacities_and_moves_little():
    load = [40, 30, 5, 5, 4, 4, 6, 6]                       # rank 0 of 2 holds 80 of 100 tokens
    perm = plan_slots(load, world=2, e_local=4)
    assert sorted(perm) == list(range(8))
    after = rank_loads([load[o] for o in perm], 4, 2)
    assert max(after) == 53 and sum(after) == 100              # 40 + the three lightest: the optimum under four slots per rank
    assert sum(1 for s, o in enumerate(perm) if s != o) <= 4   # one expert goes each way, nothing else is shuffled around
    # seven routed experts, the eighth slot is the shared expert: rank 1 has only three routed slots
    perm = plan_slots([9, 9, 9, 9, 1, 1, 1], world=2, e_local=4)
    assert sorted(perm) == list(range(7))
    assert max(rank_loads([[9, 9, 9, 9, 1, 1, 1][o] for o in perm], 4, 2)) <= 21
    # nothing to gain: already balanced, or one expert that outweighs all others wherever it sits
    assert plan_slots([5, 5, 5, 5, 5, 5, 5, 5], 2, 4) is None
    assert plan_slots([100, 0, 0, 0, 1, 1, 1, 1], 2, 4) is None
    # eight ranks, a skewed (Zipf-like) load
    rng = np.random.default_rng(0)
    load = (1000 / np.arange(1, 129) ** 0.8)[rng.permutation(128)].tolist()
    perm = plan_slots(load, world=8, e_local=16)
    after = rank_loads([load[o] for o in perm], 16, 8)
    floor = max(load) + sum(sorted(load)[:15])                 # the heaviest expert still needs fifteen companions on its rank
    assert max(after) <= 1.01 * max(floor, sum(load) / 8) and max(after) < 0.9 * max(rank_loads(load, 16, 8))


def test_meter_counts_tokens_per_slot():
    m = ExpertLoadMeter([1, 3], 7, "cpu")
    m.add(1, torch.tensor([[0, 2], [2, 6]]))
    m.add(3, torch.tensor([[5, 5]]))
    m.add(0, torch.tensor([[1]]))                            # not a MoE layer: ignored
    assert m.counts[0].tolist() == [1, 0, 2, 0, 0, 0, 1] and m.counts[1, 5] == 2
    m.reset()
    assert m.counts.sum() == 0


def test_relabelling_experts_leaves_the_model_unchanged():
    from lyra_b200.model import ModelWeights, model_apply
    from lyra_b200.nn.params import tree_dict
    from lyra_b200.training.optimizer import OptimizerState
    from tests.helpers import small_config

    c = small_config(n_routed_experts=7, n_shared_experts=1, n_active_experts=3, use_mlp_bias=True, use_router_bias=True)
    w = ModelWeights.init(0, c)
    params = tree_dict(w)
    for p, t in params.items():                              # biases start at zero: make them tell the experts apart
        if p.endswith("bias"):
            t.copy_(torch.randn_like(t) * 0.1)
    tokens = torch.randint(0, c.vocab_size, (2, c.seq_len), generator=torch.Generator().manual_seed(0))
    before, _ = model_apply(tokens, w, None, c)[:2]
    rt = SimpleNamespace(e_local=c.n_experts, rank=0, world=1, group=None)
    perm = [3, 0, 6, 1, 2, 5, 4]
    old_up = params["layers/1/mlp/mlp_up"].clone()
    apply_slot_permutation(rt, 1, perm, params, OptimizerState())
    assert torch.equal(params["layers/1/mlp/mlp_up"][0], old_up[3]) and torch.equal(params["layers/1/mlp/mlp_up"][7], old_up[7])
    after, _ = model_apply(tokens, w, None, c)[:2]
    assert torch.allclose(before, after, atol=1e-5)


def _cfg():
    from tests.helpers import small_config

    return small_config(n_routed_experts=7, n_shared_experts=1, n_active_experts=3, n_embd=64, head_dim=16, n_attn_heads=4, n_kv_heads=2,
                        vocab_size=2000, padded_vocab_size=2048, compute_dtype=torch.float32, seq_len=16, load_balance_weight=0.0)


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.model import ModelWeights
        from lyra_b200.parallel.runtime import Runtime
        from lyra_b200.training.state import init_train_state
        from lyra_b200.training.steps import Stepper
        from lyra_b200.training.train import TrainingConfig

        c = _cfg()
        tcfg = TrainingConfig(steps=8, batch_size=4, accumulation_steps=2)
        rt = Runtime.create(world_size=world, rank=rank, device="cpu", implementation="nccl", mcfg=c)
        w = ModelWeights.init(0, c, shard_fn=rt.shard_info)
        state = init_train_state(w, c, tcfg)
        st = Stepper(state, c, tcfg, device="cpu", rt=rt)
        assert rt.meter_expert_load()
        data = np.load(tmp + "/batch.npy")
        xs = data[:, rank * 2:(rank + 1) * 2]
        ys = np.roll(xs, -1, axis=-1)
        losses, reports = [], []
        for step in range(4):
            losses.append(float(st.train_step(xs, ys, step)["loss"]))
            if step == 1:
                assert float(rt.load_meter.counts.sum()) == 2 * 2 * 2 * 2 * c.seq_len * c.n_active_routed_experts   # steps x layers x microbatches x rows x T x k
                reports.append(rt.rebalance_experts(st.params, state.optimizer, min_gain=0.0))
                assert float(rt.load_meter.counts.sum()) == 0
        if rank == 0:
            torch.save({"losses": losses, "reports": reports}, f"{tmp}/placement.pt")
    finally:
        dist.destroy_process_group()


def test_two_ranks_move_experts_mid_run_and_keep_the_trajectory(tmp_path):
    from lyra_b200.model import ModelWeights
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper
    from lyra_b200.training.train import TrainingConfig

    c = _cfg()
    data = np.random.default_rng(0).integers(0, c.vocab_size, size=(2, 4, c.seq_len)).astype(np.int32)
    np.save(tmp_path / "batch.npy", data)
    mp.spawn(_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "placement.pt", weights_only=False)

    tcfg = TrainingConfig(steps=8, batch_size=4, accumulation_steps=2)
    w = ModelWeights.init(0, c)
    st = Stepper(init_train_state(w, c, tcfg), c, tcfg, device="cpu")
    want = [float(st.train_step(data, np.roll(data, -1, axis=-1), step)["loss"]) for step in range(4)]
    assert np.allclose(got["losses"], want, atol=2e-4), (got["losses"], want)
    report = got["reports"][0]
    assert report["layers_moved"] >= 1 and report["slabs_received"] >= 2          # up and down slabs of at least one expert arrived
    assert report["max_share_after"] <= report["max_share_before"]


def _loop_tcfg(tmp, run, **kw):
    from lyra_b200.data import DataLoaderConfig
    from lyra_b200.training.train import TrainingConfig

    return TrainingConfig(steps=6, batch_size=4, accumulation_steps=1, data_path=Path(tmp) / "tok.npy", eval_every=None, checkpoint_every=6,
                          checkpoint_path=Path(tmp) / run, log_every=1, data_loader=DataLoaderConfig(worker_count=1), **kw)


def _loop_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.model import ModelWeights
        from lyra_b200.parallel.runtime import Runtime
        from lyra_b200.training.train import train

        c = _cfg()
        rt = Runtime.create(world_size=world, rank=rank, device="cpu", implementation="nccl", mcfg=c)
        model = ModelWeights.init(0, c, shard_fn=rt.shard_info)
        train(model, c, _loop_tcfg(tmp, "moving", rebalance_experts_every=2, rebalance_min_gain=0.0), rt=rt, device="cpu")
    finally:
        dist.destroy_process_group()


def test_training_loop_with_periodic_re_placement_matches_the_static_run(tmp_path):
    import json

    from lyra_b200.model import ModelWeights
    from lyra_b200.training.train import train
    from tests.helpers import token_file

    c = _cfg()
    token_file(tmp_path / "tok.npy", n=4 * 8 * (c.seq_len + 1) * 4, vocab=c.vocab_size)
    mp.spawn(_loop_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    train(ModelWeights.init(0, c), c, _loop_tcfg(tmp_path, "static"), device="cpu")

    def losses(run):
        rows = [json.loads(l) for l in (tmp_path / run / "metrics.jsonl").read_text().splitlines()]
        return [r["loss"] for r in rows if r["kind"] == "train"]

    events = [json.loads(l) for l in (tmp_path / "moving" / "metrics.jsonl").read_text().splitlines() if json.loads(l)["kind"] == "experts"]
    assert [e["step"] for e in events] == [2, 4] and events[0]["layers_moved"] >= 1 and events[0]["max_share_after"] <= events[0]["max_share_before"]
    moving, static = losses("moving"), losses("static")
    assert len(moving) == len(static) == 6 and np.allclose(moving, static, atol=3e-4), (moving, static)
    # the checkpoint of the moved model is a relabelled copy of the static one: same multiset of experts per layer
    from lyra_b200.nn.checkpoints import load_leaf, resolve_checkpoint
    from lyra_b200.nn.params import ShardInfo

    a = load_leaf(resolve_checkpoint(tmp_path / "moving") / "params", "layers/1/mlp/mlp_down", ShardInfo())
    b = load_leaf(resolve_checkpoint(tmp_path / "static") / "params", "layers/1/mlp/mlp_down", ShardInfo())
    norms_a, norms_b = a.flatten(1).norm(dim=1).tolist(), b.flatten(1).norm(dim=1).tolist()
    assert np.allclose(sorted(norms_a), sorted(norms_b), rtol=2e-3)
    assert not np.allclose(norms_a, norms_b, rtol=2e-3)            # and experts did change slots
