"""Two gloo ranks on CPU: the sharding runtime in its collective ("nccl") mode must reproduce the single-process step:
leaf ownership, weight gather, gradient reduce, replicated-leaf all-reduce, expert-parallel exchange, shared expert."""

import os
import sys
from dataclasses import replace
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from tests.helpers import free_port  # noqa: E402
os.environ["LYRA_SMALL_LEAF"] = "2048"  # shard the small test model's matrices too (inherited by the spawned ranks)


def _cfg():
    from tests.helpers import small_config

    return small_config(n_routed_experts=7, n_shared_experts=1, n_active_experts=3, n_embd=64, head_dim=16, n_attn_heads=4, n_kv_heads=2,
                        vocab_size=2000, padded_vocab_size=2048, compute_dtype=torch.float32, seq_len=16,
                        load_balance_weight=0.0)  # the balance term is a product of per-rank means, so it is not additive over ranks


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.model import ModelWeights
        from lyra_b200.nn.params import tree_dict
        from lyra_b200.parallel.runtime import Runtime
        from lyra_b200.training.state import init_train_state, save_checkpoint, load_train_state
        from lyra_b200.training.steps import Stepper
        from lyra_b200.training.train import TrainingConfig

        c = _cfg()
        tcfg = TrainingConfig(steps=4, batch_size=4, accumulation_steps=2)
        rt = Runtime.create(world_size=world, rank=rank, device="cpu", implementation="nccl", mcfg=c)
        w = ModelWeights.init(0, c, shard_fn=rt.shard_info)
        state = init_train_state(w, c, tcfg)
        st = Stepper(state, c, tcfg, device="cpu", rt=rt)
        data = np.load(tmp + "/batch.npy")                      # [A, 4, T] global batch
        xs = data[:, rank * 2:(rank + 1) * 2]
        ys = np.roll(xs, -1, axis=-1)
        out = None
        for step in range(2):
            out = st.train_step(xs, ys, step)
        torch.save({"loss": float(out["loss"]), "grad_norm": float(out["grad_norm"]),
                    "params": {p: t.detach().clone() for p, t in tree_dict(w).items() if t.numel()},
                    "owner": dict(rt.plan.owner), "expert": sorted(rt.plan.expert)}, f"{tmp}/rank{rank}.pt")
        save_checkpoint(Path(tmp) / "ckpt", 2, state, b'{"position": 0}', {"resume_signature": {}}, keep=1, rt=rt)
        restored = load_train_state(Path(tmp) / "ckpt", c, tcfg, rt=rt)
        a, b = tree_dict(state.params), tree_dict(restored.state.params)
        assert all(torch.equal(a[k], b[k]) for k in a)
    finally:
        dist.destroy_process_group()


def test_two_rank_step_matches_single_process(tmp_path):
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.checkpoints import load_leaf
    from lyra_b200.nn.params import ShardInfo, tree_dict
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper
    from lyra_b200.training.train import TrainingConfig

    c = _cfg()
    rng = np.random.default_rng(0)
    data = rng.integers(0, c.vocab_size, size=(2, 4, c.seq_len)).astype(np.int32)
    np.save(tmp_path / "batch.npy", data)
    port = free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)

    tcfg = TrainingConfig(steps=4, batch_size=4, accumulation_steps=2)
    w = ModelWeights.init(0, c)
    st = Stepper(init_train_state(w, c, tcfg), c, tcfg, device="cpu")
    for step in range(2):
        out = st.train_step(data, np.roll(data, -1, axis=-1), step)
    ref = tree_dict(w)
    ranks = [torch.load(tmp_path / f"rank{r}.pt", weights_only=False) for r in range(2)]
    assert abs(ranks[0]["loss"] - float(out["loss"])) < 1e-4 and abs(ranks[0]["grad_norm"] - float(out["grad_norm"])) < 1e-3 * float(out["grad_norm"])
    owner, experts = ranks[0]["owner"], set(ranks[0]["expert"])
    assert owner and experts and set(owner.values()) == {0, 1}
    el = c.n_experts // 2
    for p, full in ref.items():
        if p in experts:
            for r in range(2):
                assert torch.allclose(ranks[r]["params"][p], full[r * el:(r + 1) * el], atol=1.5e-3), p
        elif p in owner:
            assert p in ranks[owner[p]]["params"] and p not in ranks[1 - owner[p]]["params"]
            assert torch.allclose(ranks[owner[p]]["params"][p], full, atol=1.5e-3), p
        else:
            for r in range(2):
                assert torch.allclose(ranks[r]["params"][p], full, atol=1.5e-3), p
    # the checkpoint written by two ranks holds global arrays readable without the runtime
    ck = tmp_path / "ckpt" / "step_00000002" / "params"
    some_expert = next(iter(sorted(experts)))
    assert torch.allclose(load_leaf(ck, some_expert, ShardInfo()), ref[some_expert], atol=1.5e-3)
    some_dense = next(iter(sorted(owner)))
    assert torch.allclose(load_leaf(ck, some_dense, ShardInfo()), ref[some_dense], atol=1.5e-3)


def _serve_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.generate import BatchedGenerator
        from lyra_b200.model import ModelWeights
        from lyra_b200.parallel.runtime import Runtime

        c = replace(_cfg(), sample_temperature=0.0)
        rt = Runtime.create(world_size=world, rank=rank, device="cpu", implementation="nccl", mcfg=c)
        w = ModelWeights.init(0, c, shard_fn=rt.shard_info)
        rt.register(w)
        prompts = torch.from_numpy(np.load(tmp + "/prompts.npy"))[rank * 2:(rank + 1) * 2]      # this rank's rows of the batch
        gen = BatchedGenerator(w, c, batch=2, capacity=16, device="cpu", rt=rt)
        toks = gen.decode(gen.prefill(prompts), 6)
        torch.save(toks, f"{tmp}/serve{rank}.pt")
        # experts re-placed by the load of that request: the same request gives the same tokens afterwards
        from lyra_b200.nn.params import tree_dict

        assert rt.meter_expert_load(inference=True)
        gen.decode(gen.prefill(prompts), 6)
        report = rt.rebalance_experts(tree_dict(w), min_gain=0.0)
        assert report["layers_moved"] >= 1 and report["max_share_after"] <= report["max_share_before"]
        again = BatchedGenerator(w, c, batch=2, capacity=16, device="cpu", rt=rt)
        assert torch.equal(again.decode(again.prefill(prompts), 6), toks)
    finally:
        dist.destroy_process_group()


def test_expert_parallel_serving_matches_single_process(tmp_path):
    """Prefill + greedy decode with the experts sharded over two ranks (each rank serves its own rows, weights pulled from
    their owners) produces the tokens of the single-process generator."""
    from lyra_b200.generate import BatchedGenerator
    from lyra_b200.model import ModelWeights

    c = replace(_cfg(), sample_temperature=0.0)
    prompts = np.random.default_rng(1).integers(0, c.vocab_size, size=(4, 8)).astype(np.int64)
    np.save(tmp_path / "prompts.npy", prompts)
    port = free_port()
    mp.spawn(_serve_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    w = ModelWeights.init(0, c)
    gen = BatchedGenerator(w, c, batch=4, capacity=16, device="cpu")
    want = gen.decode(gen.prefill(torch.from_numpy(prompts)), 6)
    got = torch.cat([torch.load(tmp_path / f"serve{r}.pt") for r in range(2)])
    assert torch.equal(want, got)


def _tp_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.generate import BatchedGenerator
        from lyra_b200.model import ModelWeights, model_apply
        from lyra_b200.parallel.tp import TensorParallel

        c = replace(_cfg(), sample_temperature=0.0, use_qkv_bias=True, use_attn_out_bias=True, use_mlp_bias=True, use_sdpa_output_gate=True,
                    use_learned_xsa=True)
        tp = TensorParallel(c, rank, world)
        w = ModelWeights.init(3, c, shard_fn=tp.shard_info)
        _randomise_zero_init(w)
        prompts = torch.from_numpy(np.load(tmp + "/prompts.npy"))
        with torch.no_grad():
            logits, _, _ = model_apply(prompts, w, None, c, rt=tp)
        gen = BatchedGenerator(w, c, batch=prompts.shape[0], capacity=16, device="cpu", rt=tp)
        toks = gen.decode(gen.prefill(prompts), 5)
        torch.save({"logits": logits, "tokens": toks, "q_shape": tuple(w.layers[0].attn.q.shape),
                    "kv_cache": tuple(gen.cache.layers[0].k.shape)}, f"{tmp}/tp{rank}.pt")
    finally:
        dist.destroy_process_group()


def _randomise_zero_init(w):
    """Biases, sinks, gates and XSA strengths start at zero; give them values so that their sharding is exercised. Every rank
    derives the same full tensor from the leaf's path and takes its own slice, like the initialiser does."""
    rank, world = (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)
    _randomise_zero_init_on(w, rank, world)


def test_tensor_parallel_inference_matches_single_process(tmp_path):
    """Heads and hidden units split over two ranks (Megatron layout), one all-reduce per block: same logits and greedy tokens."""
    from lyra_b200.generate import BatchedGenerator
    from lyra_b200.model import ModelWeights, model_apply

    c = replace(_cfg(), sample_temperature=0.0, use_qkv_bias=True, use_attn_out_bias=True, use_mlp_bias=True, use_sdpa_output_gate=True,
                use_learned_xsa=True)
    prompts = np.random.default_rng(2).integers(0, c.vocab_size, size=(3, 8)).astype(np.int64)
    np.save(tmp_path / "prompts.npy", prompts)
    port = free_port()
    mp.spawn(_tp_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    w = ModelWeights.init(3, c)
    _randomise_zero_init(w)
    with torch.no_grad():
        want, _, _ = model_apply(torch.from_numpy(prompts), w, None, c)
    gen = BatchedGenerator(w, c, batch=3, capacity=16, device="cpu")
    tokens = gen.decode(gen.prefill(torch.from_numpy(prompts)), 5)
    for r in range(2):
        got = torch.load(tmp_path / f"tp{r}.pt")
        assert got["q_shape"][1] * 2 == w.layers[0].attn.q.shape[1]          # half of the query heads per rank
        assert got["kv_cache"][1] * 2 == c.n_kv_heads                          # and half of the kv heads in its cache
        live = want[..., : c.vocab_size]
        assert torch.allclose(got["logits"][..., : c.vocab_size], live, atol=2e-4, rtol=1e-4), (got["logits"][..., : c.vocab_size] - live).abs().max()
        assert torch.equal(got["tokens"], tokens)


def _tp_train_cfg():
    # the balance term is kept: every rank of the model axis routes the same rows, so it is the single-process term
    return replace(_cfg(), use_qkv_bias=True, use_attn_out_bias=True, use_mlp_bias=True, use_sdpa_output_gate=True, use_learned_xsa=True,
                   load_balance_weight=1e-2)


def _exact_newton_schulz():
    """Replaces the bf16 Newton-Schulz by a float64 one for a comparison: in bf16 a last-bit difference of a gradient (summation
    order across ranks) moves the result by percents, which would hide a real error of the sharding logic."""
    import lyra_b200.training.optimizer as O

    def ns(X, eps=1e-7):
        tall = X.shape[-2] > X.shape[-1]
        X = X.double()
        X = X / (1.01 * torch.linalg.matrix_norm(X, dim=(-2, -1), keepdim=True) + eps)
        X = X.transpose(-1, -2) if tall else X
        for a, b, c in O.POLAR_EXPRESS_COEFFS:
            A = X @ X.transpose(-1, -2)
            X = a * X + (b * A + c * (A @ A)) @ X
        return (X.transpose(-1, -2) if tall else X).float()

    O.newtonschulz = ns


def _tp_tcfg():
    from lyra_b200.training.train import TrainingConfig

    return TrainingConfig(steps=4, batch_size=2, accumulation_steps=2, muon_moment_dtype=torch.float32, adam_mu_dtype=torch.float32)


def _tp_train_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _exact_newton_schulz()
    try:
        from lyra_b200.model import ModelWeights
        from lyra_b200.nn.params import tree_dict
        from lyra_b200.parallel.tp import TensorParallel
        from lyra_b200.training.state import init_train_state, load_train_state, save_checkpoint
        from lyra_b200.training.steps import Stepper
        from lyra_b200.training.train import TrainingConfig

        c = _tp_train_cfg()
        tcfg = _tp_tcfg()
        tp = TensorParallel(c, rank, world)
        w = ModelWeights.init(3, c, shard_fn=tp.shard_info)
        _randomise_zero_init(w)
        state = init_train_state(w, c, tcfg)
        st = Stepper(state, c, tcfg, device="cpu", rt=tp)
        data = np.load(tmp + "/batch.npy")                      # every rank of the model axis sees all rows
        out = None
        for step in range(3):
            out = st.train_step(data, np.roll(data, -1, axis=-1), step)
        torch.save({"loss": float(out["loss"]), "grad_norm": float(out["grad_norm"]), "rms_max": float(out["muon_grad_rms_max"]),
                    "params": {p: t.detach().clone() for p, t in tree_dict(w).items()}}, f"{tmp}/tptrain{rank}.pt")
        save_checkpoint(Path(tmp) / "tpckpt", 3, state, b'{"position": 0}', {"resume_signature": {}}, keep=1, rt=tp)
        restored = load_train_state(Path(tmp) / "tpckpt", c, tcfg, rt=tp)
        a, b = tree_dict(state.params), tree_dict(restored.state.params)
        assert all(torch.equal(a[k], b[k]) for k in a)
        assert all(torch.equal(state.optimizer.muon_moment[k], restored.state.optimizer.muon_moment[k]) for k in state.optimizer.muon_moment)
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_training_matches_single_process(tmp_path):
    """Three optimizer steps with heads and hidden units split over two ranks: the same loss, gradient norm and parameters as
    one process (partial gradients summed where a replicated tensor enters sharded layers, Muon on gathered matrices), and a
    checkpoint that holds the global arrays."""
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.checkpoints import load_leaf
    from lyra_b200.nn.params import ShardInfo, tree_dict
    from lyra_b200.parallel.tp import TensorParallel
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper
    from lyra_b200.training.train import TrainingConfig

    c = _tp_train_cfg()
    data = np.random.default_rng(5).integers(0, c.vocab_size, size=(2, 2, c.seq_len)).astype(np.int32)
    np.save(tmp_path / "batch.npy", data)
    mp.spawn(_tp_train_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)

    import lyra_b200.training.optimizer as O

    tcfg = _tp_tcfg()
    w = ModelWeights.init(3, c)
    _randomise_zero_init(w)
    st = Stepper(init_train_state(w, c, tcfg), c, tcfg, device="cpu")
    bf16_ns = O.newtonschulz
    _exact_newton_schulz()
    try:
        for step in range(3):
            out = st.train_step(data, np.roll(data, -1, axis=-1), step)
    finally:
        O.newtonschulz = bf16_ns
    ref = tree_dict(w)
    ranks = [torch.load(tmp_path / f"tptrain{r}.pt", weights_only=False) for r in range(2)]
    for r in range(2):
        assert abs(ranks[r]["loss"] - float(out["loss"])) < 1e-4
        assert abs(ranks[r]["grad_norm"] - float(out["grad_norm"])) < 1e-3 * float(out["grad_norm"])
        assert abs(ranks[r]["rms_max"] - float(out["muon_grad_rms_max"])) < 1e-3 * float(out["muon_grad_rms_max"])
    sharded = 0
    for p, full in ref.items():
        for r in range(2):
            info = TensorParallel(c, r, 2)._info(p)
            sharded += bool(info.slices)
            assert torch.allclose(ranks[r]["params"][p], info.narrow(full), atol=3e-5), (p, (ranks[r]["params"][p] - info.narrow(full)).abs().max())
    assert sharded > 20
    ck = tmp_path / "tpckpt" / "step_00000003" / "params"
    for p in ("layers/1/attn/q", "layers/1/mlp/mlp_up", "layers/0/mlp/mlp_down", "layers/1/attn/qnorm_scale", "layers/1/attn/sinks"):
        assert torch.allclose(load_leaf(ck, p, ShardInfo()), ref[p], atol=3e-5), p


def _gpt_oss_cfg(**kw):
    from lyra_b200.config import ModelConfig

    return ModelConfig(name="Tiny GPT-OSS", seq_len=32, n_embd=64, n_layers=2, mlp_map=("moe", "moe"), vocab_size=201088, padded_vocab_size=201088,
                       head_dim=16, n_attn_heads=4, n_kv_heads=2, sliding_window=8, n_routed_experts=4, n_shared_experts=0, n_active_experts=2,
                       expert_mlp_widening=2.0, rope_scale=32.0, tie_embeddings=False, use_qk_norm=False, use_qkv_bias=True,
                       use_attn_out_bias=True, use_mlp_bias=True, use_router_bias=True, param_dtype=torch.bfloat16, compute_dtype=torch.float32,
                       implementation="torch", **kw)


def _chat(model, c, rt=None, fp8=False):
    from lyra_b200.generate import InferenceConfig, serve_model

    prompts = iter(["hello there", "and again", "exit"])
    printed = []
    terminal = dict(input_fn=lambda _: next(prompts), output_fn=lambda *a, **k: printed.append("".join(map(str, a))))
    if rt is not None:
        from lyra_b200.parallel.tp import shared_terminal

        terminal = shared_terminal(rt, **terminal)
    serve_model(model, c, InferenceConfig(weights="x", max_new_tokens=6, max_cache_length=32, fp8=fp8), device="cpu", rt=rt, **terminal)
    return printed


def _tp_chat_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.gpt_oss import load_gpt_oss_model
        from lyra_b200.parallel.tp import TensorParallel

        out = {}
        for name, c in (("greedy", _gpt_oss_cfg(sample_temperature=0.0)), ("sampled", _gpt_oss_cfg(sample_temperature=1.0, sample_topk=8))):
            tp = TensorParallel(c, rank, world)
            model = load_gpt_oss_model(tmp + "/ckpt", c, shard_fn=tp.shard_info)
            assert model.layers[0].attn.q.shape[1] == c.n_attn_heads * c.head_dim // world
            out[name] = _chat(model, c, tp)
        # block-scaled e4m3 expert weights and KV cache on top of the split: every rank quantises its own slice
        from lyra_b200.generate import InferenceConfig, apply_inference_overrides

        c8 = apply_inference_overrides(_gpt_oss_cfg(sample_temperature=0.0, quant_block=(16, 16)), InferenceConfig(weights="x", fp8=True))
        tp = TensorParallel(c8, rank, world)
        out["fp8"] = _chat(load_gpt_oss_model(tmp + "/ckpt", c8, shard_fn=tp.shard_info), c8, tp, fp8=True)
        torch.save(out, f"{tmp}/chat{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_chat_from_a_gpt_oss_checkpoint(tmp_path):
    """The serving loop on two ranks of a model axis: each rank reads its heads and hidden units from the GPT-OSS files, rank 0
    owns the terminal, and the greedy reply is the single-process reply."""
    from lyra_b200.gpt_oss import load_gpt_oss_model, write_random_gpt_oss_checkpoint

    c = _gpt_oss_cfg(sample_temperature=0.0)
    write_random_gpt_oss_checkpoint(tmp_path / "ckpt", c, seed=4)
    want = _chat(load_gpt_oss_model(tmp_path / "ckpt", c), c)
    mp.spawn(_tp_chat_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    rank0, rank1 = (torch.load(tmp_path / f"chat{r}.pt", weights_only=False) for r in range(2))
    assert rank0["greedy"] == want and len("".join(want)) > len("Type a prompt")
    assert rank1["greedy"] == [] and rank1["sampled"] == []            # the other rank prints nothing
    assert len(rank0["sampled"]) == len(want)                          # both turns ran with rank 0's sampled tokens fed to both ranks
    assert len(rank0["fp8"]) >= 4 and rank1["fp8"] == []               # the quantised model answered both turns


def _mesh_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _exact_newton_schulz()
    try:
        from lyra_b200.model import ModelWeights
        from lyra_b200.nn.params import tree_dict
        from lyra_b200.parallel.tp import TensorParallel
        from lyra_b200.training.state import init_train_state, save_checkpoint
        from lyra_b200.training.steps import Stepper

        c = replace(_tp_train_cfg(), load_balance_weight=0.0)   # a product of per-replica means: not additive over the data axis
        tcfg = replace(_tp_tcfg(), batch_size=4)
        tp = TensorParallel.mesh(c, rank, world, model_axis=2)
        assert (tp.data_size, tp.data_rank, tp.tp_rank) == (2, rank // 2, rank % 2)
        w = ModelWeights.init(3, c, shard_fn=tp.shard_info)
        _randomise_zero_init_on(w, tp.tp_rank, 2)
        state = init_train_state(w, c, tcfg)
        st = Stepper(state, c, tcfg, device="cpu", rt=tp)
        data = np.load(tmp + "/batch.npy")[:, tp.data_rank * 2:(tp.data_rank + 1) * 2]   # this replica's rows
        for step in range(2):
            out = st.train_step(data, np.roll(data, -1, axis=-1), step)
        torch.save({"loss": float(out["loss"]), "grad_norm": float(out["grad_norm"]),
                    "params": {p: t.detach().clone() for p, t in tree_dict(w).items()}}, f"{tmp}/mesh{rank}.pt")
        save_checkpoint(Path(tmp) / "meshckpt", 2, state, b'{"position": 0}', {"resume_signature": {}}, keep=1, rt=tp)
    finally:
        dist.destroy_process_group()


def _randomise_zero_init_on(w, tp_rank, tp_size):
    """``_randomise_zero_init`` for a given index on a model axis of ``tp_size`` ranks (which may differ from the global rank)."""
    import zlib

    from lyra_b200.nn.params import tree_dict
    from lyra_b200.parallel.tp import _COLUMNS, _ROWS, _VECTORS

    for path, t in tree_dict(w).items():
        name = path.split("/")[-1]
        if not (name.endswith("_bias") or name in ("sinks", "xsa_alpha", "sdpa_gate")):
            continue
        dim = 1 if name in _COLUMNS else 0 if (name in _ROWS or name in _VECTORS) else t.ndim - 1 if name == "mlp_up_bias" else None
        shape = list(t.shape)
        if dim is not None:
            shape[dim] *= tp_size
        full = torch.randn(shape, generator=torch.Generator().manual_seed(zlib.crc32(path.encode()))) * 0.1
        if dim is not None:
            n = full.shape[dim] // tp_size
            full = full.narrow(dim, tp_rank * n, n)
        t.data = t.data + full.to(t.dtype)


def test_data_by_model_mesh_training_matches_single_process(tmp_path):
    """Four ranks as two replicas of a two-rank model axis: rows split over the replicas, heads and hidden units over the axis."""
    import lyra_b200.training.optimizer as O
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.checkpoints import load_leaf
    from lyra_b200.nn.params import ShardInfo, tree_dict
    from lyra_b200.parallel.tp import TensorParallel
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper

    c = replace(_tp_train_cfg(), load_balance_weight=0.0)
    data = np.random.default_rng(6).integers(0, c.vocab_size, size=(2, 4, c.seq_len)).astype(np.int32)
    np.save(tmp_path / "batch.npy", data)
    mp.spawn(_mesh_worker, args=(4, free_port(), str(tmp_path)), nprocs=4, join=True)

    tcfg = replace(_tp_tcfg(), batch_size=4)
    w = ModelWeights.init(3, c)
    _randomise_zero_init_on(w, 0, 1)
    st = Stepper(init_train_state(w, c, tcfg), c, tcfg, device="cpu")
    bf16_ns = O.newtonschulz
    _exact_newton_schulz()
    try:
        for step in range(2):
            out = st.train_step(data, np.roll(data, -1, axis=-1), step)
    finally:
        O.newtonschulz = bf16_ns
    ref = tree_dict(w)
    for r in range(4):
        got = torch.load(tmp_path / f"mesh{r}.pt", weights_only=False)
        assert abs(got["loss"] - float(out["loss"])) < 1e-4 and abs(got["grad_norm"] - float(out["grad_norm"])) < 1e-3 * float(out["grad_norm"])
        for p, full in ref.items():
            want = TensorParallel(c, r % 2, 2)._info(p).narrow(full)
            assert torch.allclose(got["params"][p], want, atol=3e-5), (r, p, (got["params"][p] - want).abs().max())
    ck = tmp_path / "meshckpt" / "step_00000002" / "params"
    for p in ("layers/1/attn/q", "layers/1/mlp/mlp_up", "tok/emb"):
        assert torch.allclose(load_leaf(ck, p, ShardInfo()), ref[p], atol=3e-5), p


def _tp_scorer_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.evals import Scorer
        from lyra_b200.evals.common import Doc
        from lyra_b200.model import ModelWeights
        from lyra_b200.parallel.tp import TensorParallel

        c = _scorer_cfg()
        tp = TensorParallel(c, rank, world)
        scorer = Scorer(ModelWeights.init(0, c, shard_fn=tp.shard_info), c, batch_size=4, rt=tp)
        torch.save(scorer.score(_scorer_docs(Doc)), f"{tmp}/scores{rank}.pt")
    finally:
        dist.destroy_process_group()


def _scorer_cfg():
    from tests.helpers import small_config

    return small_config(vocab_size=201088, padded_vocab_size=204800, n_layers=2, mlp_map=("dense", "moe"), seq_len=64, n_attn_heads=4, n_kv_heads=2,
                        n_embd=64, head_dim=16, compute_dtype=torch.float32)


def _scorer_docs(Doc):
    return [Doc("Question: 1+1?\nAnswer:", ("2", "3", "4"), 0, True), Doc("Question: sky?\nAnswer:", ("blue", "green"), 0, True)]


def test_tensor_parallel_scoring_matches_single_process(tmp_path):
    """The loglikelihood harness on a model split over two ranks gives the single-process continuation scores on both ranks."""
    from lyra_b200.evals import Scorer
    from lyra_b200.evals.common import Doc
    from lyra_b200.model import ModelWeights

    c = _scorer_cfg()
    want = Scorer(ModelWeights.init(0, c), c, batch_size=4).score(_scorer_docs(Doc))
    mp.spawn(_tp_scorer_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(tmp_path / f"scores{r}.pt", weights_only=False)
        assert all(np.allclose(a, b, atol=1e-4) for a, b in zip(got, want)), (got, want)


def _fp8_moe_cfg():
    return replace(_cfg(), mlp_map=("moe",) * 4, sample_temperature=0.0, quantize_mlp=True, quantize_cache=True, gemm_dtype=torch.float8_e4m3fn,
                   quant_block=(16, 16))


def _fp8_serve_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lyra_b200.generate import BatchedGenerator
        from lyra_b200.model import ModelWeights
        from lyra_b200.nn.params import tree_dict
        from lyra_b200.nn.quant import QArray
        from lyra_b200.parallel.runtime import Runtime

        c = _fp8_moe_cfg()
        rt = Runtime.create(world_size=world, rank=rank, device="cpu", implementation="nccl", mcfg=c)
        w = ModelWeights.init(0, c, shard_fn=rt.shard_info)
        rt.register(w)
        w = ModelWeights.quantize(w, c)
        assert isinstance(w.layers[1].mlp.mlp_up, QArray)
        prompts = torch.from_numpy(np.load(tmp + "/prompts.npy"))[rank * 2:(rank + 1) * 2]
        gen = BatchedGenerator(w, c, batch=2, capacity=16, device="cpu", rt=rt)
        toks = gen.decode(gen.prefill(prompts), 6)
        torch.save(toks, f"{tmp}/fp8serve{rank}.pt")
        rt.meter_expert_load(inference=True)
        gen.decode(gen.prefill(prompts), 6)
        report = rt.rebalance_experts(tree_dict(w), min_gain=0.0)             # values and scales of the quantised stacks move together
        assert report["layers_moved"] >= 1
        again = BatchedGenerator(w, c, batch=2, capacity=16, device="cpu", rt=rt)
        assert torch.equal(again.decode(again.prefill(prompts), 6), toks)
    finally:
        dist.destroy_process_group()


def test_expert_parallel_fp8_serving_matches_single_process_and_survives_re_placement(tmp_path):
    """Block-scaled e4m3 experts (routed quantised, the shared expert from its bf16 copy) and an e4m3 KV cache, experts sharded
    over two ranks: the tokens of the single-process quantised model, before and after the experts change ranks."""
    from lyra_b200.generate import BatchedGenerator
    from lyra_b200.model import ModelWeights

    c = _fp8_moe_cfg()
    prompts = np.random.default_rng(3).integers(0, c.vocab_size, size=(4, 8)).astype(np.int64)
    np.save(tmp_path / "prompts.npy", prompts)
    mp.spawn(_fp8_serve_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    w = ModelWeights.quantize(ModelWeights.init(0, c), c)
    gen = BatchedGenerator(w, c, batch=4, capacity=16, device="cpu")
    want = gen.decode(gen.prefill(torch.from_numpy(prompts)), 6)
    got = torch.cat([torch.load(tmp_path / f"fp8serve{r}.pt") for r in range(2)])
    assert (want == got).float().mean() >= 0.9, (want, got)   # the shared expert runs unquantised under expert parallelism: near-ties may flip
