"""Two ranks on two GPUs: the peer-memory ("b200") runtime against the collective ("nccl") runtime on the same model,
data and seeds: losses and updated parameters must agree; no kernel may report a failed wait."""

import os
import sys
from dataclasses import replace
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from tests.helpers import free_port  # noqa: E402

pytestmark = pytest.mark.gpu


def _cfg():
    from lyra_b200.config import ModelConfig

    return ModelConfig(name="dist-test", seq_len=512, n_embd=512, n_layers=4, head_dim=128, n_attn_heads=4, n_kv_heads=2,
                       use_learned_xsa=True, use_sdpa_output_gate=True, n_routed_experts=7, n_shared_experts=1, n_active_experts=3,
                       mlp_map=("dense", "moe", "dense", "moe"), vocab_size=4000, padded_vocab_size=4096, tie_embeddings=False)


def _worker(rank, world, port, tmp):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import lyra_b200.model as M
        from lyra_b200.model import ModelWeights
        from lyra_b200.nn.params import tree_dict
        from lyra_b200.ops import native
        from lyra_b200.parallel.runtime import Runtime
        from lyra_b200.training.state import init_train_state
        from lyra_b200.training.steps import Stepper
        from lyra_b200.training.train import TrainingConfig

        c = _cfg()
        tcfg = TrainingConfig(steps=4, batch_size=2 * world, accumulation_steps=2)
        rng = np.random.default_rng(rank)
        xs = rng.integers(0, c.vocab_size, size=(2, 2, c.seq_len)).astype(np.int32)
        ys = np.roll(xs, -1, axis=-1)
        results = {}
        # the second runtime takes the experts the first one chose (per layer call), so the comparison is between two ways of moving
        # the same tokens, gradients and weights, not between two sets of near-tie routing decisions
        M.ROUTING_TAPE = {"replay": False, "choices": []}
        for mode in ("nccl", "b200"):
            M.ROUTING_TAPE["replay"] = mode == "b200"
            rt = Runtime.create(world_size=world, rank=rank, device=device, implementation=mode, mcfg=c)
            w = ModelWeights.init(0, c, device=device, shard_fn=rt.shard_info)
            st = Stepper(init_train_state(w, c, tcfg), c, tcfg, device=device, rt=rt)
            init = {p: t.detach().float().cpu().clone() for p, t in tree_dict(w).items() if t.numel()}
            losses = []
            for step in range(2):
                out = st.train_step(xs, ys, step)
                losses.append(float(out["loss"]))
                if step == 0:
                    first = (float(out["grad_norm"]), {p: t.detach().float().cpu() - init[p] for p, t in tree_dict(w).items() if t.numel()})
            torch.cuda.synchronize()
            native.check_status()
            results[mode] = (losses, first)
        M.ROUTING_TAPE = None
        torch.save(results, f"{tmp}/rank{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_memory_runtime_matches_collective_runtime(tmp_path, world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"rank{r}.pt", weights_only=False)
        (l0, (g0, p0)), (l1, (g1, p1)) = res["nccl"], res["b200"]
        assert abs(l0[0] - l1[0]) < 2e-3 and abs(l0[1] - l1[1]) < 2e-2, (l0, l1)
        assert abs(g0 - g1) < 0.02 * g0, (g0, g1)
        assert p0.keys() == p1.keys()
        # the first update, leaf by leaf (small zero-initialised leaves take +-lr Adam steps whose sign is noise: skipped)
        cos = {k: torch.nn.functional.cosine_similarity(p0[k].reshape(-1), p1[k].reshape(-1), dim=0).item() for k in p0 if p0[k].numel() >= 4096}
        bad = {k: round(v, 4) for k, v in cos.items() if v < 0.98}
        assert cos and not bad, bad


def _ag_worker(rank, world, port, tmp):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from lyra_b200.ops import gemm as G, native
        from lyra_b200.parallel.comm import SymmetricSlab

        M, K, N = 1024, 2048, 1536
        g = torch.Generator(device="cuda").manual_seed(7)
        w_full = (torch.randn(K, N, device=device, generator=g) / 32).bfloat16()     # same on every rank
        x = torch.randn(M, K, device=device, generator=torch.Generator(device="cuda").manual_seed(rank)).bfloat16()
        slab = SymmetricSlab(K * N * 2, device, dist.group.WORLD.group_name)
        w_local = slab.view(0, K * N, torch.bfloat16).view(K, N)
        rows = K // world
        results = {}
        # (a) row-sharded: every rank owns K / world rows
        w_local.zero_()
        w_local[rank * rows:(rank + 1) * rows] = w_full[rank * rows:(rank + 1) * rows]
        torch.cuda.synchronize(); dist.barrier()
        flags = torch.zeros(64, dtype=torch.int32, device=device)
        src = [p + r * rows * N * 2 for r, p in enumerate(slab.peer_ptrs)]
        y = G.gemm_allgather(x, w_local, src, rank, rows, flags, epoch=1)
        torch.cuda.synchronize(); native.check_status()
        ref = x.float() @ w_full.float()
        results["rows"] = ((y.float() - ref).norm() / ref.norm()).item()
        results["rows_filled"] = bool(torch.equal(w_local, w_full))
        dist.barrier()
        # (b) single owner: rank 0 holds the whole matrix
        w_local.zero_()
        if rank == 0:
            w_local.copy_(w_full)
        torch.cuda.synchronize(); dist.barrier()
        y = G.gemm_allgather(x, w_local, [slab.peer_ptrs[0]], 0 if rank == 0 else 1, K, flags, epoch=2)
        torch.cuda.synchronize(); native.check_status()
        results["owner"] = ((y.float() - ref).norm() / ref.norm()).item()
        results["owner_filled"] = bool(torch.equal(w_local, w_full))
        dist.barrier()
        torch.save(results, f"{tmp}/ag{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_allgather_fused_gemm(tmp_path):
    import torch.multiprocessing as mp

    port = free_port()
    mp.spawn(_ag_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"ag{r}.pt", weights_only=False)
        assert res["rows"] < 1e-2 and res["owner"] < 1e-2, res
        assert res["rows_filled"] and res["owner_filled"], res


def _nvls_worker(rank, world, port, tmp):
    import ctypes

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from lyra_b200.ops import native
        from lyra_b200.parallel.comm import SymmetricSlab

        lib = native.kernels()
        n = 4 * world * 1000 + 4 * world          # a multiple of 4 x world
        slab = SymmetricSlab(n * 4, device, dist.group.WORLD.group_name)
        result = {"multicast": bool(slab.multicast_ptr)}
        if slab.multicast_ptr:
            mine = torch.randn(n, device=device, generator=torch.Generator(device="cuda").manual_seed(10 + rank))
            slab.view(0, n, torch.float32).copy_(mine)
            want = mine.clone()
            dist.all_reduce(want)                 # library sum as the oracle (same addends, possibly another order)
            torch.cuda.synchronize()
            dist.barrier()                        # every rank's copy is in place
            native.check(lib.lyra_multimem_all_reduce(ctypes.c_void_p(slab.multicast_ptr), ctypes.c_longlong(n), world, rank, native.stream_ptr()),
                         "multimem_all_reduce")
            torch.cuda.synchronize()
            dist.barrier()                        # every slice has been stored everywhere
            got = slab.view(0, n, torch.float32).clone()
            result["err"] = float((got - want).abs().max())
            result["scale"] = float(want.abs().max())
        torch.save(result, f"{tmp}/nvls{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_in_switch_all_reduce_of_a_small_buffer(tmp_path):
    """``multimem.ld_reduce`` / ``multimem.st`` over a symmetric allocation's multicast address against the library all-reduce.
    No rank leaves while the allocation is bound (the ranks exit together after the last barrier)."""
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_nvls_worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"nvls{r}.pt", weights_only=False)
        if not res["multicast"]:
            pytest.skip("no NVLink multicast support for symmetric allocations on this machine")
        assert res["err"] <= 1e-5 * max(1.0, res["scale"]), res
