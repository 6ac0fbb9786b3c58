"""Tensor parallelism on two GPUs through the CUDA kernels: heads and hidden units split Megatron-style, so the per-rank
shapes are the awkward ones (360 hidden units per rank, as the GPT-OSS experts get on eight ranks: not a multiple of 64).
Logits of a prefill, a greedy decode and one optimizer step against the single-GPU run of the same model."""

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

    return ModelConfig(name="tp-test", seq_len=256, n_embd=720, n_layers=2, head_dim=64, n_attn_heads=8, n_kv_heads=4, rope_scale=1.0,
                       use_qk_norm=False, use_qkv_bias=True, use_attn_out_bias=True, use_mlp_bias=True, use_router_bias=True,
                       n_routed_experts=4, n_shared_experts=0, n_active_experts=2, mlp_map=("dense", "moe"), vocab_size=4000,
                       padded_vocab_size=4096, tie_embeddings=False, sample_temperature=0.0, load_balance_weight=1e-2)


def _tcfg():
    from lyra_b200.training.train import TrainingConfig

    return TrainingConfig(steps=4, batch_size=2, accumulation_steps=1)


def _inputs(c):
    rng = np.random.default_rng(11)
    prompts = rng.integers(0, c.vocab_size, size=(2, 64)).astype(np.int64)
    batch = rng.integers(0, c.vocab_size, size=(1, 2, c.seq_len)).astype(np.int32)
    return prompts, batch


def _run(c, rt, device):
    from lyra_b200.generate import BatchedGenerator
    from lyra_b200.model import ModelWeights, model_apply
    from lyra_b200.ops import native
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper

    prompts, batch = _inputs(c)
    w = ModelWeights.init(3, c, device=device, shard_fn=rt.shard_info if rt is not None else None)
    with torch.no_grad():
        logits, _, _ = model_apply(torch.from_numpy(prompts).to(device), w, None, c, rt=rt)
    gen = BatchedGenerator(w, c, batch=2, capacity=96, device=device, rt=rt, use_cuda_graph=False)
    tokens = gen.decode(gen.prefill(torch.from_numpy(prompts).to(device)), 6)
    st = Stepper(init_train_state(w, c, _tcfg()), c, _tcfg(), device=device, rt=rt)
    out = st.train_step(batch, np.roll(batch, -1, axis=-1), 0)
    torch.cuda.synchronize()
    native.check_status()
    return {"logits": logits[..., : c.vocab_size].float().cpu(), "tokens": tokens.cpu(), "loss": float(out["loss"]), "grad_norm": float(out["grad_norm"])}


def _worker(rank, world, port, tmp):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from lyra_b200.parallel.tp import TensorParallel

        c = _cfg()
        torch.save(_run(c, TensorParallel(c, rank, world), device), f"{tmp}/tp{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_on_two_gpus_matches_one_gpu(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    want = _run(_cfg(), None, torch.device("cuda", 0))
    for r in range(2):
        got = torch.load(tmp_path / f"tp{r}.pt", weights_only=False)
        err = ((got["logits"] - want["logits"]).norm() / want["logits"].norm()).item()
        assert err < 3e-2, err
        assert got["tokens"].shape == want["tokens"].shape
        assert abs(got["loss"] - want["loss"]) < 2e-2 * max(1.0, abs(want["loss"])), (got["loss"], want["loss"])
        assert abs(got["grad_norm"] - want["grad_norm"]) < 0.05 * want["grad_norm"], (got["grad_norm"], want["grad_norm"])
