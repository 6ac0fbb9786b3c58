"""Chat with a checkpoint (own Orbax-layout checkpoints or GPT-OSS ``original/`` checkpoints).

Under ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 scripts/serve.py ...`` the model is split
over the N ranks tensor-parallel (heads and hidden units; a model that does not fit one GPU): rank 0 owns the terminal, reads
the prompt and prints the reply, the others receive the prompt and take part in every model call."""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Literal

import tyro

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # load kernels with the library, not at first launch (multi-rank waits)

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


@dataclass(frozen=True)
class Args:
    variant: str = "lyra-small"
    """Model variant."""
    weights: str | None = None
    """Checkpoint path; defaults to chkpt/<variant>."""
    format: Literal["orbax", "gpt-oss"] = "orbax"
    """Checkpoint format."""
    device: Literal["auto", "cpu", "gpu"] = "auto"
    """Device."""
    max_new_tokens: int = 256
    """Tokens to generate per turn."""
    max_cache_length: int | None = None
    """Prompt plus generation length; defaults to the model's context length."""
    temperature: float | None = None
    """Sampling temperature; defaults to the variant's."""
    top_k: int | None = None
    """Top-k sampling; defaults to the variant's."""
    fp8: bool = False
    """Store MLP weights and the KV cache in block-scaled FP8."""


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    import torch

    from lyra_b200.generate import InferenceConfig, apply_inference_overrides, load_model, serve_model
    from lyra_b200.gpt_oss import load_gpt_oss_model
    from lyra_b200.variants import model_variant

    use_gpu = args.device == "gpu" or (args.device == "auto" and torch.cuda.is_available())
    world, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    if use_gpu:
        torch.cuda.set_device(local)
    device = f"cuda:{local}" if use_gpu else "cpu"
    icfg = InferenceConfig(weights=args.weights or str(ROOT / "chkpt" / args.variant), max_new_tokens=args.max_new_tokens,
                           max_cache_length=args.max_cache_length, temperature=args.temperature, top_k=args.top_k, fp8=args.fp8)
    mcfg = apply_inference_overrides(model_variant(args.variant), icfg)
    rt, io = None, {}
    if world > 1:
        import torch.distributed as dist

        from lyra_b200.parallel.tp import TensorParallel, shared_terminal

        dist.init_process_group("nccl" if use_gpu else "gloo")
        rt = TensorParallel(mcfg, dist.get_rank(), world)
        io = shared_terminal(rt)
    if args.format == "gpt-oss":
        model = load_gpt_oss_model(icfg.weights, mcfg, device=device, shard_fn=rt.shard_info if rt is not None else None)
    else:
        model = load_model(mcfg, icfg, device=device, rt=rt)
    serve_model(model, mcfg, icfg, harmony=args.format == "gpt-oss", device=device, rt=rt, **io)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
