"""Loglikelihood evaluation (MMLU, ARC-Challenge, ARC-Easy, HellaSwag) of a checkpoint."""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Literal

import tyro

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


@dataclass(frozen=True)
class Args:
    variant: str = "lyra-small"
    """Model variant."""
    weights: str | None = None
    """Checkpoint path; defaults to chkpt/<variant>."""
    tasks: tuple[Literal["mmlu", "arc-challenge", "arc-easy", "hellaswag"], ...] = ("mmlu", "arc-challenge", "arc-easy", "hellaswag")
    """Evaluation tasks."""
    format: Literal["orbax", "gpt-oss"] = "orbax"
    """Checkpoint format."""
    device: Literal["auto", "cpu", "gpu"] = "auto"
    """Device."""
    batch_size: int = 8
    """Sequences per forward pass."""
    limit: int | None = None
    """Maximum documents per task."""
    fewshot: dict[str, int] = field(default_factory=dict)
    """Few-shot examples per task; tasks not listed are zero-shot."""
    fewshot_seed: int = 1234
    """Seed for choosing ARC and HellaSwag few-shot examples."""


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    import torch

    from lyra_b200.evals import TASKS, Scorer, evaluate
    from lyra_b200.gpt_oss import load_gpt_oss_model
    from lyra_b200.model import ModelWeights
    from lyra_b200.variants import model_variant

    use_gpu = args.device == "gpu" or (args.device == "auto" and torch.cuda.is_available())
    world, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    if use_gpu:
        torch.cuda.set_device(local)
    device = f"cuda:{local}" if use_gpu else "cpu"
    config = model_variant(args.variant)
    weights = args.weights or str(ROOT / "chkpt" / args.variant)
    rt = None
    if world > 1:   # under torch.distributed.run the model is split tensor-parallel; every rank scores the same documents
        import torch.distributed as dist

        from lyra_b200.parallel.tp import TensorParallel

        dist.init_process_group("nccl" if use_gpu else "gloo")
        rt = TensorParallel(config, dist.get_rank(), world)
    say = print if rt is None or rt.rank == 0 else (lambda *a, **k: None)
    if args.format == "gpt-oss":
        model = load_gpt_oss_model(weights, config, device=device, shard_fn=rt.shard_info if rt is not None else None)
    else:
        model = ModelWeights.load(weights, config, device=device, rt=rt)
    scorer = Scorer(model, config, batch_size=args.batch_size, harmony=args.format == "gpt-oss", device=device, rt=rt)
    results = []
    for task in args.tasks:
        shots = args.fewshot.get(task, 0)
        docs = TASKS[task](limit=args.limit, num_fewshot=shots, fewshot_seed=args.fewshot_seed)
        say(f"Running {task} ({shots}-shot) on {len(docs)} documents...", flush=True)
        results.append(evaluate(task, docs, scorer))
        say(results[-1], flush=True)
    say("\nResults")
    for result in results:
        say(result)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
