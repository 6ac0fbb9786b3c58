"""Loglikelihood evaluation (MMLU, ARC-Challenge, ARC-Easy, HellaSwag) of a checkpoint."""

from __future__ import annotations

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

    device = "cuda" if (args.device == "gpu" or (args.device == "auto" and torch.cuda.is_available())) else "cpu"
    config = model_variant(args.variant)
    weights = args.weights or str(ROOT / "chkpt" / args.variant)
    model = load_gpt_oss_model(weights, config, device=device) if args.format == "gpt-oss" else ModelWeights.load(weights, config, device=device)
    scorer = Scorer(model, config, batch_size=args.batch_size, harmony=args.format == "gpt-oss", device=device)
    results = []
    for task in args.tasks:
        shots = args.fewshot.get(task, 0)
        docs = TASKS[task](limit=args.limit, num_fewshot=shots, fewshot_seed=args.fewshot_seed)
        print(f"Running {task} ({shots}-shot) on {len(docs)} documents...", flush=True)
        results.append(evaluate(task, docs, scorer))
        print(results[-1], flush=True)
    print("\nResults")
    for result in results:
        print(result)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
