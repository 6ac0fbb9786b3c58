"""Multiple-choice evaluation of a checkpoint by continuation log-likelihood: MMLU, ARC-Challenge, ARC-Easy, HellaSwag.

Flags follow the reference's ``scripts/evals.py``. Launched under ``python -m torch.distributed.run --nproc-per-node N``
the model is split tensor-parallel over the N processes and every process scores the same documents; the first one
reports."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

import tyro

try:
    from scripts._launch import default_weights, join_tensor_parallel, place
except ImportError:                        # run as a file: scripts/ itself is the import root
    from _launch import default_weights, join_tensor_parallel, place

TaskName = Literal["mmlu", "arc-challenge", "arc-easy", "hellaswag"]


@dataclass(frozen=True)
class Args:
    variant: str = "lyra-small"
    """Which model variant the checkpoint belongs to."""
    weights: str | None = None
    """Checkpoint (or run) directory; chkpt/<variant> when omitted."""
    tasks: tuple[TaskName, ...] = ("mmlu", "arc-challenge", "arc-easy", "hellaswag")
    """Tasks to run, in this order."""
    format: Literal["orbax", "gpt-oss"] = "orbax"
    """orbax: a checkpoint written by scripts/train.py; gpt-oss: an original/ GPT-OSS checkpoint (Harmony prompts)."""
    device: Literal["auto", "cpu", "gpu"] = "auto"
    """auto takes a GPU when there is one."""
    batch_size: int = 8
    """Continuations scored per forward pass."""
    limit: int | None = None
    """Score only the first N documents of each task."""
    fewshot: dict[str, int] = field(default_factory=dict)
    """Number of in-context examples per task, e.g. --fewshot mmlu=5; unlisted tasks get none."""
    fewshot_seed: int = 1234
    """Seed of the draw of ARC and HellaSwag in-context examples."""


def open_model(args: Args, where, config):
    from lyra_b200.gpt_oss import load_gpt_oss_model
    from lyra_b200.model import ModelWeights

    source = args.weights or default_weights(args.variant)
    if args.format == "gpt-oss":
        return load_gpt_oss_model(source, config, device=where.device, shard_fn=where.shard_fn)
    return ModelWeights.load(source, config, device=where.device, rt=where.runtime)


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    from lyra_b200.evals import TASKS, Scorer, evaluate
    from lyra_b200.variants import model_variant

    config = model_variant(args.variant)
    where = join_tensor_parallel(place(args.device), config)
    scorer = Scorer(open_model(args, where, config), config, batch_size=args.batch_size, harmony=args.format == "gpt-oss",
                    device=where.device, rt=where.runtime)
    summary = []
    for name in args.tasks:
        shots = args.fewshot.get(name, 0)
        documents = TASKS[name](limit=args.limit, num_fewshot=shots, fewshot_seed=args.fewshot_seed)
        where.say(f"[{name}] {len(documents)} documents, {shots}-shot ...", flush=True)
        outcome = evaluate(name, documents, scorer)
        where.say(f"[{name}] {outcome}", flush=True)
        summary.append(outcome)
    where.say("\nSummary")
    for outcome in summary:
        where.say(f"  {outcome}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
