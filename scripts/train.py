"""Pretraining entry point. Same flags as the reference CLI (scripts/train.py:13-85 there); launch one process per GPU
with ``python -m torch.distributed.run --nproc-per-node N scripts/train.py ...`` for multi-GPU runs."""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass, replace
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
    run: str | None = None
    """Training preset; defaults to the variant's (lyra-small -> train-small)."""
    device: Literal["auto", "cpu", "gpu"] = "auto"
    """Device."""
    implementation: Literal["auto", "b200", "torch", "nccl"] = "auto"
    """Kernel path: hand-written sm_100a kernels (auto / b200) or PyTorch + NCCL library ops (torch / nccl)."""
    print_config: bool = False
    """Print the resolved configuration and exit."""
    seed: int | None = None
    """Initialization and data seed."""
    steps: int | None = None
    """Total optimizer steps, including any already run."""
    batch_size: int | None = None
    """Sequences per microbatch."""
    acc_steps: int | None = None
    """Microbatches per optimizer step."""
    data: str | None = None
    """Training data."""
    eval_data: str | None = None
    """Validation data."""
    out: str | None = None
    """Checkpoint directory."""
    resume: str | None = None
    """Checkpoint, or run directory, to resume from; `auto` continues from the newest checkpoint in --out if there is one and
    starts a new run otherwise (the same command line then serves every restart of `torch.distributed.run --max-restarts`)."""
    eval_every: int | None = None
    """Validation interval in steps."""
    eval_batches: int | None = None
    """Validation batches per evaluation."""
    sample_every: int | None = None
    """Prompt sampling interval in steps."""
    sample_prompts: tuple[str, ...] | None = None
    """Prompts to sample."""
    numerics_every: int | None = None
    """Routing diagnostics interval in steps."""
    chkpt_every: int | None = None
    """Checkpoint interval in steps."""
    chkpt_keep: int | None = None
    """Checkpoints to keep."""
    decay_type: Literal["linear", "cosine"] | None = None
    """Learning-rate decay."""
    warmup_fraction: float | None = None
    """Fraction of steps spent warming up."""
    stable_fraction: float | None = None
    """Fraction of steps held at the peak learning rate."""
    adam_lr: float | None = None
    """Peak Adam learning rate."""
    muon_lr: float | None = None
    """Peak Muon learning rate."""
    grad_clip: float | None = None
    """Per-matrix Muon gradient RMS limit."""
    tensor_parallel: bool = False
    """Multi-rank runs: split heads and hidden units over the ranks of a model axis instead of leaf ownership + expert parallelism."""
    model_axis: int | None = None
    """With --tensor-parallel: ranks per model axis (default: all of them); the remaining factor of the ranks is data parallel."""
    rebalance_experts_every: int | None = None
    """Multi-GPU runs: re-place the experts on the ranks by measured token counts every this many steps."""


FIELDS = {
    "steps": "steps", "batch_size": "batch_size", "acc_steps": "accumulation_steps", "eval_every": "eval_every",
    "eval_batches": "eval_batches", "sample_every": "sample_every", "sample_prompts": "sample_prompts",
    "numerics_every": "numerics_every", "chkpt_every": "checkpoint_every", "chkpt_keep": "checkpoint_keep",
    "decay_type": "decay_type", "warmup_fraction": "warmup_fraction", "stable_fraction": "stable_fraction",
    "adam_lr": "adam_max_lr", "muon_lr": "muon_max_lr", "grad_clip": "muon_grad_clip",
    "rebalance_experts_every": "rebalance_experts_every",
}
PATH_FIELDS = {"data": "data_path", "eval_data": "eval_data_path", "out": "checkpoint_path", "resume": "resume_from"}


def training_config(args: Args):
    from lyra_b200.training.presets import TRAINING_PRESETS

    run = args.run or f"train-{args.variant.removeprefix('lyra-')}"
    if run not in TRAINING_PRESETS:
        raise SystemExit(f"error: no training preset {run!r}; pass --run (choices: {', '.join(TRAINING_PRESETS)})")
    config = TRAINING_PRESETS[run]
    overrides = {field: getattr(args, flag) for flag, field in FIELDS.items() if getattr(args, flag) is not None}
    overrides |= {field: Path(getattr(args, flag)).expanduser() for flag, field in PATH_FIELDS.items() if getattr(args, flag) is not None}
    if args.resume == "auto":
        from lyra_b200.nn.checkpoints import checkpoint_steps

        out = overrides.get("checkpoint_path", config.checkpoint_path)
        overrides["resume_from"] = out if (out.is_dir() and checkpoint_steps(out)) else None
    if args.seed is not None:
        overrides["data_loader"] = replace(config.data_loader, seed=args.seed)
    return replace(config, **overrides)


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    import torch

    from lyra_b200.model import ModelWeights
    from lyra_b200.training.train import train
    from lyra_b200.variants import model_variant

    tcfg = training_config(args)
    mcfg = replace(model_variant(args.variant), implementation=args.implementation)
    if args.seed is not None:
        mcfg = replace(mcfg, seed=args.seed)
    if args.print_config:
        from pprint import pprint

        pprint(mcfg)
        pprint(tcfg)
        return 0

    use_gpu = args.device == "gpu" or (args.device == "auto" and torch.cuda.is_available())
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rt = None
    if use_gpu:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1:
        import torch.distributed as dist

        from lyra_b200.parallel.runtime import Runtime

        dist.init_process_group("nccl" if use_gpu else "gloo")
    if world > 1 and args.tensor_parallel:
        from lyra_b200.parallel.tp import TensorParallel

        rt = TensorParallel.mesh(mcfg, dist.get_rank(), world, args.model_axis or world)
    elif world > 1:
        rt = Runtime.create(world_size=world, rank=dist.get_rank(), device=device,
                            implementation="nccl" if (args.implementation in ("torch", "nccl") or not use_gpu) else "b200", mcfg=mcfg)
    if rt is None or rt.rank == 0:
        print(f"Training {mcfg.name} for {tcfg.steps:,} steps")
    model = None
    if tcfg.resume_from is None:
        model = ModelWeights.init(mcfg.seed, mcfg, device=device, shard_fn=rt.shard_info if rt is not None else None)
    train(model, mcfg, tcfg, rt=rt, device=device)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
