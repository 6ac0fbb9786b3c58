"""Pretraining entry point. The flags are those of the reference's ``scripts/train.py`` (plus the multi-GPU ones at the end);
launch one process per GPU with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 scripts/train.py ...``
for multi-GPU runs. Every flag left unset keeps the value of the training preset."""

from __future__ import annotations

import os
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Literal

import tyro

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # load kernels with the library, not at first launch (multi-rank waits)

try:
    from scripts._launch import ROOT, place
except ImportError:                        # run as a file: scripts/ itself is the import root
    from _launch import ROOT, place


@dataclass(frozen=True)
class Args:
    variant: str = "lyra-small"
    """Model variant to train (see lyra_b200/variants.py)."""
    run: str | None = None
    """Training preset to start from; by default the one named after the variant (lyra-small -> train-small)."""
    device: Literal["auto", "cpu", "gpu"] = "auto"
    """auto takes a GPU when there is one."""
    implementation: Literal["auto", "b200", "torch", "nccl"] = "auto"
    """Kernel path: hand-written sm_100a kernels (auto / b200) or PyTorch + NCCL library ops (torch / nccl)."""
    print_config: bool = False
    """Show the model and training configuration that would be used, then stop."""
    seed: int | None = None
    """Seed of the weight initialisation and of the data order."""
    steps: int | None = None
    """Optimizer steps of the whole run (a resumed run counts the steps it already made)."""
    batch_size: int | None = None
    """Sequences in one microbatch (all data-parallel ranks together)."""
    acc_steps: int | None = None
    """Microbatches whose gradients are accumulated into one optimizer step."""
    data: str | None = None
    """Training tokens: a .npy file or a directory of ArrayRecord shards."""
    eval_data: str | None = None
    """Held-out tokens for the periodic evaluation, same formats."""
    out: str | None = None
    """Run directory: checkpoints, metrics.jsonl, samples and plots go here."""
    resume: str | None = None
    """Checkpoint, or run directory, to resume from; `auto` continues from the newest checkpoint in --out if there is one and
    starts a new run otherwise (the same command line then serves every restart of `torch.distributed.run --max-restarts`)."""
    eval_every: int | None = None
    """Evaluate on the held-out data every this many steps."""
    eval_batches: int | None = None
    """Batches read from the held-out data per evaluation."""
    sample_every: int | None = None
    """Generate from the sample prompts every this many steps."""
    sample_prompts: tuple[str, ...] | None = None
    """Prompts for those samples."""
    numerics_every: int | None = None
    """Write router and activation statistics (numerics.jsonl) every this many steps."""
    chkpt_every: int | None = None
    """Save a checkpoint every this many steps (and always at the end)."""
    chkpt_keep: int | None = None
    """Number of most recent checkpoints that are kept."""
    decay_type: Literal["linear", "cosine"] | None = None
    """Shape of the learning-rate decay after the stable phase."""
    warmup_fraction: float | None = None
    """Share of the steps in which the learning rates ramp up."""
    stable_fraction: float | None = None
    """Share of the steps at the peak learning rates."""
    adam_lr: float | None = None
    """Peak learning rate of the Adam group (embeddings, biases, scalars)."""
    muon_lr: float | None = None
    """Peak learning rate of the Muon group (matrices)."""
    grad_clip: float | None = None
    """Muon clips each matrix's gradient to this RMS."""
    tensor_parallel: bool = False
    """Multi-rank runs: split heads and hidden units over the ranks of a model axis instead of leaf ownership + expert parallelism."""
    model_axis: int | None = None
    """With --tensor-parallel: ranks per model axis (default: all of them); the remaining factor of the ranks is data parallel."""
    rebalance_experts_every: int | None = None
    """Multi-GPU runs: re-place the experts on the ranks by measured token counts every this many steps."""


# flag -> field of TrainingConfig, for the flags whose value is taken as it is
_PLAIN = (("steps", "steps"), ("batch_size", "batch_size"), ("acc_steps", "accumulation_steps"), ("eval_every", "eval_every"),
          ("eval_batches", "eval_batches"), ("sample_every", "sample_every"), ("sample_prompts", "sample_prompts"),
          ("numerics_every", "numerics_every"), ("chkpt_every", "checkpoint_every"), ("chkpt_keep", "checkpoint_keep"),
          ("decay_type", "decay_type"), ("warmup_fraction", "warmup_fraction"), ("stable_fraction", "stable_fraction"),
          ("adam_lr", "adam_max_lr"), ("muon_lr", "muon_max_lr"), ("grad_clip", "muon_grad_clip"),
          ("rebalance_experts_every", "rebalance_experts_every"))
# flag -> field, for the flags that name a place on disk (``~`` is expanded)
_PLACES = (("data", "data_path"), ("eval_data", "eval_data_path"), ("out", "checkpoint_path"), ("resume", "resume_from"))


def preset_of(args: Args):
    from lyra_b200.training.presets import TRAINING_PRESETS

    name = args.run if args.run is not None else "train-" + args.variant.removeprefix("lyra-")
    try:
        return TRAINING_PRESETS[name]
    except KeyError:
        raise SystemExit(f"error: there is no training preset {name!r} (known: {', '.join(TRAINING_PRESETS)}); name one with --run") from None


def training_config(args: Args):
    """The preset with every flag that was given laid over it."""
    preset = preset_of(args)
    changed = {}
    for flag, name in _PLAIN:
        value = getattr(args, flag)
        if value is not None:
            changed[name] = value
    for flag, name in _PLACES:
        value = getattr(args, flag)
        if value is not None:
            changed[name] = Path(value).expanduser()
    if args.resume == "auto":             # continue the run in --out if it has a checkpoint, start it otherwise
        from lyra_b200.nn.checkpoints import checkpoint_steps

        run_dir = changed.get("checkpoint_path", preset.checkpoint_path)
        changed["resume_from"] = run_dir if run_dir.is_dir() and checkpoint_steps(run_dir) else None
    if args.seed is not None:
        changed["data_loader"] = replace(preset.data_loader, seed=args.seed)
    return replace(preset, **changed)


def sharding_runtime(args: Args, where, mcfg, device):
    """Several processes: tensor parallelism on request, otherwise leaf ownership + expert parallelism."""
    if where.world == 1:
        return None
    import torch.distributed as dist

    dist.init_process_group("nccl" if where.on_gpu else "gloo")
    if args.tensor_parallel:
        from lyra_b200.parallel.tp import TensorParallel

        return TensorParallel.mesh(mcfg, dist.get_rank(), where.world, args.model_axis or where.world)
    from lyra_b200.parallel.runtime import Runtime

    library_paths = args.implementation in ("torch", "nccl") or not where.on_gpu
    return Runtime.create(world_size=where.world, rank=dist.get_rank(), device=device, implementation="nccl" if library_paths else "b200", mcfg=mcfg)


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

        for config in (mcfg, tcfg):
            pprint(config)
        return 0

    where = place(args.device)
    device = torch.device(where.device)
    rt = sharding_runtime(args, where, mcfg, device)
    if rt is None or rt.rank == 0:
        print(f"{mcfg.name}: {tcfg.steps:,} optimizer steps on {where.world} process(es), run directory {tcfg.checkpoint_path}")
    fresh = tcfg.resume_from is None
    model = ModelWeights.init(mcfg.seed, mcfg, device=device, shard_fn=rt.shard_info if rt is not None else None) if fresh else None
    train(model, mcfg, tcfg, rt=rt, device=device)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
