"""Training loop (lyra/training/train.py:160-292): data loader, resume guard, metrics / samples / numerics
logs, evaluation, sampling, checkpoints, hooks."""

from __future__ import annotations

import itertools
import json
import math
import shutil
import time
from contextlib import AbstractContextManager, nullcontext
from dataclasses import asdict, dataclass, field, replace
from pathlib import Path
from typing import Literal

import numpy as np
import torch

from lyra_b200.config import ModelConfig
from lyra_b200.data import DataLoader, DataLoaderConfig
from lyra_b200.model import ModelWeights
from lyra_b200.nn.checkpoints import checkpoint_path, checkpoint_run_config, checkpoint_steps, resolve_checkpoint
from lyra_b200.training.metrics import RULE, MetricsLogger, format_duration
from lyra_b200.training.plotting import plot_run
from lyra_b200.training.probe import Probe, to_floats
from lyra_b200.training.state import TrainState, init_train_state, load_train_state, save_checkpoint
from lyra_b200.training.steps import Stepper, run_validation

ROOT = Path(__file__).resolve().parents[2]
CHECKPOINT_DIR = ROOT / "chkpt"
DATA_DIR = ROOT / "data"
DEFAULT_SAMPLE_PROMPTS = (
    "The surprising thing about the ocean is",
    "To make a cup of tea, first",
    "In a small village by the sea,",
    "Here is a simple explanation of gravity:",
    "The history of astronomy begins with",
)
RUN_ARTIFACTS = ("metrics.jsonl", "samples.jsonl", "numerics.jsonl")
MODEL_FIELDS_IGNORED_ON_RESUME = ("w_init", "b_init", "norm_init", "mode", "sample_topk", "sample_temperature", "quantize_cache",
                                  "implementation", "sharding")
SCHEDULE_FIELDS = ("steps", "batch_size", "accumulation_steps", "decay_type", "warmup_fraction", "stable_fraction")


_RUN_COUNTER = itertools.count()


@dataclass(frozen=True, kw_only=True)
class TrainingConfig:
    # Schedule
    steps: int = 20000
    batch_size: int = 4
    accumulation_steps: int = 64
    decay_type: Literal["linear", "cosine"] = "cosine"
    warmup_fraction: float = 0.03
    stable_fraction: float = 0.0

    # Muon
    muon_max_lr: float = 1.5e-3
    muon_momentum: float = 0.95
    muon_update_rms: float = 0.2
    muon_wd: float = 0.1
    muon_nesterov: bool = True
    muon_grad_clip: float = 1.0
    muon_moment_dtype: torch.dtype = torch.bfloat16

    # Adam
    adam_max_lr: float = 2e-4
    adam_betas: tuple[float, float] = (0.90, 0.95)
    adam_mu_dtype: torch.dtype = torch.bfloat16
    adam_nu_dtype: torch.dtype = torch.float32

    # Data
    data_path: Path = DATA_DIR / "train"
    data_loader: DataLoaderConfig = field(default_factory=DataLoaderConfig)
    eval_data_path: Path | None = None
    eval_batches: int = 4

    log_every: int = 5
    eval_every: int | None = 500
    sample_every: int | None = None
    numerics_every: int | None = None
    checkpoint_every: int = 1000
    checkpoint_keep: int = 2
    peer_timeout_seconds: float = 600.0
    """Multi-rank runs: how long a rank waits at a step boundary for the others' heartbeat before it gives up (an addition; the reference has no failure detection)."""

    rebalance_experts_every: int | None = None
    """Expert-parallel runs: every this many steps the experts of each MoE layer are re-placed on the ranks by the token counts
    measured since the last time (an addition; None = static placement as in the reference)."""
    rebalance_min_gain: float = 0.05
    """A layer is re-placed only if its heaviest rank gets at least this much lighter."""

    sample_prompts: tuple[str, ...] = DEFAULT_SAMPLE_PROMPTS
    sample_tokens: int = 128
    checkpoint_path: Path = CHECKPOINT_DIR / "model"
    resume_from: Path | None = None

    @property
    def warmup_steps(self) -> int:
        return min(math.ceil(self.warmup_fraction * self.steps), self.steps - 1)

    @property
    def stable_steps(self) -> int:
        return round(self.stable_fraction * self.steps)

    @property
    def decay_steps(self) -> int:
        return self.steps - self.warmup_steps - self.stable_steps


def _jsonable(d: dict) -> dict:
    return json.loads(json.dumps(d, default=lambda o: str(o).replace("torch.", "")))


def resume_signature(mcfg: ModelConfig, tcfg: TrainingConfig, loader: DataLoader) -> dict:
    model = {k: v for k, v in mcfg.to_dict().items() if k not in MODEL_FIELDS_IGNORED_ON_RESUME}
    training = {k: v for k, v in asdict(tcfg).items() if k in SCHEDULE_FIELDS or k.startswith(("muon_", "adam_"))}
    data = {"tokens": loader.token_count, "shuffle": tcfg.data_loader.shuffle, "seed": tcfg.data_loader.seed}
    return _jsonable({"model": model, "training": training, "data": data})


def check_resume(path: Path, signature: dict) -> None:
    saved = checkpoint_run_config(path)["resume_signature"]
    differing = [section for section in signature if saved.get(section) != signature[section]]
    if differing:
        raise ValueError(f"The {' and '.join(differing)} settings differ from {path}. Resume with the original run configuration.")


@dataclass
class TrainHooks:
    """Attachment points of the loop. ``on_lowered`` / ``on_compiled`` are called once after the first
    (warm-up) step is built, with wall-clock timings; ``step_scope`` wraps every step (start a profiler
    window there); ``times_step`` opts a step into synchronous timing reported to ``after_step``."""

    compiler_options: dict | None = None

    def on_lowered(self, lowered) -> None:
        pass

    def on_compiled(self, compiled, timing: dict) -> None:
        pass

    def before_step(self, step: int, index: int, state: TrainState, xs: np.ndarray, ys: np.ndarray) -> None:
        pass

    def step_scope(self, step: int) -> AbstractContextManager:
        return nullcontext()

    def times_step(self, step: int) -> bool:
        return False

    def after_step(self, step: int, state: TrainState, aux: dict, step_time: float | None) -> None:
        pass

    def on_checkpoint(self, step: int, checkpoint_path: Path, run_path: Path) -> None:
        pass


def train(model: ModelWeights | None, mcfg: ModelConfig, tcfg: TrainingConfig, *, hooks: TrainHooks | None = None, rt=None,
          device=None) -> TrainState:
    hooks = hooks or TrainHooks()
    primary = rt is None or rt.rank == 0
    device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    out = checkpoint_path(tcfg.checkpoint_path)
    run_dir = out
    if primary:
        run_dir.mkdir(parents=True, exist_ok=True)
    if tcfg.resume_from is None and checkpoint_steps(out):
        raise FileExistsError(f"{out} already has checkpoints. Pass --resume, or choose another --out.")
    data_ranks = rt.data_size if rt is not None else 1
    if tcfg.batch_size % data_ranks:
        raise ValueError(f"--batch-size {tcfg.batch_size} must be a multiple of the {data_ranks} data-parallel devices.")
    local_batch = tcfg.batch_size // data_ranks

    # every rank reads its own rows of each global block
    loader = DataLoader(tcfg.data_path, tcfg.batch_size, mcfg.seq_len, config=tcfg.data_loader, quiet=not primary)
    loader.check_steps(tcfg.steps, tcfg.accumulation_steps)
    signature = resume_signature(mcfg, tcfg, loader)
    eval_loader = None
    if tcfg.eval_data_path is not None:
        eval_config = replace(tcfg.data_loader, shuffle=False, num_epochs=None, worker_count=1)
        eval_loader = DataLoader(tcfg.eval_data_path, tcfg.batch_size, mcfg.seq_len, config=eval_config, quiet=not primary)
        eval_start = eval_loader.get_state()

    def local_rows(a: np.ndarray) -> np.ndarray:
        if data_ranks == 1:
            return a
        r = rt.data_rank
        return a[..., r * local_batch:(r + 1) * local_batch, :]

    if tcfg.resume_from is None:
        assert model is not None, "a new run needs initial weights"
        start_step = 0
        state = init_train_state(model, mcfg, tcfg)
        if primary:
            for name in RUN_ARTIFACTS:
                (run_dir / name).unlink(missing_ok=True)
    else:
        path = resolve_checkpoint(tcfg.resume_from)
        check_resume(path, signature)
        restored = load_train_state(path, mcfg, tcfg, device=device, rt=rt)
        state, start_step = restored.state, restored.step
        loader.set_state(restored.loader_state)
        if primary:
            for name, text in checkpoint_run_config(path)["run_artifacts"].items():
                (run_dir / name).write_text(text)
            print(f"Resumed from {path} at step {start_step:,}")

    run_config = _jsonable({"model": mcfg.to_dict(), "training": asdict(tcfg), "resume_signature": signature})
    if primary:
        (run_dir / "config.json").write_text(json.dumps(run_config, indent=2))

    acc = tcfg.accumulation_steps
    tokens_per_step = acc * tcfg.batch_size * mcfg.seq_len
    build_start = time.perf_counter()
    stepper = Stepper(state, mcfg, tcfg, device=device, rt=rt)
    hooks.on_lowered(stepper)
    hooks.on_compiled(stepper, {"lower_seconds": 0.0, "xla_compile_seconds": 0.0, "total_seconds": time.perf_counter() - build_start})
    metrics = MetricsLogger(run_dir, tokens_per_step=tokens_per_step, initial_step=start_step, enabled=primary)

    def due(every: int | None, step: int) -> bool:
        return step == tcfg.steps or (every is not None and step % every == 0)

    def evaluate(step: int) -> None:
        eval_loader.set_state(eval_start)
        batches = ((local_rows(x), local_rows(y)) for x, y in eval_loader)
        metrics.log_eval(step, run_validation(stepper, batches, eval_batches=tcfg.eval_batches, microbatches=acc))

    if tcfg.sample_every is not None:
        from lyra_b200.generate import sample_eval_step
        from lyra_b200.tokenizer import LyraTokenizer

        tokenizer = LyraTokenizer()
        encoded = [[tokenizer.eos_token, *tokenizer.encode_ordinary(prompt)] for prompt in tcfg.sample_prompts]

        def sample(step: int) -> None:
            for index, (prompt, ids) in enumerate(zip(tcfg.sample_prompts, encoded)):
                tokens = sample_eval_step(state.params, ids, index, tcfg.sample_tokens, mcfg, device=device, rt=rt)
                completion = tokenizer.decode(tokens[: tokens.index(tokenizer.eos_token)] if tokenizer.eos_token in tokens else tokens)
                record = {"step": step, "total_tokens": step * tokens_per_step, "prompt": prompt, "completion": completion}
                if primary:
                    with (run_dir / "samples.jsonl").open("a") as stream:
                        stream.write(json.dumps(record, ensure_ascii=False) + "\n")
                    print(f"\n{RULE}\nstep {step:,} | {prompt}{completion}\n{RULE}\n")

    probe = Probe(routing_only=True) if tcfg.numerics_every is not None else None

    with metrics.paused():
        if eval_loader is not None:
            evaluate(start_step)
        if tcfg.sample_every is not None:
            sample(start_step)

    # With several ranks every step starts with a host-side roll call through the rendezvous store: a rank that died or left
    # is noticed before the next kernels (which would wait for it) are launched.
    heartbeat = None
    if rt is not None and rt.world > 1 and torch.distributed.is_available() and torch.distributed.is_initialized():
        from torch.distributed.distributed_c10d import _get_default_store

        from lyra_b200.parallel.health import Heartbeat

        # one key space per call of train() in this process group: the farewell of an earlier run must not read as a lost peer
        heartbeat = Heartbeat(_get_default_store(), rt.rank, rt.world, prefix=f"lyra/hb/{next(_RUN_COUNTER)}")

    rebalancing = tcfg.rebalance_experts_every is not None and rt is not None and rt.meter_expert_load()

    run_start = time.perf_counter()
    try:
        for step in range(start_step + 1, tcfg.steps + 1):
            if heartbeat is not None:
                heartbeat.beat(step)
                heartbeat.check(step, timeout=float(tcfg.peer_timeout_seconds))
            xs, ys = (np.stack(arrays) for arrays in zip(*(next(loader) for _ in range(acc))))
            xs, ys = local_rows(xs), local_rows(ys)
            if probe is not None and (step == 1 or due(tcfg.numerics_every, step)):
                record = {"kind": "step", "step": step, "records": to_floats(stepper.numerics_step(xs[:1], probe))}
                if primary:
                    with (run_dir / "numerics.jsonl").open("a") as stream:
                        stream.write(json.dumps(record) + "\n")

            hooks.before_step(step, step - 1, state, xs, ys)
            timed = hooks.times_step(step)
            step_start = time.perf_counter()
            with hooks.step_scope(step):
                aux = stepper.train_step(xs, ys, step - 1)
                if timed and device.type == "cuda":
                    torch.cuda.synchronize()
            metrics.record(aux)
            hooks.after_step(step, state, aux, time.perf_counter() - step_start if timed else None)
            if rebalancing and step % tcfg.rebalance_experts_every == 0 and step < tcfg.steps:
                moved = rt.rebalance_experts(stepper.params, state.optimizer, min_gain=tcfg.rebalance_min_gain)
                metrics.log_event("experts", step, moved)
                if primary and moved["layers_moved"]:
                    print(f"\n[experts] step {step:,}: re-placed {moved['layers_moved']} layers; heaviest rank's share of the tokens "
                          f"{moved['max_share_before']:.3f} -> {moved['max_share_after']:.3f} (balanced: {1 / rt.world:.3f})")

            checkpoint = due(tcfg.checkpoint_every, step)
            evaluating = eval_loader is not None and due(tcfg.eval_every, step)
            sampling = tcfg.sample_every is not None and due(tcfg.sample_every, step)
            if step == start_step + 1 or step % tcfg.log_every == 0 or checkpoint or evaluating:
                metrics.log_train(step)
            with metrics.paused() if checkpoint or evaluating or sampling else nullcontext():
                if checkpoint:
                    artifacts = {name: (run_dir / name).read_text() for name in RUN_ARTIFACTS if (run_dir / name).exists()}
                    save_checkpoint(out, step, state, loader.get_state(), run_config | {"run_artifacts": artifacts},
                                    keep=tcfg.checkpoint_keep, rt=rt)
                    hooks.on_checkpoint(step, out, run_dir)
                if evaluating:
                    evaluate(step)
                if sampling:
                    sample(step)
    finally:
        if heartbeat is not None:   # finished or failed: tell the others now, so that none of them waits out its time limit
            try:
                heartbeat.leave()
            except Exception:
                pass
        metrics.close()
        loader.close()
        if eval_loader is not None:
            eval_loader.close()

    if primary:
        plot_run(run_dir)
        print(f"{RULE}\nTraining finished in {format_duration(time.perf_counter() - run_start)}\n{RULE}")
    return state
