"""Training loop (lyra/training/train.py:160-292): data loader, resume guard, metrics / samples / numerics
logs, evaluation, sampling, checkpoints, hooks."""

from __future__ import annotations

import itertools
import json
import math
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
from lyra_b200.nn.checkpoints import checkpoint_path, checkpoint_run_config, checkpoint_steps, resolve_checkpoint, sync_remote
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


def check_device_status(device: torch.device) -> None:
    """Raises ``NativeError`` if a kernel on ``device`` has recorded a failure since the last check (CUDA devices only)."""
    if device.type == "cuda":
        from lyra_b200.ops import native

        native.check_status()


class _Periodic:
    """Decides which of the loop's side jobs fall on a step: a job is due on its own cadence and always on the last step."""

    def __init__(self, tcfg: TrainingConfig, first_step: int, has_eval: bool):
        self.t, self.first, self.has_eval = tcfg, first_step, has_eval

    def _every(self, every: int | None, step: int) -> bool:
        return step == self.t.steps or (every is not None and step % every == 0)

    def numerics(self, step: int) -> bool:
        return self.t.numerics_every is not None and (step == 1 or self._every(self.t.numerics_every, step))

    def checkpoint(self, step: int) -> bool:
        return self._every(self.t.checkpoint_every, step)

    def evaluation(self, step: int) -> bool:
        return self.has_eval and self._every(self.t.eval_every, step)

    def sampling(self, step: int) -> bool:
        return self.t.sample_every is not None and self._every(self.t.sample_every, step)

    def log_line(self, step: int) -> bool:
        return step == self.first or step % self.t.log_every == 0 or self.checkpoint(step) or self.evaluation(step)

    def rebalance(self, step: int) -> bool:
        every = self.t.rebalance_experts_every
        return every is not None and step % every == 0 and step < self.t.steps


class TrainingRun:
    """One run of the loop, built in the order the device-side state needs: data -> state (fresh or restored) -> ``Stepper``
    (which binds the sharding runtime to the parameter tree) -> logs. ``advance`` is one optimizer step plus whatever side
    jobs fall on it; ``close`` releases files and says goodbye to the other ranks. ``train`` below drives it.

    Behaviour follows lyra/training/train.py:160-292 (refusal to reuse a run directory, resume signature, artifacts restored
    from the checkpoint, throughput that leaves out evaluation / sampling / checkpoint time); the additions are the rank
    roll call at step boundaries, the kernel status check before anything is logged or saved, and expert re-placement."""

    def __init__(self, model: ModelWeights | None, mcfg: ModelConfig, tcfg: TrainingConfig, hooks: TrainHooks, rt, device):
        self.mcfg, self.tcfg, self.hooks, self.rt = mcfg, tcfg, hooks, rt
        self.primary = rt is None or rt.rank == 0
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.out = checkpoint_path(tcfg.checkpoint_path)
        if self.primary:
            self.out.mkdir(parents=True, exist_ok=True)
        if tcfg.resume_from is None and checkpoint_steps(self.out):
            raise FileExistsError(f"{self.out} already has checkpoints. Pass --resume, or choose another --out.")
        self.data_ranks = rt.data_size if rt is not None else 1
        if tcfg.batch_size % self.data_ranks:
            raise ValueError(f"--batch-size {tcfg.batch_size} must be a multiple of the {self.data_ranks} data-parallel devices.")
        self.local_batch = tcfg.batch_size // self.data_ranks
        self.tokens_per_step = tcfg.accumulation_steps * tcfg.batch_size * mcfg.seq_len
        self.heartbeat = self.metrics = self.loader = self.eval_loader = None
        try:
            self._open_data()
            self._open_state(model)
            self._open_stepper()
        except BaseException:
            self.close()
            raise

    def _open_stepper(self) -> None:
        mcfg, tcfg, hooks, rt = self.mcfg, self.tcfg, self.hooks, self.rt
        self.run_config = _jsonable({"model": mcfg.to_dict(), "training": asdict(tcfg), "resume_signature": self.signature})
        if self.primary:
            (self.out / "config.json").write_text(json.dumps(self.run_config, indent=2))
        built = time.perf_counter()
        self.stepper = Stepper(self.state, mcfg, tcfg, device=self.device, rt=rt)
        hooks.on_lowered(self.stepper)
        hooks.on_compiled(self.stepper, {"lower_seconds": 0.0, "xla_compile_seconds": 0.0, "total_seconds": time.perf_counter() - built})
        self.metrics = MetricsLogger(self.out, tokens_per_step=self.tokens_per_step, initial_step=self.start_step, enabled=self.primary)
        self.due = _Periodic(tcfg, self.start_step + 1, self.eval_loader is not None)
        self.probe = Probe(routing_only=True) if tcfg.numerics_every is not None else None
        self._sampler = self._build_sampler() if tcfg.sample_every is not None else None
        self.rebalancing = tcfg.rebalance_experts_every is not None and rt is not None and rt.meter_expert_load()
        self._join_roll_call()

    # ------------------------------------------------------------------ construction
    def _open_data(self) -> None:
        t = self.tcfg
        self.loader = DataLoader(t.data_path, t.batch_size, self.mcfg.seq_len, config=t.data_loader, quiet=not self.primary)
        self.loader.check_steps(t.steps, t.accumulation_steps)
        self.signature = resume_signature(self.mcfg, t, self.loader)
        if t.eval_data_path is not None:   # validation replays the same batches every time
            fixed = replace(t.data_loader, shuffle=False, num_epochs=None, worker_count=1)
            self.eval_loader = DataLoader(t.eval_data_path, t.batch_size, self.mcfg.seq_len, config=fixed, quiet=not self.primary)
            self._eval_start = self.eval_loader.get_state()

    def _open_state(self, model: ModelWeights | None) -> None:
        t = self.tcfg
        if t.resume_from is None:
            assert model is not None, "a new run needs initial weights"
            self.start_step, self.state = 0, init_train_state(model, self.mcfg, t)
            if self.primary:
                for name in RUN_ARTIFACTS:
                    (self.out / name).unlink(missing_ok=True)
            return
        path = resolve_checkpoint(t.resume_from)
        check_resume(path, self.signature)
        restored = load_train_state(path, self.mcfg, t, device=self.device, rt=self.rt)
        self.state, self.start_step = restored.state, restored.step
        self.loader.set_state(restored.loader_state)
        if self.primary:   # the logs are cut back to what the checkpoint had seen
            for name, text in checkpoint_run_config(path)["run_artifacts"].items():
                (self.out / name).write_text(text)
            print(f"Resumed from {path} at step {self.start_step:,}")

    def _build_sampler(self):
        from lyra_b200.generate import sample_eval_step
        from lyra_b200.tokenizer import LyraTokenizer

        tok = LyraTokenizer()
        prompts = [(text, [tok.eos_token, *tok.encode_ordinary(text)]) for text in self.tcfg.sample_prompts]

        def sample(step: int) -> None:
            for index, (text, ids) in enumerate(prompts):
                new = sample_eval_step(self.state.params, ids, index, self.tcfg.sample_tokens, self.mcfg, device=self.device, rt=self.rt)
                if tok.eos_token in new:
                    new = new[: new.index(tok.eos_token)]
                completion = tok.decode(new)
                self._append("samples.jsonl", {"step": step, "total_tokens": step * self.tokens_per_step, "prompt": text, "completion": completion},
                             ensure_ascii=False)
                if self.primary:
                    print(f"\n{RULE}\nstep {step:,} | {text}{completion}\n{RULE}\n")

        return sample

    def _join_roll_call(self) -> None:
        """Several ranks: every step starts with a host-side roll call through the rendezvous store, so a rank that died or left
        is noticed before kernels that would wait for it are launched."""
        rt = self.rt
        if rt is None or rt.world <= 1 or not (torch.distributed.is_available() and torch.distributed.is_initialized()):
            return
        from torch.distributed.distributed_c10d import _get_default_store

        from lyra_b200.parallel.health import Heartbeat

        # one key space per run in this process group: the farewell of an earlier run must not read as a lost peer
        self.heartbeat = Heartbeat(_get_default_store(), rt.rank, rt.world, prefix=f"lyra/hb/{next(_RUN_COUNTER)}")

    # ------------------------------------------------------------------ helpers
    def _append(self, name: str, record: dict, **json_kw) -> None:
        if self.primary:
            with (self.out / name).open("a") as stream:
                stream.write(json.dumps(record, **json_kw) + "\n")

    def _local_rows(self, a: np.ndarray) -> np.ndarray:
        if self.data_ranks == 1:
            return a
        r = self.rt.data_rank
        return a[..., r * self.local_batch:(r + 1) * self.local_batch, :]

    def _next_batch(self) -> tuple[np.ndarray, np.ndarray]:
        pairs = [next(self.loader) for _ in range(self.tcfg.accumulation_steps)]
        return self._local_rows(np.stack([x for x, _ in pairs])), self._local_rows(np.stack([y for _, y in pairs]))

    def device_health(self) -> None:
        """Kernels report a wait that ran out (a peer flag, a TMA stage) or an overflowing expert receive buffer through a
        status word instead of trapping; reading it synchronises, so it is read where the loop synchronises anyway. A bad
        status raises: the step's results are garbage and must reach neither the log nor a checkpoint."""
        check_device_status(self.device)

    # ------------------------------------------------------------------ side jobs
    def evaluate(self, step: int) -> None:
        self.eval_loader.set_state(self._eval_start)
        batches = ((self._local_rows(x), self._local_rows(y)) for x, y in self.eval_loader)
        result = run_validation(self.stepper, batches, eval_batches=self.tcfg.eval_batches, microbatches=self.tcfg.accumulation_steps)
        self.device_health()
        self.metrics.log_eval(step, result)

    def save(self, step: int) -> None:
        self.device_health()
        artifacts = {name: (self.out / name).read_text() for name in RUN_ARTIFACTS if (self.out / name).exists()}
        save_checkpoint(self.out, step, self.state, self.loader.get_state(), self.run_config | {"run_artifacts": artifacts},
                        keep=self.tcfg.checkpoint_keep, rt=self.rt)
        if self.primary:
            sync_remote(self.out)                              # a gs:// run directory is a local mirror: push the new checkpoint
        self.hooks.on_checkpoint(step, self.out, self.out)

    def replace_experts(self, step: int) -> None:
        moved = self.rt.rebalance_experts(self.stepper.params, self.state.optimizer, min_gain=self.tcfg.rebalance_min_gain)
        self.metrics.log_event("experts", step, moved)
        if self.primary and moved["layers_moved"]:
            print(f"\n[experts] step {step:,}: re-placed {moved['layers_moved']} layers; heaviest rank's share of the tokens "
                  f"{moved['max_share_before']:.3f} -> {moved['max_share_after']:.3f} (balanced: {1 / self.rt.world:.3f})")

    def before_first_step(self) -> None:
        with self.metrics.paused():
            if self.eval_loader is not None:
                self.evaluate(self.start_step)
            if self._sampler is not None:
                self._sampler(self.start_step)

    # ------------------------------------------------------------------ one step
    def advance(self, step: int) -> None:
        if self.heartbeat is not None:
            self.heartbeat.beat(step)
            self.heartbeat.check(step, timeout=float(self.tcfg.peer_timeout_seconds))
        xs, ys = self._next_batch()
        if self.probe is not None and self.due.numerics(step):
            self._append("numerics.jsonl", {"kind": "step", "step": step, "records": to_floats(self.stepper.numerics_step(xs[:1], self.probe))})

        hooks = self.hooks
        hooks.before_step(step, step - 1, self.state, xs, ys)
        timed = hooks.times_step(step)
        began = time.perf_counter()
        with hooks.step_scope(step):
            aux = self.stepper.train_step(xs, ys, step - 1)
            if timed and self.device.type == "cuda":
                torch.cuda.synchronize()
        self.metrics.record(aux)
        hooks.after_step(step, self.state, aux, time.perf_counter() - began if timed else None)
        if self.rebalancing and self.due.rebalance(step):
            self.replace_experts(step)

        saving, evaluating, sampling = self.due.checkpoint(step), self.due.evaluation(step), self.due.sampling(step)
        if self.due.log_line(step):
            self.device_health()
            self.metrics.log_train(step)
        if saving or evaluating or sampling:
            with self.metrics.paused():
                if saving:
                    self.save(step)
                if evaluating:
                    self.evaluate(step)
                if sampling:
                    self._sampler(step)

    def close(self, finished: bool = False) -> None:
        if self.heartbeat is not None:   # finished or failed: tell the others now, so that none of them waits out its time limit
            try:
                self.heartbeat.done() if finished else self.heartbeat.leave()
            except Exception:
                pass
        if self.metrics is not None:
            self.metrics.close()
        for loader in (self.loader, self.eval_loader):
            if loader is not None:
                loader.close()


def train(model: ModelWeights | None, mcfg: ModelConfig, tcfg: TrainingConfig, *, hooks: TrainHooks | None = None, rt=None,
          device=None) -> TrainState:
    """Runs (or resumes) training to ``tcfg.steps`` and returns the final state."""
    run = TrainingRun(model, mcfg, tcfg, hooks or TrainHooks(), rt, device)
    began = time.perf_counter()
    finished = False
    try:
        run.before_first_step()
        for step in range(run.start_step + 1, tcfg.steps + 1):
            run.advance(step)
        finished = True
    finally:
        run.close(finished)
    if run.primary:
        plot_run(run.out)
        sync_remote(run.out)                                   # logs, plot and the last checkpoint of a gs:// run
        print(f"{RULE}\nTraining finished in {format_duration(time.perf_counter() - began)}\n{RULE}")
    return run.state
