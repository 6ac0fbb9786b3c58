"""Run logging: ``metrics.jsonl`` rows and the console table.

The file format is the reference's (lyra/training/metrics.py:15-78): ``{"kind": "train", "step", <step metrics averaged
over the logging window>, "perplexity", "step_time", "tps", "total_tokens"}`` and ``{"kind": "eval", "step", "eval_*"}``.
How it is produced is this framework's own: a step's metrics stay on the device as tensors; when a line is due each
metric's window is averaged on the device and all of them cross to the host in one copy, so a step costs no
synchronisation and a log line costs one. Time spent in evaluation, sampling and checkpointing is taken out of the
window by a stopwatch that can be held, so ``step_time`` and ``tps`` describe training steps only."""

from __future__ import annotations

import json
import math
import time
from contextlib import contextmanager
from pathlib import Path

import torch

RULE = "─" * 60
PPL_CE_CLAMP = 20.0


def format_duration(seconds: float) -> str:
    minutes, secs = divmod(int(seconds), 60)
    hours, minutes = divmod(minutes, 60)
    return f"{hours}h {minutes}m {secs}s" if hours else f"{minutes}m {secs}s" if minutes else f"{seconds:.1f}s"


def _tokens(v: float) -> str:
    return f"{v / 1e9:.3f}B" if v >= 1e9 else f"{v / 1e6:.3f}M"


class _Table:
    """Fixed-width console table: (record key, heading, formatter) per column; the heading is printed before the first row."""

    COLUMNS = (
        ("step", "step", lambda v: f"{int(v):,}"),
        ("loss", "loss", lambda v: f"{v:.4f}"),
        ("ce_loss", "ce_loss", lambda v: f"{v:.4f}"),
        ("aux_loss", "aux", lambda v: f"{v:.4f}"),
        ("perplexity", "ppl", lambda v: f"{v:,.0f}"),
        ("step_time", "step_ms", lambda v: f"{v * 1e3:.1f}"),
        ("tps", "tok/s", lambda v: f"{v:,.0f}"),
        ("total_tokens", "tokens", _tokens),
    )

    def __init__(self) -> None:
        self.started = False

    def row(self, record: dict) -> None:
        if not self.started:
            print("  ".join(heading.ljust(8) for _, heading, _ in self.COLUMNS))
            self.started = True
        print("  ".join(fmt(record[key]).ljust(8) for key, _, fmt in self.COLUMNS))




class _Stopwatch:
    """Wall time since the last ``lap`` that was not spent inside ``hold``."""

    def __init__(self) -> None:
        self.origin = time.perf_counter()

    @staticmethod
    def _drain() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @contextmanager
    def hold(self):
        self._drain()                       # queued training work belongs to the window, not to what runs inside the hold
        entered = time.perf_counter()
        try:
            yield
        finally:
            self._drain()
            self.origin += time.perf_counter() - entered

    def lap(self) -> float:
        now = time.perf_counter()
        elapsed, self.origin = now - self.origin, now
        return elapsed


def _window_means(window: list[dict]) -> dict[str, float]:
    """Mean of every metric over the window. Tensors are averaged where they live and fetched together."""
    keys = list(window[0])
    tensors = [k for k in keys if isinstance(window[0][k], torch.Tensor)]
    means = {k: sum(float(row[k]) for row in window) / len(window) for k in keys if k not in tensors}
    if tensors:
        device = next((window[0][k].device for k in tensors if window[0][k].is_cuda), torch.device("cpu"))
        stacked = torch.stack([torch.stack([row[k].detach().to(device=device, dtype=torch.float64).reshape(()) for row in window]).mean() for k in tensors])
        means.update(zip(tensors, stacked.tolist()))          # the one device -> host copy of the log line
    return {k: means[k] for k in keys}


class MetricsLogger:
    def __init__(self, run_dir: Path, tokens_per_step: int = 0, initial_step: int = 0, enabled: bool = True):
        self.tokens_per_step = tokens_per_step
        self.total_tokens = initial_step * tokens_per_step
        self.enabled = enabled
        self.file = (Path(run_dir) / "metrics.jsonl").open("a") if enabled else None
        self.window: list[dict] = []
        self.clock = _Stopwatch()
        self.table = _Table()

    # ------------------------------------------------------------------ training steps
    def record(self, aux: dict) -> None:
        self.window.append(aux)
        self.total_tokens += self.tokens_per_step

    def log_train(self, step: int) -> None:
        steps = len(self.window)
        if not steps:
            return
        record = {"kind": "train", "step": step} | _window_means(self.window)     # synchronises: do it before reading the clock
        elapsed = self.clock.lap()
        record["perplexity"] = math.exp(min(record["ce_loss"], PPL_CE_CLAMP))
        record["step_time"] = elapsed / steps
        record["tps"] = self.tokens_per_step * steps / elapsed
        record["total_tokens"] = self.total_tokens
        self.window = []
        if self.enabled:
            self.table.row(record)
            self._write(record)

    def paused(self):
        """Leave evaluation, sampling and checkpointing out of the step time and throughput."""
        return self.clock.hold()

    # ------------------------------------------------------------------ other rows
    def log_eval(self, step: int, metrics: dict) -> None:
        record = {"kind": "eval", "step": step} | {k: float(v) for k, v in metrics.items()}
        if self.enabled:
            print(f"eval | step {step:,} | loss {record['eval_loss']:.4f} | ce_loss {record['eval_ce_loss']:.4f}")
            self._write(record)

    def log_event(self, kind: str, step: int, fields: dict) -> None:
        """A row of another kind (e.g. ``experts``: one expert re-placement) for tools that read ``metrics.jsonl``."""
        if self.enabled:
            self._write({"kind": kind, "step": step} | {k: float(v) for k, v in fields.items()})

    def _write(self, record: dict) -> None:
        self.file.write(json.dumps(record) + "\n")
        self.file.flush()

    def close(self) -> None:
        if self.file is not None:
            self.file.close()
