"""Run logging: ``metrics.jsonl`` rows and the console table (fields of lyra/training/metrics.py:15-78).
Per-step metric tensors stay on the device until a log line is due, so logging adds no per-step sync;
time spent in evaluation, sampling and checkpointing is excluded from step time and tokens/s."""

from __future__ import annotations

import json
import math
import time
from contextlib import contextmanager
from pathlib import Path

import torch

RULE = "─" * 60
PPL_CE_CLAMP = 20.0

TRAIN_COLUMNS = (
    ("step", "step", lambda v: f"{int(v):,}"),
    ("loss", "loss", lambda v: f"{v:.4f}"),
    ("ce_loss", "ce_loss", lambda v: f"{v:.4f}"),
    ("aux_loss", "aux", lambda v: f"{v:.4f}"),
    ("perplexity", "ppl", lambda v: f"{v:,.0f}"),
    ("step_time", "step_ms", lambda v: f"{v * 1e3:.1f}"),
    ("tps", "tok/s", lambda v: f"{v:,.0f}"),
    ("total_tokens", "tokens", lambda v: f"{v / 1e9:.3f}B" if v >= 1e9 else f"{v / 1e6:.3f}M"),
)


def format_duration(seconds: float) -> str:
    minutes, secs = divmod(int(seconds), 60)
    hours, minutes = divmod(minutes, 60)
    return f"{hours}h {minutes}m {secs}s" if hours else f"{minutes}m {secs}s" if minutes else f"{seconds:.1f}s"


def _sync() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()


class MetricsLogger:
    def __init__(self, run_dir: Path, tokens_per_step: int = 0, initial_step: int = 0, enabled: bool = True):
        self.tokens_per_step = tokens_per_step
        self.total_tokens = initial_step * tokens_per_step
        self.enabled = enabled
        self.file = (Path(run_dir) / "metrics.jsonl").open("a") if enabled else None
        self.window: list[dict] = []
        self.window_start = time.perf_counter()
        self.printed_header = False

    def record(self, aux: dict) -> None:
        self.window.append(aux)
        self.total_tokens += self.tokens_per_step

    def log_train(self, step: int) -> None:
        if not self.window:
            return
        rows = [{k: float(v) for k, v in row.items()} for row in self.window]  # device -> host here
        elapsed = time.perf_counter() - self.window_start
        avg = {k: sum(r[k] for r in rows) / len(rows) for k in rows[0]}
        avg["perplexity"] = math.exp(min(avg["ce_loss"], PPL_CE_CLAMP))
        avg["step_time"] = elapsed / len(rows)
        avg["tps"] = self.tokens_per_step * len(rows) / elapsed
        avg["total_tokens"] = self.total_tokens
        record = {"kind": "train", "step": step} | avg
        if self.enabled:
            if not self.printed_header:
                print("  ".join(h.ljust(8) for _, h, _ in TRAIN_COLUMNS))
                self.printed_header = True
            print("  ".join(fmt(record[k]).ljust(8) for k, _, fmt in TRAIN_COLUMNS))
            self._write(record)
        self.window = []
        self.window_start = time.perf_counter()

    @contextmanager
    def paused(self):
        """Leave evaluation, sampling and checkpointing out of the step time and throughput."""
        _sync()
        start = time.perf_counter()
        try:
            yield
        finally:
            _sync()
            self.window_start += time.perf_counter() - start

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
