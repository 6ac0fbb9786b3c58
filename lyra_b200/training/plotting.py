"""Plot a run's loss, gradient norm and expert routing balance into ``metrics.png``:
``python -m lyra_b200.training.plotting <run_dir>`` (three panels as lyra/training/plotting.py:28-93).

Rendering is CPU-only and headless. matplotlib (Agg) is used when it is installed; otherwise a small built-in
rasteriser draws the same three panels (axes, grid, polylines, no text) and encodes the PNG with zlib."""

from __future__ import annotations

import json
import math
import struct
import sys
import zlib
from itertools import accumulate
from pathlib import Path

import numpy as np


def _rows(path: Path) -> list[dict]:
    return [json.loads(line) for line in path.read_text().splitlines() if line.strip()] if path.exists() else []


def _routing_series(run_dir: Path) -> tuple[list[int], list[float], list[float]]:
    """Busiest and least-used expert load relative to uniform, averaged over MoE layers."""
    steps, busiest, least = [], [], []
    for row in _rows(run_dir / "numerics.jsonl"):
        routers = [s for s in row["records"].values() if "load_max_ratio" in s]
        if routers:
            steps.append(row["step"])
            busiest.append(sum(s["load_max_ratio"] for s in routers) / len(routers))
            least.append(sum(s["load_min_ratio"] for s in routers) / len(routers))
    return steps, busiest, least


def _ema(values: list[float]) -> list[float]:
    return list(accumulate(values, lambda prev, v: prev + 0.2 * (v - prev)))


def _series(run_dir: Path):
    rows = _rows(run_dir / "metrics.jsonl")
    train = [r for r in rows if r["kind"] == "train"]
    evals = [r for r in rows if r["kind"] == "eval"]
    if not train:
        return None
    tps = train[-1]["total_tokens"] / max(train[-1]["step"], 1) / 1e6
    x = lambda rs: [r["step"] * tps for r in rs]
    steps, busiest, least = _routing_series(run_dir)
    return {
        "loss": [(x(train), [r["ce_loss"] for r in train], "#2563eb", True), (x(evals), [r["eval_ce_loss"] for r in evals], "#d97706", False)],
        "grad": [(x(train), [r["grad_norm"] for r in train], "#2563eb", True)],
        "routing": [([s * tps for s in steps], busiest, "#7c3aed", False), ([s * tps for s in steps], least, "#0f766e", False)],
    }


# --------------------------------------------------------------------------- built-in rasteriser
def _hex(c: str) -> np.ndarray:
    return np.array([int(c[i:i + 2], 16) for i in (1, 3, 5)], dtype=np.float32)


def _line(img: np.ndarray, x0, y0, x1, y1, color: np.ndarray, alpha: float = 1.0) -> None:
    n = int(max(abs(x1 - x0), abs(y1 - y0))) + 1
    xs = np.clip(np.round(np.linspace(x0, x1, n)).astype(int), 0, img.shape[1] - 1)
    ys = np.clip(np.round(np.linspace(y0, y1, n)).astype(int), 0, img.shape[0] - 1)
    img[ys, xs] = (1 - alpha) * img[ys, xs] + alpha * color


def _panel(img: np.ndarray, box, lines, log_y: bool = False, y_floor: float | None = None) -> None:
    l, t, r, b = box
    grid, axis = _hex("#e2e8f0"), _hex("#cbd5e1")
    for i in range(1, 5):
        gy = t + (b - t) * i / 5
        _line(img, l, gy, r, gy, grid)
        gx = l + (r - l) * i / 5
        _line(img, gx, t, gx, b, grid)
    _line(img, l, b, r, b, axis)
    _line(img, l, t, l, b, axis)
    pts = [(x, y) for xs, ys, _, _ in lines for x, y in zip(xs, ys) if math.isfinite(y) and (not log_y or y > 0)]
    if not pts:
        return
    f = (lambda v: math.log10(v)) if log_y else (lambda v: v)
    xmin, xmax = min(p[0] for p in pts), max(p[0] for p in pts)
    ymin, ymax = min(f(p[1]) for p in pts), max(f(p[1]) for p in pts)
    if y_floor is not None:
        ymin = min(ymin, y_floor)
    xspan, yspan = (xmax - xmin) or 1.0, (ymax - ymin) or 1.0
    px = lambda v: l + 6 + (v - xmin) / xspan * (r - l - 12)
    py = lambda v: b - 6 - (f(v) - ymin) / yspan * (b - t - 12)
    for xs, ys, color, smooth in lines:
        keep = [(x, y) for x, y in zip(xs, ys) if math.isfinite(y) and (not log_y or y > 0)]
        if len(keep) < 1:
            continue
        c = _hex(color)
        passes = [([k[1] for k in keep], 0.25), (_ema([k[1] for k in keep]), 1.0)] if smooth else [([k[1] for k in keep], 1.0)]
        for vals, alpha in passes:
            for i in range(len(keep) - 1):
                for dy in (0, 1):
                    _line(img, px(keep[i][0]), py(vals[i]) + dy, px(keep[i + 1][0]), py(vals[i + 1]) + dy, c, alpha)
            if len(keep) == 1:
                _line(img, px(keep[0][0]) - 2, py(vals[0]), px(keep[0][0]) + 2, py(vals[0]), c, alpha)


def _write_png(path: Path, img: np.ndarray) -> None:
    h, w, _ = img.shape
    raw = b"".join(b"\x00" + img[y].astype(np.uint8).tobytes() for y in range(h))
    chunk = lambda tag, data: struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)
    path.write_bytes(b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) +
                     chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


def _plot_builtin(run_dir: Path, series: dict) -> None:
    W, H = 1500, 480
    img = np.full((H, W, 3), 255.0, dtype=np.float32)
    boxes = [(60 + i * 490, 60, 60 + i * 490 + 420, 420) for i in range(3)]
    _panel(img, boxes[0], series["loss"])
    _panel(img, boxes[1], series["grad"], log_y=True)
    _panel(img, boxes[2], series["routing"] + [([0.0, 1.0], [1.0, 1.0], "#64748b", False)] if series["routing"][0][0] else [], y_floor=0.0)
    _write_png(run_dir / "metrics.png", img)


def _plot_matplotlib(run_dir: Path, series: dict, title: str) -> None:
    import matplotlib

    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    fig, axes = plt.subplots(1, 3, figsize=(15, 4.8))
    names = [("loss", "Loss", "Cross-entropy (nats)"), ("grad", "Gradient Norm (log scale)", "Global gradient L2 norm"),
             ("routing", "Routing Balance", "Expert load / uniform load")]
    for ax, (key, ttl, ylabel) in zip(axes, names):
        for xs, ys, color, smooth in series[key]:
            if not xs:
                continue
            if smooth:
                ax.plot(xs, ys, color=color, alpha=0.2, linewidth=0.8)
                ys = _ema(ys)
            ax.plot(xs, ys, color=color, linewidth=1.8)
        ax.set_title(ttl, fontsize=14, pad=12)
        ax.set_ylabel(ylabel, fontsize=11)
        ax.set_xlabel("Training tokens (millions)", fontsize=11, labelpad=8)
        ax.grid(True, color="#e2e8f0", linewidth=0.7)
    axes[1].set_yscale("log", nonpositive="mask")
    if series["routing"][0][0]:
        axes[2].axhline(1.0, color="#64748b", linestyle="--", linewidth=1)
        axes[2].set_ylim(bottom=0)
    fig.suptitle(title, fontsize=17, fontweight="bold", y=0.97)
    fig.subplots_adjust(left=0.055, right=0.99, top=0.8, bottom=0.16, wspace=0.3)
    fig.savefig(run_dir / "metrics.png", format="png", dpi=180, facecolor="white")
    plt.close(fig)


def plot_run(run_dir) -> None:
    run_dir = Path(run_dir)
    series = _series(run_dir)
    if series is None:
        return
    config = json.loads((run_dir / "config.json").read_text()) if (run_dir / "config.json").exists() else {}
    try:
        _plot_matplotlib(run_dir, series, config.get("model", {}).get("name", "Training progress"))
    except ImportError:
        _plot_builtin(run_dir, series)


if __name__ == "__main__":
    plot_run(sys.argv[1])
