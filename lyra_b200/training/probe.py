"""Numerics probe: named summary statistics recorded while a forward pass runs.

Stat names and definitions follow the reference (lyra/training/probe.py:37-283) so ``numerics.jsonl``
files are comparable. Everything is computed under ``no_grad`` on detached fp32 copies: probing never
changes outputs or gradients.
"""

from __future__ import annotations

import copy
import math
from enum import IntEnum
from typing import Mapping

import torch

EPS = 1e-30
MASKED_LOGIT = -1e20  # padded vocabulary columns must not move the summary moments

Stats = dict


class Level(IntEnum):
    OFF = 0
    BASIC = 1
    FULL = 2


def _f32(x) -> torch.Tensor:
    return x.detach().float()


@torch.no_grad()
def tensor_stats(x, *, level: Level = Level.FULL) -> Stats:
    t = _f32(x)
    finite = torch.isfinite(t)
    safe = torch.where(finite, t, torch.zeros_like(t))
    flat = safe.reshape(-1)
    mean = flat.mean()
    second = (flat * flat).mean()
    var = (second - mean * mean).clamp_min(0.0)
    out = {
        "mean": mean,
        "rms": second.sqrt(),
        "std": var.sqrt(),
        "absmax": flat.abs().max(),
        "n_nonfinite": (~finite).sum().float(),
    }
    if level < Level.FULL:
        return out
    out["kurtosis"] = ((flat - mean) ** 4).mean() / (var * var + EPS)
    if safe.ndim >= 2:
        lead = tuple(range(safe.ndim - 1))
        chan_rms = (safe * safe).mean(dim=lead).sqrt()
        chan_mean = safe.mean(dim=lead)
        row_rms = (safe * safe).mean(dim=-1).sqrt()
        out.update({
            "chan_rms_max": chan_rms.max(),
            "chan_rms_ratio": chan_rms.max() / (chan_rms.mean() + EPS),
            "chan_mean_absmax": chan_mean.abs().max(),
            "row_rms_max": row_rms.max(),
        })
    return out


@torch.no_grad()
def residual_stats(x, delta) -> Stats:
    x32, d32 = _f32(x), _f32(delta)
    o32 = x32 + d32
    qx, qd, qo = (x32 * x32).mean(), (d32 * d32).mean(), (o32 * o32).mean()
    cross = (x32 * d32).mean()
    lead = tuple(range(o32.ndim - 1))
    chan_rms = (o32 * o32).mean(dim=lead).sqrt()
    chan_mean = o32.mean(dim=lead)
    tok_cos = (x32 * o32).sum(-1) / ((x32 * x32).sum(-1).sqrt() * (o32 * o32).sum(-1).sqrt() + EPS)
    absorbed = ((o32.to(x.dtype) == x.detach()) & (d32 != 0)).float().sum() / (d32 != 0).sum().clamp_min(1)
    return {
        "x_rms": qx.sqrt(),
        "delta_rms": qd.sqrt(),
        "out_rms": qo.sqrt(),
        "branch_ratio": (qd / (qx + EPS)).sqrt(),
        "correlation": cross / (qx * qd + EPS).sqrt(),
        "input_output_cosine": (qx + cross) / ((qx * qo).sqrt() + EPS),
        "token_cosine_mean": tok_cos.mean(),
        "growth": (qo / (qx + EPS)).sqrt(),
        "delta_mean": d32.mean(),
        "out_mean": o32.mean(),
        "out_absmax": o32.abs().max(),
        "out_chan_rms_ratio": chan_rms.max() / (chan_rms.mean() + EPS),
        "out_chan_mean_absmax": chan_mean.abs().max(),
        "branch_absorbed_frac": absorbed,
        "n_nonfinite": (~torch.isfinite(o32)).sum().float(),
    }


@torch.no_grad()
def swiglu_stats(x, limit: float, *, level: Level = Level.FULL) -> Stats:
    """Clip statistics of packed ``[gate | value]`` pre-activations; the gate has no lower bound."""
    bound = torch.tensor(limit, dtype=x.dtype).float().item()
    gate, value = _f32(x).chunk(2, dim=-1)
    out = {
        "gate_clip_frac": (gate > bound).float().mean(),
        "value_clip_frac": (value.abs() > bound).float().mean(),
    }
    if level >= Level.FULL:
        for name, raw, clipped in (("gate", gate, gate.clamp(max=bound)), ("value", value, value.clamp(-bound, bound))):
            out[f"{name}_clip_energy_frac"] = (raw**2 - clipped**2).sum() / ((raw**2).sum() + EPS)
    return out


@torch.no_grad()
def routing_stats(router_logits, expert_scores, group_sizes, n_experts: int, n_active: int) -> Stats:
    logits = _f32(router_logits)
    counts = _f32(group_sizes)
    load = counts / (counts.sum() + EPS)
    probs = torch.softmax(logits, dim=-1)
    usage = probs.mean(0)
    scores = _f32(expert_scores)
    dev = logits.device
    return {
        "logit_rms": (logits * logits).mean().sqrt(),
        "logit_absmax": logits.abs().max(),
        "lse_mean": torch.logsumexp(logits, dim=-1).mean(),
        "load_max_ratio": load.max() * n_experts,
        "load_min_ratio": load.min() * n_experts,
        "load_std": load.std(unbiased=False) * n_experts,
        "experts_unused": (counts == 0).sum().float(),
        "hard_usage_entropy": -(load * (load + EPS).log()).sum(),
        "usage_entropy": -(usage * (usage + EPS).log()).sum(),
        "usage_entropy_uniform": torch.tensor(math.log(n_experts), device=dev),
        "token_entropy": (-(probs * (probs + EPS).log()).sum(-1)).mean(),
        "top1_score": scores[..., 0].mean(),
        "topk_score_min": scores[..., -1].mean(),
        "n_experts": torch.tensor(float(n_experts), device=dev),
        "n_active": torch.tensor(float(n_active), device=dev),
    }


@torch.no_grad()
def logit_stats(logits) -> Stats:
    z = _f32(logits)
    flat = z.reshape(-1, z.shape[-1])
    width = flat.shape[-1]
    live = flat > MASKED_LOGIT
    row_count = live.sum(-1).float().clamp_min(1.0)
    n_live = row_count.mean()
    safe = torch.where(live, flat, torch.zeros_like(flat))
    row_mean = safe.sum(-1) / row_count
    row_second = (safe * safe).sum(-1) / row_count
    lse = torch.logsumexp(flat, dim=-1)
    logp = flat - lse[:, None]
    entropy = -torch.where(live, logp.exp() * logp, torch.zeros_like(logp)).sum(-1)
    return {
        "rms": row_second.mean().sqrt(),
        "absmax": safe.abs().max(),
        "token_std": (row_second - row_mean * row_mean).clamp_min(0.0).mean().sqrt(),
        "max_mean": flat.max(-1).values.mean(),
        "lse_mean": lse.mean(),
        "random_target_ce": (lse - row_mean).mean(),
        "entropy": entropy.mean(),
        "entropy_uniform": n_live.log(),
        "masked_frac": 1.0 - n_live / width,
        "n_nonfinite": (torch.isnan(flat) | torch.isposinf(flat)).sum().float(),
    }


class Probe:
    """Collects named statistics during a forward pass; ``scope`` returns a view writing into the same store."""

    def __init__(self, *, level: Level = Level.FULL, logit_subsample_tokens: int = 64, routing_only: bool = False) -> None:
        self.level = level
        self.logit_subsample_tokens = logit_subsample_tokens
        self.routing_only = routing_only
        self._prefix = ""
        self._values: dict[str, Stats] = {}

    @property
    def enabled(self) -> bool:
        return self.level > Level.OFF

    @property
    def detailed(self) -> bool:
        return self.enabled and not self.routing_only

    def scope(self, name: str) -> "Probe":
        if not self.enabled:
            return self
        child = copy.copy(self)  # shares _values
        child._prefix = f"{self._prefix}.{name}" if self._prefix else name
        return child

    def start(self) -> None:
        self._values.clear()

    def collect(self) -> dict[str, Stats]:
        out = dict(self._values)
        self._values.clear()
        return out

    def _add(self, name: str, stats: Stats) -> None:
        self._values[f"{self._prefix}.{name}" if self._prefix else name] = stats

    def tensor(self, name, x) -> None:
        if self.detailed:
            self._add(name, tensor_stats(x, level=self.level))

    def residual(self, name, x, delta) -> None:
        if self.detailed:
            self._add(name, residual_stats(x, delta))

    def swiglu(self, name, x, *, limit: float) -> None:
        if self.detailed:
            self._add(name, swiglu_stats(x, limit, level=self.level))

    def scalars(self, name, stats: Mapping) -> None:
        if self.enabled and (self.detailed or name == "aux_loss"):
            self._add(name, {k: torch.as_tensor(v).detach().float() for k, v in stats.items()})

    def routing(self, name, **kw) -> None:
        if self.enabled:
            self._add(name, routing_stats(**kw))

    def logits(self, name, logits) -> None:
        if self.detailed:
            self._add(name, logit_stats(logits))

    @torch.no_grad()
    def logit_subsample(self, name, hidden, unemb, *, vocab_size: int) -> None:
        """Logit statistics on a few evenly spaced tokens (training never materialises full logits)."""
        if not self.detailed:
            return
        flat = hidden.detach().reshape(-1, hidden.shape[-1])
        n = min(self.logit_subsample_tokens, flat.shape[0])
        pick = torch.linspace(0, flat.shape[0] - 1, n, device=flat.device).to(torch.int64)
        z = flat[pick].float() @ unemb.detach().float().t()
        z[:, vocab_size:] = MASKED_LOGIT
        self._add(name, logit_stats(z))


NO_PROBE = Probe(level=Level.OFF)


def to_floats(values: Mapping[str, Stats]) -> dict[str, dict[str, float]]:
    return {path: {k: float(v) for k, v in stats.items()} for path, stats in values.items()}


def mean_over_ranks(values: Mapping[str, Stats], group=None) -> dict[str, Stats]:
    """Average of every statistic over the data-parallel ranks (the reference's ``pmean``, lyra/training/steps.py:146)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(values)
    keys = [(p, k) for p, s in values.items() for k in s]
    if not keys:
        return {}
    flat = torch.stack([torch.as_tensor(values[p][k]).float().reshape(()) for p, k in keys])
    dist.all_reduce(flat, group=group)
    flat /= dist.get_world_size(group)
    out: dict[str, Stats] = {}
    for (p, k), v in zip(keys, flat):
        out.setdefault(p, {})[k] = v
    return out
