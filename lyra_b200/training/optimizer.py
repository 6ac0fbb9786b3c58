"""Hybrid optimizer: Muon (Polar-Express Newton-Schulz) on ``Tag.MATRIX`` leaves, Adam on the rest,
warmup-stable-decay schedule, per-matrix RMS clipping and the non-finite-gradient step skip.
Numerics follow lyra/training/optimizer.py:21-192.

State is a flat ``{leaf path: tensor}`` mapping per moment, holding this rank's shard of every leaf.
Updates are applied in place. On CUDA the elementwise parts run as fused kernels and Newton-Schulz as
batched tcgen05 GEMMs (``lyra_b200.ops.cuda_ops``); the PyTorch statements below are the oracle and the CPU path.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from lyra_b200.nn.params import Tag, tree_dict

MUON_TAGS = {Tag.MATRIX}
ADAM_TAGS = {Tag.DEFAULT, Tag.BIAS, Tag.EMBEDDING, Tag.SCALAR}

_POLAR_EXPRESS = (
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
)
POLAR_EXPRESS_COEFFS = tuple((a / 1.01, b / 1.01**3, c / 1.01**5) for a, b, c in _POLAR_EXPRESS)


def is_mlp_up(path: str) -> bool:
    return path.split("/")[-1] == "mlp_up"


def as_matrices(path: str, x: torch.Tensor) -> tuple[torch.Tensor, bool]:
    """View of a leaf as a stack of matrices. For any ``mlp_up [..., C, 2, H]`` the SwiGLU halves are swapped
    in front so each half of each expert is its own ``[C, H]`` matrix (lyra/training/optimizer.py:41-44)."""
    if is_mlp_up(path):
        return x.transpose(-3, -2), True
    return x, False


@dataclass
class OptimizerState:
    muon_moment: dict[str, torch.Tensor] = field(default_factory=dict)
    adam_mu: dict[str, torch.Tensor] = field(default_factory=dict)
    adam_nu: dict[str, torch.Tensor] = field(default_factory=dict)
    adam_count: torch.Tensor | None = None

    @classmethod
    def init(cls, params: Any, spec: Any, tcfg) -> "OptimizerState":
        p, s = tree_dict(params), tree_dict(spec)
        st = cls()
        for path, leaf in p.items():
            if leaf.numel() == 0 and math.prod(s[path].shape) > 0:
                continue  # owned by another rank
            if s[path].tag in MUON_TAGS:
                st.muon_moment[path] = torch.zeros_like(leaf, dtype=tcfg.muon_moment_dtype)
            else:
                st.adam_mu[path] = torch.zeros_like(leaf, dtype=tcfg.adam_mu_dtype)
                st.adam_nu[path] = torch.zeros_like(leaf, dtype=tcfg.adam_nu_dtype)
        dev = next(iter(p.values())).device
        st.adam_count = torch.zeros((), dtype=torch.int32, device=dev)
        return st


def wsd_lr(step: int, tcfg) -> tuple[float, float, float]:
    """Warmup-stable-decay multiplier at 0-based ``step`` (lyra/training/optimizer.py:81-88)."""
    s = float(step)
    warmup = min((s + 1.0) / max(tcfg.warmup_steps, 1), 1.0)
    decay_start = tcfg.warmup_steps + tcfg.stable_steps
    progress = min(max((s - decay_start) / max(tcfg.decay_steps - 1, 1), 0.0), 1.0)
    decay = 0.5 * (1.0 + math.cos(math.pi * progress)) if tcfg.decay_type == "cosine" else 1.0 - progress
    scale = warmup if s < tcfg.warmup_steps else decay
    return tcfg.adam_max_lr * scale, tcfg.muon_max_lr * scale, scale


def newtonschulz(X: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """Five Polar-Express iterations in bf16 on a stack of matrices (lyra/training/optimizer.py:114-126)."""
    dtype = X.dtype
    tall = X.shape[-2] > X.shape[-1]
    X = X.to(torch.bfloat16)
    norm = torch.linalg.matrix_norm(X.float(), dim=(-2, -1), keepdim=True).to(torch.bfloat16)
    X = X / (1.01 * norm + eps)
    if tall:
        X = X.transpose(-1, -2)
    for a, b, c in POLAR_EXPRESS_COEFFS:
        A = X @ X.transpose(-1, -2)
        X = a * X + (b * A + c * (A @ A)) @ X
    if tall:
        X = X.transpose(-1, -2)
    return X.to(dtype)


def _sumsq(t: torch.Tensor) -> torch.Tensor:
    f = t.float()
    return (f * f).sum()


@torch.no_grad()
def optimizer_step(params: dict[str, torch.Tensor], grads: dict[str, torch.Tensor], state: OptimizerState, step: int, tcfg,
                   *, rt=None) -> dict[str, torch.Tensor]:
    """One update of every leaf, in place. ``params``/``grads`` map leaf path -> this rank's shard.
    Returns the metric tensors of the reference's ``optimizer_step`` (lyra/training/optimizer.py:166-192).

    A non-finite global gradient norm turns the step into a no-op: learning rates 0, momentum and betas 1,
    gradients 0, so parameters and moments keep their values and ``adam_count`` does not advance."""
    adam_lr, muon_lr, lr_scale = wsd_lr(step, tcfg)
    dev = state.adam_count.device
    muon_paths = [p for p in params if p in state.muon_moment]
    adam_paths = [p for p in params if p in state.adam_mu]

    # ---- norms and per-matrix RMS (global quantities: summed over ranks for sharded leaves)
    zero = torch.zeros((), dtype=torch.float32, device=dev)
    once = (lambda p: rt.counts_once(p)) if rt is not None else (lambda p: True)
    muon_sq = sum((_sumsq(grads[p]) for p in muon_paths if once(p)), zero)
    adam_sq = sum((_sumsq(grads[p]) for p in adam_paths if once(p)), zero)
    if rt is not None:
        muon_sq, adam_sq = rt.sum_over_ranks(muon_sq, adam_sq)
    grad_norm = (muon_sq + adam_sq).sqrt()
    finite = torch.isfinite(grad_norm)
    enabled = finite.float()

    # Under tensor parallelism a rank holds a column or row slice of each matrix: the per-matrix RMS and Newton-Schulz need
    # the whole matrix, so the runtime gathers it (``gather_leaf``) and hands back this rank's slice (``slice_leaf``).
    gather = getattr(rt, "gather_leaf", None)
    take = getattr(rt, "slice_leaf", None)
    all_rms = []
    clipped: dict[str, torch.Tensor] = {}
    for p in muon_paths:
        g = grads[p]
        local, swapped = as_matrices(p, g.float())
        m = as_matrices(p, gather(p, g).float())[0] if gather is not None else local
        msq = (m * m).sum(dim=(-2, -1), keepdim=True)
        numel = m.shape[-2] * m.shape[-1]
        r = (msq / numel).sqrt()
        all_rms.append(r.reshape(-1))
        scale = torch.where(torch.isfinite(r), torch.clamp(tcfg.muon_grad_clip / (r + 1e-8), max=1.0), torch.ones_like(r))
        c = local * scale
        clipped[p] = (c.transpose(-3, -2) if swapped else c).to(g.dtype)
    all_rms_t = torch.cat(all_rms) if all_rms else torch.zeros(1, device=dev)
    metrics = {
        "adam_lr": torch.tensor(adam_lr), "muon_lr": torch.tensor(muon_lr), "lr_scale": torch.tensor(lr_scale),
        "grad_norm": grad_norm, "muon_grad_norm": muon_sq.sqrt(), "adam_grad_norm": adam_sq.sqrt(),
        "grad_is_finite": finite,
        "muon_grad_rms_max": all_rms_t.max(), "muon_grad_clip_frac": (all_rms_t > tcfg.muon_grad_clip).float().mean(),
    }
    if rt is not None:
        metrics["muon_grad_rms_max"] = rt.max_over_ranks(metrics["muon_grad_rms_max"])
        clipped_n, total_n = rt.sum_over_ranks((all_rms_t > tcfg.muon_grad_clip).float().sum(), torch.tensor(float(all_rms_t.numel()), device=dev))
        metrics["muon_grad_clip_frac"] = clipped_n / total_n.clamp_min(1.0)

    # ---- Muon
    lr_m = muon_lr * enabled
    momentum = torch.where(finite, torch.tensor(tcfg.muon_momentum, device=dev), torch.ones((), device=dev))
    for p in muon_paths:
        g = torch.where(finite, clipped[p].float(), torch.zeros((), device=dev))
        m_new = (momentum * state.muon_moment[p].float() + g).to(tcfg.muon_moment_dtype)
        state.muon_moment[p].copy_(m_new)
        d = (g + tcfg.muon_momentum * m_new.float()) if tcfg.muon_nesterov else m_new.float()
        dm, swapped = as_matrices(p, gather(p, d) if gather is not None else d)
        ns = newtonschulz(dm)  # every matrix is whole here: owned as a whole leaf, or gathered over the model axis
        rows, cols = dm.shape[-2], dm.shape[-1]
        stepv = lr_m * ns.float() * (math.sqrt(max(rows, cols)) * tcfg.muon_update_rms)
        stepv = stepv.transpose(-3, -2) if swapped else stepv
        if take is not None:
            stepv = take(p, stepv)
        w = params[p]
        w.copy_((w.float() - (stepv + lr_m * tcfg.muon_wd * w.float())).to(w.dtype))

    # ---- Adam
    b1, b2 = tcfg.adam_betas
    lr_a = adam_lr * enabled
    keep1 = torch.where(finite, torch.tensor(b1, device=dev), torch.ones((), device=dev))
    keep2 = torch.where(finite, torch.tensor(b2, device=dev), torch.ones((), device=dev))
    count = state.adam_count.item() if dev.type == "cpu" else int(state.adam_count)
    c1, c2 = 1.0 / (1.0 - b1 ** (count + 1)), 1.0 / (1.0 - b2 ** (count + 1))
    for p in adam_paths:
        g = torch.where(finite, grads[p].float(), torch.zeros((), device=dev))
        mu = (keep1 * state.adam_mu[p].float() + (1.0 - keep1) * g).to(tcfg.adam_mu_dtype)
        nu = (keep2 * state.adam_nu[p].float() + (1.0 - keep2) * g * g).to(tcfg.adam_nu_dtype)
        state.adam_mu[p].copy_(mu)
        state.adam_nu[p].copy_(nu)
        w = params[p]
        w.copy_((w.float() - lr_a * (mu.float() * c1) / ((nu.float() * c2).sqrt() + 1e-8)).to(w.dtype))
    state.adam_count += finite.to(state.adam_count.dtype)
    return metrics
