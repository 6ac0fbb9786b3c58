"""CUDA execution of the hybrid optimizer step: same numerics as ``optimizer.optimizer_step``
(lyra/training/optimizer.py:96-192), organised for a 180 GB device.

* no leaf-sized fp32 temporaries: norms are reductions over the stored dtype, the momentum / direction pass
  and both parameter updates are single fused kernels (``csrc/optim/optim.cu``) that also refresh the bf16
  compute copy of the weights;
* Newton-Schulz runs as batched tcgen05 GEMMs over chunks of stacked matrices, tall matrices through
  MN-major operands instead of transposes;
* the finite-gradient gate stays on the device (an ``enabled`` flag read by every kernel), so a step has no
  host synchronisation.
"""

from __future__ import annotations

import math

import torch

from lyra_b200.ops import gemm as G
from lyra_b200.ops import native
from lyra_b200.ops.native import c_float, c_int, c_ll, ptr
from lyra_b200.training.optimizer import POLAR_EXPRESS_COEFFS, OptimizerState, as_matrices, is_mlp_up, newtonschulz, wsd_lr

BF16 = torch.bfloat16
NS_CHUNK_ELEMS = 1 << 29


def _sumsq(t: torch.Tensor) -> torch.Tensor:
    n = torch.linalg.vector_norm(t.reshape(-1), 2, dtype=torch.float32)
    return n * n


def newtonschulz_gemm(X: torch.Tensor) -> torch.Tensor:
    """Five Polar-Express iterations on ``X [G, m, n]`` (bf16, contiguous, already normalised) with the batched
    tcgen05 GEMM. Wide matrices iterate ``A = X X^T; X <- aX + (bA + cA^2) X``; tall ones iterate on the Gram
    matrix of the other side (``A = X^T X; X <- aX + X (bA + cA^2)``), which equals transposing, iterating and
    transposing back."""
    Gn, m, n = X.shape
    tall = m > n
    k = n if tall else m
    A = torch.empty(Gn, k, k, dtype=BF16, device=X.device)
    B = torch.empty_like(A)
    Y = torch.empty_like(X)
    for a, b, c in POLAR_EXPRESS_COEFFS:
        if tall:
            G.batched_gemm(X, X, a_mn=True, b_mn=True, out=A, symmetric=True)            # X^T X
            G.batched_gemm(A, A, out=B, alpha=c, beta=b, c_in=A, symmetric=True)         # bA + cA^2  (A symmetric)
            G.batched_gemm(X, B, out=Y, alpha=1.0, beta=a, c_in=X)       # aX + X B   (B symmetric)
        else:
            G.batched_gemm(X, X, out=A, symmetric=True)                                  # X X^T
            G.batched_gemm(A, A, out=B, alpha=c, beta=b, c_in=A, symmetric=True)
            G.batched_gemm(B, X, b_mn=True, out=Y, alpha=1.0, beta=a, c_in=X)
        X, Y = Y, X
    return X


def _matrix_geometry(path: str, shape: tuple[int, ...]) -> tuple[int, int, int, int, int]:
    """``(stack, mats_lo, rows, cols, stride_lo)`` of a MATRIX leaf in its own memory layout."""
    if is_mlp_up(path):
        *lead, C, two, H = shape
        return math.prod(lead) if lead else 1, two, C, H, H
    *lead, m, n = shape
    return math.prod(lead) if lead else 1, 1, m, n, 1


@torch.no_grad()
def optimizer_step_cuda(params: dict[str, torch.Tensor], grads: dict[str, torch.Tensor], state: OptimizerState, step: int, tcfg,
                        shadows: dict[str, torch.Tensor] | None = None, rt=None) -> dict[str, torch.Tensor]:
    lib = native.kernels()
    adam_lr, muon_lr, lr_scale = wsd_lr(step, tcfg)
    dev = state.adam_count.device
    shadows = shadows or {}
    muon_paths = [p for p in params if p in state.muon_moment]
    adam_paths = [p for p in params if p in state.adam_mu]
    stream = native.stream_ptr()

    # ---- global norm, finite gate, per-matrix RMS clip factors
    zero = torch.zeros((), dtype=torch.float32, device=dev)
    once = (lambda p: rt.counts_once(p)) if rt is not None else (lambda p: True)
    # leaves that arrived through the fused pull-reduce bring their sums of squares (per matrix) with them
    known = getattr(rt, "grad_sumsq", None) or {}
    leaf_sq = lambda p: known[p].sum() if p in known else _sumsq(grads[p])
    muon_sq = sum((leaf_sq(p) for p in muon_paths if once(p)), zero)
    adam_sq = sum((leaf_sq(p) for p in adam_paths if once(p)), zero)
    if rt is not None:
        muon_sq, adam_sq = rt.sum_over_ranks(muon_sq, adam_sq)
    grad_norm = (muon_sq + adam_sq).sqrt()
    finite = torch.isfinite(grad_norm)
    enabled = finite.float().reshape(1).contiguous()

    clips: dict[str, torch.Tensor] = {}
    all_rms = []
    for p in muon_paths:
        gm, _ = as_matrices(p, grads[p])
        n_mats = gm.numel() // (gm.shape[-2] * gm.shape[-1])
        if p in known and known[p].numel() == n_mats:
            norm = known[p].sqrt()
        else:
            norm = torch.linalg.vector_norm(gm, 2, dim=(-2, -1), dtype=torch.float32)
        r = (norm / math.sqrt(gm.shape[-2] * gm.shape[-1])).reshape(-1)
        all_rms.append(r)
        clips[p] = torch.where(torch.isfinite(r), torch.clamp(tcfg.muon_grad_clip / (r + 1e-8), max=1.0), torch.ones_like(r)).contiguous()
    all_rms_t = torch.cat(all_rms) if all_rms else torch.zeros(1, device=dev)
    metrics = {
        "adam_lr": torch.tensor(adam_lr), "muon_lr": torch.tensor(muon_lr), "lr_scale": torch.tensor(lr_scale),
        "grad_norm": grad_norm, "muon_grad_norm": muon_sq.sqrt(), "adam_grad_norm": adam_sq.sqrt(), "grad_is_finite": finite,
        "muon_grad_rms_max": all_rms_t.max(), "muon_grad_clip_frac": (all_rms_t > tcfg.muon_grad_clip).float().mean(),
    }

    if rt is not None:
        metrics["muon_grad_rms_max"] = rt.max_over_ranks(metrics["muon_grad_rms_max"])
        clipped_n, total_n = rt.sum_over_ranks((all_rms_t > tcfg.muon_grad_clip).float().sum(), torch.tensor(float(all_rms_t.numel()), device=dev))
        metrics["muon_grad_clip_frac"] = clipped_n / total_n.clamp_min(1.0)

    # ---- Muon
    nesterov = tcfg.muon_momentum if tcfg.muon_nesterov else -1.0
    for p in muon_paths:
        w, g, mom = params[p], grads[p].contiguous(), state.muon_moment[p]
        if w.dtype != torch.float32 or mom.dtype != BF16 or g.dtype not in (BF16, torch.float32):
            raise TypeError(f"{p}: the fused Muon kernels need fp32 parameters, a bf16 moment and bf16 or fp32 gradients "
                            f"(got {w.dtype}, {mom.dtype}, {g.dtype})")
        stack, mats_lo, rows, cols, stride_lo = _matrix_geometry(p, tuple(w.shape))
        per_stack = mats_lo * rows * cols
        d = torch.empty(w.shape, dtype=BF16, device=dev)
        native.check(lib.lyra_muon_moment(ptr(g), c_int(int(g.dtype == BF16)), ptr(mom), ptr(d), ptr(clips[p]), c_ll(w.numel()),
                                          c_ll(per_stack), c_ll(stride_lo), c_int(mats_lo), c_float(tcfg.muon_momentum), c_float(nesterov),
                                          ptr(enabled), stream), "muon_moment")
        native.count_launch()
        dm, swapped = as_matrices(p, d)                       # [..., rows, cols] view of d
        dm = dm.reshape(stack, mats_lo, rows, cols) if swapped else dm.reshape(stack, 1, rows, cols)
        use_gemm = rows % 8 == 0 and cols % 8 == 0 and min(rows, cols) >= 64
        chunk = max(1, NS_CHUNK_ELEMS // per_stack)
        ns_scale = math.sqrt(max(rows, cols)) * tcfg.muon_update_rms
        wflat, shadow = w.detach().reshape(stack, -1), shadows.get(p)
        sflat = shadow.reshape(stack, -1) if shadow is not None else None
        dflat = d.reshape(stack, -1)
        for s0 in range(0, stack, chunk):
            s1 = min(stack, s0 + chunk)
            X = dm[s0:s1].reshape(-1, rows, cols).contiguous()              # [(s1-s0)*mats_lo, rows, cols]
            norm = torch.linalg.vector_norm(X, 2, dim=(-2, -1), keepdim=True, dtype=torch.float32).to(BF16)
            X = X / (1.01 * norm + 1e-7)
            if use_gemm:
                Y = newtonschulz_gemm(X.contiguous())
            else:
                Y = _ns_unnormalised(X)
            dm[s0:s1].copy_(Y.reshape(s1 - s0, dm.shape[1], rows, cols))    # back into the leaf layout
            n = (s1 - s0) * per_stack
            native.check(lib.lyra_muon_update(ptr(wflat[s0:s1]), ptr(dflat[s0:s1]), ptr(sflat[s0:s1] if sflat is not None else None), c_ll(n),
                                              c_float(muon_lr), c_float(ns_scale), c_float(tcfg.muon_wd), ptr(enabled), stream), "muon_update")
            native.count_launch()
        del d

    # ---- Adam
    b1, b2 = tcfg.adam_betas
    for p in adam_paths:
        w, g = params[p], grads[p].contiguous()
        shadow = shadows.get(p)
        if w.dtype != torch.float32 or state.adam_mu[p].dtype != BF16 or state.adam_nu[p].dtype != torch.float32 or g.dtype not in (BF16, torch.float32):
            raise TypeError(f"{p}: the fused Adam kernel needs fp32 parameters, bf16 mu and fp32 nu")
        native.check(lib.lyra_adam(ptr(w), ptr(g), c_int(int(g.dtype == BF16)), ptr(state.adam_mu[p]), ptr(state.adam_nu[p]), ptr(shadow),
                                   c_ll(w.numel()), c_float(adam_lr), c_float(b1), c_float(b2), ptr(state.adam_count), c_float(1e-8),
                                   ptr(enabled), stream), "adam")
        native.count_launch()
    state.adam_count += finite.to(state.adam_count.dtype)
    return metrics


def _ns_unnormalised(X: torch.Tensor) -> torch.Tensor:
    """PyTorch Newton-Schulz for shapes the GEMM kernel does not take (tiny test models); ``X`` is already normalised."""
    tall = X.shape[-2] > X.shape[-1]
    if tall:
        X = X.transpose(-1, -2)
    for a, b, c in POLAR_EXPRESS_COEFFS:
        A = X @ X.transpose(-1, -2)
        X = a * X + (b * A + c * (A @ A)) @ X
    return X.transpose(-1, -2) if tall else X
