"""Routing after the fp32 router product (``csrc/moe/route.cu``): top-k, scores, auxiliary loss, per-expert counts and the
expert-sorted permutation in three launches; the backward pass is one kernel that turns the gradients of the scores and of
the auxiliary loss into the gradient of the logits (semantics of lyra/model.py:418-491)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from lyra_b200.ops import native
from lyra_b200.ops.native import c_float, c_int, ptr

MAX_EXPERTS, MAX_K = 256, 8


@dataclass
class RoutingPlan:
    """What the exchange / permutation needs besides the chosen experts, all int32 on the device: ``counts [Er]``,
    ``starts [Er + 1]`` (exclusive prefix), ``order [F k]`` (assignments sorted by expert, token order inside an expert) and
    ``rank_in_expert [F k]``."""

    counts: torch.Tensor
    starts: torch.Tensor
    order: torch.Tensor
    rank_in_expert: torch.Tensor


def supported(n_routed: int, k: int) -> bool:
    return 1 <= k <= MAX_K and k <= n_routed <= MAX_EXPERTS


class _Route(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, k, lb_weight, z_weight):
        F_, Er = logits.shape
        dev = logits.device
        logits = logits.contiguous()
        b = bias.detach().float().reshape(Er).contiguous() if bias is not None else None
        nb = (F_ + 31) // 32
        idx = torch.empty(F_, k, dtype=torch.int64, device=dev)
        scores = torch.empty(F_, k, dtype=torch.float32, device=dev)
        lse = torch.empty(F_, dtype=torch.float32, device=dev)
        ints = torch.empty(Er + (Er + 1) + 2 * F_ * k + nb * Er + F_ * k, dtype=torch.int32, device=dev)
        counts, starts, order, rank, block_counts, local_rank = torch.split(ints, [Er, Er + 1, F_ * k, F_ * k, nb * Er, F_ * k])
        floats = torch.empty(nb * Er + nb + 1, dtype=torch.float32, device=dev)
        part_colsum, part_z, aux = torch.split(floats, [nb * Er, nb, 1])
        lib = native.kernels()
        native.check(lib.lyra_route(ptr(logits), ptr(b), c_int(F_), c_int(Er), c_int(k), c_float(lb_weight), c_float(z_weight), ptr(idx), ptr(scores),
                                    ptr(lse), ptr(counts), ptr(starts), ptr(order), ptr(rank), ptr(aux), ptr(part_colsum), ptr(part_z),
                                    ptr(block_counts), ptr(local_rank), native.stream_ptr()), "lyra_route")
        native.count_launch(3)
        ctx.save_for_backward(logits, b, lse, idx, scores, counts)
        ctx.cfg = (k, lb_weight, z_weight, bias is not None)
        ctx.mark_non_differentiable(idx, counts, starts, order, rank)
        return scores, idx, aux.reshape(()), counts, starts, order, rank

    @staticmethod
    def backward(ctx, dscores, _didx, daux, *_):
        logits, b, lse, idx, scores, counts = ctx.saved_tensors
        k, lb_weight, z_weight, has_bias = ctx.cfg
        F_, Er = logits.shape
        d_logits = torch.empty_like(logits)
        ds = dscores.float().contiguous() if dscores is not None else None
        da = daux.float().reshape(1).contiguous() if daux is not None else None
        lib = native.kernels()
        native.check(lib.lyra_route_bwd(ptr(logits), ptr(b), ptr(lse), ptr(idx), ptr(scores), ptr(ds), ptr(counts), ptr(da), c_int(F_), c_int(Er), c_int(k),
                                        c_float(lb_weight), c_float(z_weight), ptr(d_logits), native.stream_ptr()), "lyra_route_bwd")
        native.count_launch()
        return d_logits, (d_logits.sum(0) if has_bias else None), None, None, None


def route(logits: torch.Tensor, bias: torch.Tensor | None, k: int, lb_weight: float, z_weight: float):
    """``logits [F, Er]`` fp32 (router product without the bias) -> ``(scores [F, k], idx [F, k] int64, aux, RoutingPlan)``."""
    scores, idx, aux, counts, starts, order, rank = _Route.apply(logits.float(), bias, k, lb_weight, z_weight)
    return scores, idx, aux, RoutingPlan(counts, starts, order, rank)


def gather_by_plan(x: torch.Tensor, plan: RoutingPlan, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Rows of ``x [F, C]`` (bf16) in the plan's expert order, and ``dest [F k]`` (int64) with ``dest[assignment] = sorted
    position``: what a small-batch expert product and its weighted combine need, in one launch."""
    A, C = plan.order.numel(), x.shape[1]
    out = torch.empty(A, C, dtype=torch.bfloat16, device=x.device)
    dest = torch.empty(A, dtype=torch.int64, device=x.device)
    native.check(native.kernels().lyra_gather_by_plan(ptr(x), ptr(plan.order), c_int(A), c_int(k), c_int(C), ptr(out), ptr(dest),
                                                      native.stream_ptr()), "lyra_gather_by_plan")
    native.count_launch()
    return out, dest
