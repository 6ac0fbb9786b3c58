"""Routing kernels (top-k, scores, auxiliary loss, counts, expert-sorted permutation and their backward) against the PyTorch
statement of the same routing (lyra/model.py:418-491 in the reference)."""

from dataclasses import replace

import pytest
import torch

pytestmark = pytest.mark.gpu


def _torch_routing(logits, bias, k, lb_w, z_w):
    z = logits + (bias if bias is not None else 0.0)
    vals, idx = torch.topk(z, k, dim=-1)
    scores = torch.softmax(vals, dim=-1)
    F_, E = z.shape
    counts = torch.bincount(idx.reshape(-1), minlength=E).float()
    lb = E * (torch.softmax(z, -1).sum(0) / F_ * (counts / (F_ * k)).detach()).sum()
    zt = torch.logsumexp(z, -1).square().mean()
    return scores, idx, lb_w * lb + z_w * zt


@pytest.mark.parametrize("shape", [(8192, 31, 3), (1000, 128, 4), (77, 7, 2), (4096, 15, 3)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_route_matches_torch(shape, with_bias):
    from lyra_b200.ops import native, routing

    F_, E, k = shape
    torch.manual_seed(F_ + E)
    logits0 = torch.randn(F_, E, device="cuda") * 1.5
    bias0 = torch.randn(E, device="cuda") * 0.3 if with_bias else None
    gs = torch.randn(F_, k, device="cuda")
    res = {}
    for impl in ("torch", "kernel"):
        logits = logits0.clone().requires_grad_(True)
        bias = bias0.clone().requires_grad_(True) if with_bias else None
        if impl == "torch":
            scores, idx, aux = _torch_routing(logits, bias, k, 1e-2, 1e-4)
            plan = None
        else:
            scores, idx, aux, plan = routing.route(logits, bias, k, 1e-2, 1e-4)
        ((scores * gs).sum() + 3.0 * aux).backward()
        res[impl] = (scores.detach(), idx, aux.detach(), logits.grad, bias.grad if with_bias else None, plan)
    native.check_status()
    (s0, i0, a0, g0, b0, _), (s1, i1, a1, g1, b1, plan) = res["torch"], res["kernel"]
    assert torch.equal(i0, i1)
    assert (s0 - s1).abs().max().item() < 1e-5
    assert abs(a0.item() - a1.item()) < 1e-5 * max(1.0, abs(a0.item()))
    assert ((g0 - g1).norm() / g0.norm()).item() < 1e-4
    if with_bias:
        assert ((b0 - b1).norm() / b0.norm()).item() < 1e-4
    # the plan is the stable counting sort of the assignments by expert
    flat = i1.reshape(-1)
    assert torch.equal(plan.counts.long(), torch.bincount(flat, minlength=E))
    assert torch.equal(plan.order.long(), torch.argsort(flat, stable=True))
    starts = plan.starts.long()
    assert starts[0] == 0 and torch.equal(starts[1:], torch.cumsum(plan.counts.long(), 0))
    pos = starts[flat] + plan.rank_in_expert.long()
    assert torch.equal(plan.order.long()[pos], torch.arange(flat.numel(), device="cuda"))
    # same bits on a second call
    s2, i2, a2, plan2 = routing.route(logits0, bias0, k, 1e-2, 1e-4)
    assert torch.equal(s1, s2) and torch.equal(a1, a2) and torch.equal(plan.order, plan2.order)


def test_top_k_ties_take_the_lower_expert():
    from lyra_b200.ops import routing

    logits = torch.zeros(5, 40, device="cuda")
    logits[:, 33] = 1.0
    logits[:, 2] = 1.0
    _, idx, _, _ = routing.route(logits, None, 3, 0.0, 0.0)
    assert idx.tolist() == [[2, 33, 0]] * 5
