"""Fused elementwise / row-movement kernels and the fused optimizer against their PyTorch statements."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("C", [256, 2880, 4096])
def test_rmsnorm_fwd_bwd(C):
    from lyra_b200.ops import elementwise as ew, reference as ref

    torch.manual_seed(0)
    x = torch.randn(777, C, device="cuda").bfloat16()
    scale = torch.rand(C, device="cuda") + 0.5
    dy = torch.randn(777, C, device="cuda").bfloat16()
    xs, ss = x.clone().requires_grad_(True), scale.clone().requires_grad_(True)
    y = ew.RMSNorm.apply(xs, ss, 1e-5)
    y.backward(dy)
    xr, sr = x.float().requires_grad_(True), scale.clone().requires_grad_(True)
    yr = ref.rms_norm(xr, sr, 1e-5)
    yr.backward(dy.float())
    assert _rel(y, yr) < 5e-3 and _rel(xs.grad, xr.grad) < 1e-2 and _rel(ss.grad, sr.grad) < 1e-2


def test_swiglu_fwd_bwd():
    from lyra_b200.ops import elementwise as ew, reference as ref

    torch.manual_seed(1)
    M, H = 300, 512
    pre = (torch.randn(M, 2 * H, device="cuda") * 4).bfloat16()
    d = torch.randn(M, H, device="cuda").bfloat16()
    pr = pre.float().requires_grad_(True)
    out = ref.swiglu(pr.view(M, 2, H))
    out.backward(d.float())
    assert _rel(ew.swiglu_fwd(pre, 1.702, 7.0), out) < 5e-3
    assert _rel(ew.swiglu_bwd(pre, d, 1.702, 7.0), pr.grad) < 1e-2


def test_moe_row_movement():
    from lyra_b200.ops import cuda_ops, elementwise as ew

    torch.manual_seed(2)
    F_, K, E, C = 200, 3, 6, 256
    xn = torch.randn(F_, C, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(F_)])
    scores = torch.rand(F_, K, device="cuda")
    dest, tile_group, offsets, R = cuda_ops.moe_routing_layout(idx, E)
    # rows of one expert are contiguous, in token order, starting at a multiple of 128
    flat = idx.reshape(-1)
    for e in range(E):
        d = dest[flat == e]
        assert int(offsets[e]) % 128 == 0
        assert torch.equal(d, torch.arange(int(offsets[e]), int(offsets[e]) + d.numel(), device="cuda"))
    x_perm = ew.scatter_rows(xn, dest, K, R)
    assert torch.equal(x_perm[dest], xn.repeat_interleave(K, 0))
    out = ew.combine_rows(x_perm, dest, scores, F_, K)
    ref_out = (x_perm[dest].view(F_, K, C).float() * scores[..., None]).sum(1)
    assert _rel(out, ref_out) < 5e-3
    dout = torch.randn(F_, C, device="cuda").bfloat16()
    d_rows, dscores = ew.combine_rows_bwd(x_perm, dout, dest, scores, R)
    assert _rel(dscores, (x_perm[dest].view(F_, K, C).float() * dout.float()[:, None]).sum(-1)) < 5e-3
    assert _rel(d_rows[dest].view(F_, K, C), scores[..., None] * dout.float()[:, None]) < 5e-3


def test_fused_optimizer_matches_reference_step():
    from dataclasses import replace

    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.params import tree_dict
    from lyra_b200.training.optimizer import OptimizerState, optimizer_step
    from lyra_b200.training.optimizer_cuda import optimizer_step_cuda
    from lyra_b200.training.train import TrainingConfig
    from lyra_b200.config import ModelConfig

    cfg = ModelConfig(name="opt-test", seq_len=64, n_embd=256, n_layers=2, head_dim=64, n_attn_heads=4, n_kv_heads=2, n_routed_experts=3,
                      n_shared_experts=1, n_active_experts=2, mlp_map=("dense", "moe"), vocab_size=1000, padded_vocab_size=1024)
    tcfg = TrainingConfig(steps=10, batch_size=2, accumulation_steps=1)
    spec = ModelWeights.spec(cfg)
    res = []
    for fused in (False, True):
        w = ModelWeights.init(0, cfg, device="cuda")
        params = tree_dict(w)
        state = OptimizerState.init(w, spec, tcfg)
        g = torch.Generator(device="cuda").manual_seed(7)
        for step in range(2):
            grads = {p: torch.randn(t.shape, device="cuda", generator=g) * 0.02 for p, t in params.items()}
            if fused:
                m = optimizer_step_cuda(params, grads, state, step, tcfg)
            else:
                m = optimizer_step(params, grads, state, step, tcfg)
        res.append((params, state, m))
    (p0, s0, m0), (p1, s1, m1) = res
    assert abs(float(m0["grad_norm"]) - float(m1["grad_norm"])) < 1e-3 * float(m0["grad_norm"])
    for p in p0:
        init = ModelWeights.init(0, cfg, device="cuda")
        base = tree_dict(init)[p]
        upd0, upd1 = p0[p] - base, p1[p] - base
        assert _rel(upd1, upd0) < 6e-2, (p, _rel(upd1, upd0))
    for p in s0.muon_moment:
        assert _rel(s1.muon_moment[p], s0.muon_moment[p]) < 1e-2
    for p in s0.adam_nu:
        assert _rel(s1.adam_nu[p], s0.adam_nu[p]) < 1e-3
    assert int(s0.adam_count) == int(s1.adam_count) == 2
    # a non-finite gradient leaves everything unchanged
    before = {p: t.clone() for p, t in p1.items()}
    grads = {p: torch.full_like(t, float("nan")) for p, t in p1.items()}
    m = optimizer_step_cuda(p1, grads, s1, 2, tcfg)
    assert not bool(m["grad_is_finite"]) and int(s1.adam_count) == 2
    assert all(torch.equal(before[p], p1[p]) for p in p1)


@pytest.mark.parametrize("D,use_norm", [(128, True), (64, False)])
def test_qk_norm_rope_kernel(D, use_norm):
    from lyra_b200.ops import elementwise as ew

    torch.manual_seed(3)
    B, T, N = 2, 96, 4
    q = torch.randn(B, T, N, D, device="cuda").bfloat16()
    k = torch.randn(B, T, 2, D, device="cuda").bfloat16()
    cos, sin = torch.rand(1, T, 1, D // 2, device="cuda"), torch.rand(1, T, 1, D // 2, device="cuda")
    qs = (torch.rand(D, device="cuda") + 0.5) if use_norm else None
    ks = (torch.rand(D, device="cuda") + 0.5) if use_norm else None
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    res = []
    for fn in (lambda *a: (ew._QKNormRope.apply(a[0], a[2], cos, sin, 1e-5), ew._QKNormRope.apply(a[1], a[3], cos, sin, 1e-5)),
               lambda *a: ew.qk_norm_rope(a[0], a[1], a[2], a[3], cos, sin, 1e-5)):
        ins = [q.clone().requires_grad_(True), k.clone().requires_grad_(True)] + [s.clone().requires_grad_(True) if s is not None else None for s in (qs, ks)]
        oq, ok = fn(*ins)
        torch.autograd.backward([oq, ok], [dq, dk])
        res.append([oq, ok] + [i.grad for i in ins if i is not None])
    for a, b in zip(*res):
        assert _rel(b, a) < 1.5e-2


@pytest.mark.parametrize("gate,xsa", [(True, True), (True, False), (False, True)])
def test_gate_xsa_kernel(gate, xsa):
    from lyra_b200.ops import api

    torch.manual_seed(4)
    B, T, Nq, Nkv, D, C = 2, 80, 8, 2, 128, 256
    t = torch.randn(B, T, Nq, D, device="cuda").bfloat16().transpose(1, 2)
    v = torch.randn(B, T, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
    h = torch.randn(B, T, C, device="cuda").bfloat16()
    wg = (torch.randn(C, Nq, device="cuda") * 0.1) if gate else None
    al = (torch.randn(Nq, device="cuda") * 0.5) if xsa else None
    d = torch.randn(B, T, Nq, D, device="cuda").bfloat16().transpose(1, 2)
    res = []
    for impl in ("torch", "auto"):
        ins = [x.clone().requires_grad_(True) if x is not None else None for x in (t, h, wg, v, al)]
        out = api.gate_xsa(ins[0], ins[1], ins[2], ins[3], ins[4], impl)
        out.backward(d)
        res.append([out] + [i.grad for i in ins if i is not None and i.grad is not None])
    assert len(res[0]) == len(res[1])
    for a, b in zip(*res):
        assert _rel(b, a) < 2.5e-2
