"""End-to-end: the kernel path (implementation="auto") against the PyTorch path on the same GPU."""

from dataclasses import replace

import pytest
import torch

pytestmark = pytest.mark.gpu
TOLERANCE = 0.10   # relative L2 error of any leaf's gradient; both paths compute in bf16 and take the same routing (measured: up to 0.08)


def _cfgs():
    from lyra_b200.config import ModelConfig, full_moe
    from lyra_b200.variants import model_variant

    tiny = replace(model_variant("tiny"), vocab_size=2048, padded_vocab_size=2304)
    mid = ModelConfig(name="test-mid", seq_len=256, n_embd=512, n_layers=4, head_dim=128, n_attn_heads=4, n_kv_heads=2,
                      use_learned_xsa=True, use_sdpa_output_gate=True, n_routed_experts=7, n_shared_experts=1, n_active_experts=3,
                      mlp_map=("dense", "moe", "dense", "moe"), vocab_size=4000, padded_vocab_size=4096, tie_embeddings=False)
    dense = replace(mid, name="test-dense", mlp_map=("dense",) * 4)
    return {"tiny": tiny, "mid": mid, "dense": dense}


@pytest.mark.parametrize("name", ["tiny", "mid", "dense"])
def test_loss_and_grads_match_torch_path(name, monkeypatch):
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.params import tree_dict
    from lyra_b200.ops import native
    from lyra_b200.training.steps import loss_parts

    cfg = _cfgs()[name]
    torch.manual_seed(0)
    tokens = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
    labels = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
    results = {}
    import lyra_b200.model as M

    tape = {"replay": False, "choices": []}    # the kernel path takes the experts the PyTorch path chose: no top-k flips between them
    monkeypatch.setattr(M, "ROUTING_TAPE", tape)
    for impl in ("torch", "auto"):
        tape["replay"] = impl == "auto"
        c = replace(cfg, implementation=impl)
        w = ModelWeights.init(1, c, device="cuda")
        leaves = tree_dict(w)
        # break the symmetry of zero-initialised parameters so every path carries signal
        g = torch.Generator(device="cuda").manual_seed(5)
        for p, t in leaves.items():
            if p.endswith(("sinks", "xsa_alpha", "sdpa_gate", "router_bias")):
                t.copy_(torch.randn(t.shape, device="cuda", generator=g) * 0.3)
            t.requires_grad_(True)
        ce, aux = loss_parts(w, tokens, labels, c)
        loss = ce.float() / tokens.numel() + aux
        loss.backward()
        results[impl] = (loss.item(), {p: t.grad.float().clone() for p, t in leaves.items() if t.grad is not None})
    native.check_status()
    (l0, g0), (l1, g1) = results["torch"], results["auto"]
    assert abs(l0 - l1) < 2e-2 * max(1.0, abs(l0)), (l0, l1)
    assert set(g0) == set(g1)
    bad = []
    for p in g0:
        denom = g0[p].norm().clamp_min(1e-6)
        err = ((g0[p] - g1[p]).norm() / denom).item()
        if err > TOLERANCE:
            bad.append((p, round(err, 4)))
    assert not bad, bad


def test_moe_experts_op():
    """Grouped expert MLP with fixed routing: outputs and every gradient (incl. the routing scores) vs the PyTorch statement."""
    from lyra_b200.ops import api

    torch.manual_seed(0)
    F_, K, E, C, H = 300, 3, 5, 256, 384
    xn = torch.randn(F_, C, device="cuda").bfloat16()
    indices = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(F_)])
    scores = torch.softmax(torch.randn(F_, K, device="cuda"), -1)
    w_up = (torch.randn(E, C, 2, H, device="cuda") / 16)
    w_down = (torch.randn(E, H, C, device="cuda") / 16)
    dout = (torch.randn(F_, C, device="cuda") * 0.1).bfloat16()
    res = {}
    for impl in ("torch", "auto"):
        a = [t.clone().requires_grad_(True) for t in (xn, scores, w_up, w_down)]
        out = api.moe_experts(a[0], a[1], indices, a[2], None, a[3], None, 1.702, 7.0, impl)
        out.backward(dout)
        res[impl] = [out.detach().float()] + [t.grad.float() for t in a]
    for name, r, k in zip(("out", "dx", "dscores", "dw_up", "dw_down"), res["torch"], res["auto"]):
        err = ((r - k).norm() / r.norm().clamp_min(1e-9)).item()
        assert err < 3e-2, (name, err)
