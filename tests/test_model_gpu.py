"""End-to-end: the kernel path (implementation="auto") against the PyTorch path on the same GPU."""

from dataclasses import replace

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfgs():
    from lyra_b200.config import ModelConfig, full_moe
    from lyra_b200.variants import model_variant

    tiny = replace(model_variant("tiny"), vocab_size=2048, padded_vocab_size=2304)
    mid = ModelConfig(name="test-mid", seq_len=256, n_embd=512, n_layers=4, head_dim=128, n_attn_heads=4, n_kv_heads=2,
                      use_learned_xsa=True, use_sdpa_output_gate=True, n_routed_experts=7, n_shared_experts=1, n_active_experts=3,
                      mlp_map=("dense", "moe", "dense", "moe"), vocab_size=4000, padded_vocab_size=4096, tie_embeddings=False)
    return {"tiny": tiny, "mid": mid}


@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_loss_and_grads_match_torch_path(name):
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.params import tree_dict
    from lyra_b200.ops import native
    from lyra_b200.training.steps import loss_parts

    cfg = _cfgs()[name]
    torch.manual_seed(0)
    tokens = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
    labels = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len), device="cuda")
    results = {}
    for impl in ("torch", "auto"):
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
        if err > 0.08:
            bad.append((p, err))
    assert not bad, bad
