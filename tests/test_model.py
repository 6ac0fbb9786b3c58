from dataclasses import replace

import torch

from lyra_b200.model import ModelWeights, model_apply
from lyra_b200.variants import model_variant
from tests.helpers import small_config


def test_dev_forward_shapes_padding_and_determinism():
    c = replace(model_variant("dev"), implementation="torch")
    w = ModelWeights.init(0, c)
    tokens = torch.randint(0, c.vocab_size, (1, 24))
    logits, aux, cache = model_apply(tokens, w, None, c)
    assert logits.shape == (1, 24, c.padded_vocab_size) and cache is None
    assert torch.isfinite(logits[..., : c.vocab_size]).all()
    assert torch.isinf(logits[..., c.vocab_size:]).all() and (logits[..., c.vocab_size:] < 0).all()
    assert aux.item() >= 0
    again, _, _ = model_apply(tokens, w, None, c)
    assert torch.equal(logits, again)


def test_hidden_states_path_returns_normed_hidden():
    c = small_config()
    w = ModelWeights.init(0, c)
    h, aux, _ = model_apply(torch.randint(0, 500, (2, 16)), w, None, c, return_hidden_states=True)
    assert h.shape == (2, 16, c.n_embd) and h.dtype == c.compute_dtype


def test_attention_gate_starts_as_identity_and_learns():
    c = small_config(n_layers=2, mlp_map=("dense", "dense"), compute_dtype=torch.float32)
    tokens = torch.arange(8)[None]
    base = ModelWeights.init(0, c)
    base_logits, _, _ = model_apply(tokens, base, None, c)
    gc = replace(c, use_sdpa_output_gate=True)
    gated = ModelWeights.init(0, gc)
    assert torch.equal(base.tok.emb, gated.tok.emb)
    for a, b in zip(base.layers, gated.layers):
        assert torch.equal(a.attn.q, b.attn.q) and torch.equal(a.mlp.mlp_up, b.mlp.mlp_up)
        assert (b.attn.sdpa_gate == 0).all()
    gate_logits, _, _ = model_apply(tokens, gated, None, gc)
    assert torch.equal(base_logits, gate_logits)
    g = gated.layers[0].attn.sdpa_gate.requires_grad_(True)
    loss = model_apply(tokens, gated, None, gc)[0][..., : c.vocab_size].pow(2).mean()
    loss.backward()
    assert g.grad.norm() > 0
    with torch.no_grad():
        g -= 0.01 * g.grad
    assert model_apply(tokens, gated, None, gc)[0][..., : c.vocab_size].pow(2).mean() < loss


def test_sliding_window_and_sink_semantics():
    from lyra_b200.ops import reference as ref

    torch.manual_seed(0)
    q, k, v = torch.randn(1, 2, 6, 4), torch.randn(1, 1, 6, 4), torch.randn(1, 1, 6, 4)
    out, lse = ref.attention(q, k, v, torch.zeros(2), 0.5, window=2)
    # row 5 of a window-2 layer sees keys 4 and 5 only, plus the sink column
    logits = (q[0, 0, 5] @ k[0, 0, 4:6].t()) * 0.5
    p = torch.softmax(torch.cat([logits, torch.zeros(1)]), 0)
    assert torch.allclose(out[0, 0, 5], p[:2] @ v[0, 0, 4:6], atol=1e-6)
    assert torch.allclose(lse[0, 0, 5], torch.logsumexp(torch.cat([logits, torch.zeros(1)]), 0), atol=1e-6)
    # a very negative sink recovers plain softmax attention
    plain, _ = ref.attention(q, k, v, torch.full((2,), -1e9), 0.5, window=0)
    expect = torch.nn.functional.scaled_dot_product_attention(q, k.expand(1, 2, 6, 4), v.expand(1, 2, 6, 4), is_causal=True, scale=0.5)
    assert torch.allclose(plain, expect, atol=1e-5)


def test_prefill_then_decode_matches_full_forward():
    from lyra_b200.config import Mode
    from lyra_b200.model import ModelCache

    c = small_config(compute_dtype=torch.float32, sliding_window=8)
    w = ModelWeights.init(0, c)
    tokens = torch.randint(0, 500, (1, 12))
    full, _, _ = model_apply(tokens, w, None, c)
    cache = ModelCache.create(replace(c, mode=Mode.PREFILL), 1, 16, "cpu")
    pre, _, cache = model_apply(tokens[:, :9], w, cache, replace(c, mode=Mode.PREFILL))
    assert torch.allclose(pre[..., :500], full[:, :9, :500], atol=1e-4)
    for t in range(9, 12):
        step, _, cache = model_apply(tokens[:, t:t + 1], w, cache, replace(c, mode=Mode.DECODE))
        assert torch.allclose(step[0, 0, :500], full[0, t, :500], atol=1e-4)
    assert cache.pos == 12
