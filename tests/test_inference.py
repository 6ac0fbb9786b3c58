from dataclasses import replace

import pytest
import torch

from lyra_b200.generate import InferenceConfig, apply_inference_overrides, sample_token, sample_tokens, serve_model
from lyra_b200.model import ModelCache, ModelWeights, model_apply
from lyra_b200.nn.quant import QArray, dequantize, quantize, qupdate
from tests.helpers import small_config


def test_inference_overrides():
    c = small_config()
    o = apply_inference_overrides(c, InferenceConfig(weights="x", fp8=True, temperature=0.0, top_k=7))
    assert o.quantize_mlp and o.quantize_cache and not o.quantize_attn and o.gemm_dtype == torch.float8_e4m3fn
    assert o.sample_temperature == 0.0 and o.sample_topk == 7


def test_quantize_round_trip_and_zero_blocks():
    torch.manual_seed(0)
    x = torch.randn(4, 64, 96)
    x[0, :32, :32] = 0
    q = quantize(x, torch.float8_e4m3fn, (32, 32))
    assert q.scale.shape == (4, 2, 3) and q.scale[0, 0, 0] == 1.0
    assert (dequantize(q, torch.float32) - x).abs().max() < 0.07 * x.abs().max()
    with pytest.raises(ValueError):
        quantize(x, torch.float8_e4m3fn, (48, 32))
    with pytest.raises(ValueError):
        quantize(x, torch.bfloat16)


def test_qupdate_writes_values_and_scales_in_place():
    cache = quantize(torch.zeros(1, 2, 8, 16), torch.float8_e4m3fn, (1, 16))
    new = torch.randn(1, 2, 3, 16)
    out = qupdate(cache, new, (0, 0, 4, 0))
    assert isinstance(out, QArray) and out.qval.data_ptr() == cache.qval.data_ptr()
    d = dequantize(out, torch.float32)
    assert (d[:, :, 4:7] - new).abs().max() < 0.1 * new.abs().max() and d[:, :, :4].abs().max() == 0
    with pytest.raises(ValueError):
        qupdate(quantize(torch.zeros(4, 64, 64), torch.float8_e4m3fn, (32, 32)), torch.zeros(4, 32, 32), (0, 5, 0))


def test_greedy_is_argmax_and_topk_samples_stay_in_the_topk_set():
    c = small_config(sample_temperature=0.0)
    logits = torch.tensor([0.1, 2.0, -1.0, 2.0, 0.5])
    assert int(sample_token(logits, None, c)) == 1  # ties resolve to the lower index
    c = replace(c, sample_temperature=1.0, sample_topk=2)
    g = torch.Generator().manual_seed(0)
    picks = {int(sample_token(logits, g, c)) for _ in range(50)}
    assert picks <= {1, 3} and len(picks) == 2


def test_fp8_model_and_cache_generate_finite_tokens_deterministically():
    c = apply_inference_overrides(small_config(head_dim=8, quant_block=(8, 8)), InferenceConfig(weights="x", fp8=True))
    w = ModelWeights.quantize(ModelWeights.init(0, c), c)
    assert isinstance(w.layers[1].mlp.mlp_up, QArray) and isinstance(w.layers[0].mlp.mlp_down, QArray)
    a = sample_tokens(w, (c.seed, 0), c, [199 % 500, 5, 9, 11], 6)
    b = sample_tokens(w, (c.seed, 0), c, [199 % 500, 5, 9, 11], 6)
    assert a == b and len(a) == 6 and all(0 <= t < c.vocab_size for t in a)
    cache = ModelCache.create(c, 1, 16, "cpu")
    assert isinstance(cache.layers[0].k, QArray) and cache.layers[0].k.scale.shape == (1, c.n_kv_heads, 16, 1)


def test_serve_repl_plain_chat(monkeypatch):
    c = small_config(vocab_size=201088, padded_vocab_size=204800, n_layers=1, mlp_map=("dense",), sample_temperature=0.0)
    w = ModelWeights.init(0, c)
    prompts = iter(["hi", "", "exit"])
    printed = []
    serve_model(w, c, InferenceConfig(weights="x", max_new_tokens=3, max_cache_length=24), input_fn=lambda _: next(prompts),
                output_fn=lambda *a, **k: printed.append(a))
    assert printed and "Type a prompt" in printed[0][0]


@pytest.mark.parametrize("fp8_cache", [False, True])
def test_decode_with_device_resident_position_matches_host_position(fp8_cache):
    """The position of a single-token decode step may live in a device scalar (what CUDA-graph replay needs)."""
    from dataclasses import replace

    from lyra_b200.generate import BatchedGenerator
    from lyra_b200.model import ModelWeights
    from lyra_b200.variants import model_variant

    c = replace(model_variant("dev"), sample_temperature=0.0, quantize_cache=fp8_cache)
    m = ModelWeights.init(0, c)
    B, P, N = 2, 8, 5
    prompts = torch.randint(0, c.vocab_size, (B, P), generator=torch.Generator().manual_seed(0))
    g = BatchedGenerator(m, c, batch=B, capacity=P + N, device="cpu")
    want = g.decode(g.prefill(prompts), N)
    g2 = BatchedGenerator(m, c, batch=B, capacity=P + N, device="cpu")
    tok = g2.prefill(prompts)
    g2.cache.pos_dev = torch.tensor([g2.cache.pos], dtype=torch.int32)
    got = [tok]
    for _ in range(N - 1):
        tok = g2.decode_step(tok)
        g2.cache.pos_dev += 1
        got.append(tok)
    assert torch.equal(want, torch.stack(got, dim=1))
