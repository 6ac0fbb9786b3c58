import torch

from lyra_b200.config import ModelConfig
from lyra_b200.gpt_oss import dequantize_mxfp4, load_gpt_oss_model, quantize_mxfp4, write_random_gpt_oss_checkpoint
from lyra_b200.model import model_apply


def _config():
    return ModelConfig(name="Tiny GPT-OSS", seq_len=16, n_embd=32, n_layers=1, mlp_map=("moe",), vocab_size=16, padded_vocab_size=32, head_dim=4,
                       n_attn_heads=2, n_kv_heads=1, sliding_window=4, n_routed_experts=2, n_shared_experts=0, n_active_experts=1,
                       expert_mlp_widening=2.0, rope_scale=32.0, tie_embeddings=False, use_qk_norm=False, use_qkv_bias=True,
                       use_attn_out_bias=True, use_mlp_bias=True, use_router_bias=True, param_dtype=torch.bfloat16, implementation="torch")


def test_mxfp4_codec():
    blocks = torch.full((2, 3, 1, 16), 0x22, dtype=torch.uint8)
    assert (dequantize_mxfp4(blocks, torch.full((2, 3, 1), 127, dtype=torch.uint8)) == 1.0).all()
    assert (dequantize_mxfp4(blocks, torch.full((2, 3, 1), 128, dtype=torch.uint8)) == 2.0).all()
    x = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -6.0] * 16)[:128].reshape(1, 128)
    b, s = quantize_mxfp4(x)
    assert torch.equal(dequantize_mxfp4(b, s).float(), x)


def test_load_checks_layout_transposes_and_padding(tmp_path):
    from safetensors.torch import save_file

    c = _config()
    q_dim, kv = c.n_attn_heads * c.head_dim, c.n_kv_heads * c.head_dim
    qkv, H2, H = q_dim + 2 * kv, int(c.n_embd * c.expert_mlp_widening), c.expert_hidden
    bf = torch.bfloat16
    ar = lambda *s: torch.arange(int(torch.tensor(s).prod()), dtype=torch.float32).reshape(*s).to(bf)
    t = {
        "embedding.weight": ar(c.vocab_size, c.n_embd), "unembedding.weight": ar(c.vocab_size, c.n_embd), "norm.scale": torch.ones(c.n_embd, dtype=bf),
        "block.0.attn.norm.scale": torch.ones(c.n_embd, dtype=bf), "block.0.attn.out.bias": ar(c.n_embd), "block.0.attn.out.weight": ar(c.n_embd, q_dim),
        "block.0.attn.qkv.bias": ar(qkv), "block.0.attn.qkv.weight": ar(qkv, c.n_embd), "block.0.attn.sinks": ar(c.n_attn_heads),
        "block.0.mlp.gate.bias": ar(c.n_experts), "block.0.mlp.gate.weight": ar(c.n_experts, c.n_embd), "block.0.mlp.norm.scale": torch.ones(c.n_embd, dtype=bf),
        "block.0.mlp.mlp1_bias": torch.zeros(c.n_experts, H2, dtype=bf),
        "block.0.mlp.mlp1_weight.blocks": torch.full((c.n_experts, H2, c.n_embd // 32, 16), 0x22, dtype=torch.uint8),
        "block.0.mlp.mlp1_weight.scales": torch.full((c.n_experts, H2, c.n_embd // 32), 127, dtype=torch.uint8),
        "block.0.mlp.mlp2_bias": torch.zeros(c.n_experts, c.n_embd, dtype=bf),
        "block.0.mlp.mlp2_weight.blocks": torch.full((c.n_experts, c.n_embd, H // 32, 16), 0x22, dtype=torch.uint8),
        "block.0.mlp.mlp2_weight.scales": torch.full((c.n_experts, c.n_embd, H // 32), 127, dtype=torch.uint8),
    }
    (tmp_path / "original").mkdir()
    save_file(t, str(tmp_path / "original" / "model.safetensors"))
    w = load_gpt_oss_model(tmp_path, c)
    a, m = w.layers[0].attn, w.layers[0].mlp
    assert w.tok.emb.shape == (32, 32) and (w.tok.emb[16:] == 0).all()
    assert torch.equal(a.q, t["block.0.attn.qkv.weight"][:q_dim].T) and torch.equal(a.v, t["block.0.attn.qkv.weight"][q_dim + kv:].T)
    assert torch.equal(a.k_bias, t["block.0.attn.qkv.bias"][q_dim:q_dim + kv]) and torch.equal(a.out, t["block.0.attn.out.weight"].T)
    assert m.mlp_up.shape == (2, 32, 2, H) and m.mlp_up.dtype == bf and (m.mlp_up == 1).all() and (m.mlp_down == 1).all()
    assert m.router.shape == (32, 2) and m.mlp_up_bias.shape == (2, 2, H)
    logits, _, _ = model_apply(torch.arange(8)[None] % 16, w, None, c)
    assert torch.isinf(logits[..., 16:]).all()


def test_random_checkpoint_writer_round_trips(tmp_path):
    c = _config()
    write_random_gpt_oss_checkpoint(tmp_path, c, seed=1)
    w = load_gpt_oss_model(tmp_path, c)
    logits, _, _ = model_apply(torch.arange(8)[None] % 16, w, None, c)
    assert torch.isfinite(logits[..., :16]).all()
    half = load_gpt_oss_model(tmp_path, c, expert_slice=(1, 2))
    assert torch.equal(half.layers[0].mlp.mlp_up[0], w.layers[0].mlp.mlp_up[1])
