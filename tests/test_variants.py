import pytest

from lyra_b200.config import flops_per_token
from lyra_b200.model import ModelWeights
from lyra_b200.nn.params import param_count
from lyra_b200.tokenizer import PADDED_VOCAB_SIZE
from lyra_b200.variants import MODEL_VARIANTS, model_variant


@pytest.mark.parametrize("name", list(MODEL_VARIANTS))
def test_variant_invariants(name):
    c = model_variant(name)
    assert len(c.mlp_map) == c.n_layers
    assert c.n_experts == c.n_routed_experts + c.n_shared_experts
    assert 0 < c.n_active_routed_experts <= c.n_routed_experts
    assert c.n_attn_heads % c.n_kv_heads == 0
    assert c.n_attn_heads % c.sharding.model_axis_size == 0 and c.n_kv_heads % c.sharding.model_axis_size == 0
    assert c.n_experts % c.sharding.expert_axis_size == 0
    assert c.expert_hidden % c.sharding.model_axis_size == 0
    assert c.padded_vocab_size >= c.vocab_size and c.padded_vocab_size == PADDED_VOCAB_SIZE


def test_unknown_variant():
    with pytest.raises(ValueError, match="Unknown model variant"):
        model_variant("nope")


def test_parameter_counts_and_flops_match_published_figures():
    counts = {n: param_count(ModelWeights.spec(model_variant(n))) for n in ("lyra-small", "lyra-medium", "lyra-max", "gpt-oss-120b")}
    assert round(counts["lyra-small"] / 1e9, 2) == 1.62
    assert round(counts["lyra-medium"] / 1e9, 2) == 17.72
    assert round(counts["lyra-max"] / 1e9, 2) == 99.87
    assert round(counts["gpt-oss-120b"] / 1e9, 2) == 116.85
    assert int(flops_per_token(model_variant("lyra-small"))) == 6_475_926_528
    assert int(flops_per_token(model_variant("lyra-medium"))) == 35_271_684_096
    assert int(flops_per_token(model_variant("lyra-max"))) == 52_223_471_616


def test_moe_layer_placement_is_one_based():
    c = model_variant("lyra-small")
    assert [i for i, k in enumerate(c.mlp_map) if k == "moe"] == [3, 7, 11, 15]
    assert c.layer_window(0) == 128 and c.layer_window(1) == 0
