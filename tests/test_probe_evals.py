import torch

from lyra_b200.evals.common import Doc, Scorer, evaluate
from lyra_b200.model import ModelWeights, model_apply
from lyra_b200.training.probe import Level, Probe, swiglu_stats, to_floats
from tests.helpers import small_config


def test_probing_changes_neither_outputs_nor_gradients():
    c = small_config(compute_dtype=torch.float32)
    tokens = torch.randint(0, 500, (2, 16))
    outs = []
    for probe in (None, Probe(level=Level.FULL)):
        w = ModelWeights.init(0, c)
        w.layers[0].attn.q.requires_grad_(True)
        kw = {} if probe is None else {"probe": probe}
        if probe is not None:
            probe.start()
        h, aux, _ = model_apply(tokens, w, None, c, return_hidden_states=True, **kw)
        (h.float().pow(2).mean() + aux).backward()
        outs.append((h.detach(), w.layers[0].attn.q.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    rec = to_floats(probe.collect())
    assert "layer.01.mlp.routing" in rec and "layer.01.mlp.aux_loss" in rec and "head.logits_subsample" in rec
    assert {"load_max_ratio", "load_min_ratio", "token_entropy"} <= set(rec["layer.01.mlp.routing"])
    assert {"branch_ratio", "growth", "branch_absorbed_frac"} <= set(rec["layer.00.attn.residual"])


def test_routing_only_probe_records_just_routing():
    c = small_config()
    probe = Probe(routing_only=True)
    probe.start()
    model_apply(torch.randint(0, 500, (1, 16)), ModelWeights.init(0, c), None, c, return_hidden_states=True, probe=probe)
    keys = set(probe.collect())
    assert keys == {"layer.01.mlp.routing", "layer.01.mlp.aux_loss", "layer.03.mlp.routing", "layer.03.mlp.aux_loss"}


def test_swiglu_clip_stats_golden():
    x = torch.tensor([[8.0, 1.0, -9.0, 2.0, 10.0, -8.0, 0.0, 1.0]])  # gate half then value half
    s = swiglu_stats(x, 7.0)
    assert float(s["gate_clip_frac"]) == 0.25 and float(s["value_clip_frac"]) == 0.5


def test_scorer_masks_only_the_continuation_and_evaluate_scores():
    c = small_config(vocab_size=201088, padded_vocab_size=204800, n_layers=1, mlp_map=("dense",), seq_len=64)
    scorer = Scorer(ModelWeights.init(0, c), c, batch_size=4)
    docs = [Doc("Question: 1+1?\nAnswer:", ("2", "3", "4"), 0, True), Doc("Question: sky?\nAnswer:", ("blue", "green"), 0, True)]
    reqs = scorer.requests(docs)
    assert len(reqs) == 5 and all(r.ids[0] == scorer.tokenizer.eos_token for r in reqs)
    assert [(r.doc, r.choice) for r in reqs] == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1)]
    tok = scorer.tokenizer
    assert all(tok.decode(r.ids[r.scored_from:]) == " " + docs[r.doc].choices[r.choice] for r in reqs)   # only the choice is scored
    # a context that does not fit loses tokens from the left; the continuation is kept whole
    long_doc = Doc("word " * 200 + "Answer:", ("yes",), 0)
    (r,) = scorer.requests([long_doc])
    assert len(r.ids) == c.seq_len and tok.decode(r.ids[r.scored_from:]) == " yes"
    # the order in which requests are batched does not change a request's score
    one_by_one = Scorer(scorer.model, c, batch_size=1).score(docs)
    together = scorer.score(docs)
    assert all(abs(a - b) < 1e-3 * max(1.0, abs(a)) for x, y in zip(one_by_one, together) for a, b in zip(x, y))
    res = evaluate("toy", docs, scorer)
    assert res.num_docs == 2 and 0.0 <= res.acc <= 1.0 and res.acc_norm is not None
    assert "acc_norm" in str(res)
