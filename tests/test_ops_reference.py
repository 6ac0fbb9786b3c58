"""The PyTorch oracle ops (the CPU path and the yardstick of every kernel test) against independent formulations."""

import torch

from lyra_b200.ops import reference as ref


def test_combine_is_the_weighted_sum_of_the_selected_rows_and_differentiable():
    torch.manual_seed(0)
    F_, K, C = 5, 3, 8
    rows = torch.randn(F_ * K + 4, C, requires_grad=True)
    scores = torch.rand(F_, K, requires_grad=True)
    unperm = torch.randperm(F_ * K + 4)[: F_ * K]
    out = ref.combine(rows, scores, unperm)
    want = torch.stack([sum(scores[f, k] * rows[unperm[f * K + k]] for k in range(K)) for f in range(F_)])
    assert torch.allclose(out, want, atol=1e-6)
    g = torch.randn_like(out)
    d_rows, d_scores = torch.autograd.grad(out, (rows, scores), g)
    assert torch.allclose(d_scores[2, 1], (rows[unperm[2 * K + 1]] * g[2]).sum(), atol=1e-5)
    assert torch.allclose(d_rows[unperm[4 * K]], scores[4, 0] * g[4], atol=1e-6)
    untouched = torch.ones(rows.shape[0], dtype=torch.bool)
    untouched[unperm] = False
    assert (d_rows[untouched] == 0).all()


def test_swiglu_clamps_gate_from_above_and_linear_on_both_sides():
    x = torch.tensor([[[10.0, -10.0, 1.0], [9.0, -9.0, 0.5]]])          # [1, 2, H]: gate row, linear row
    out = ref.swiglu(x, beta=1.702, limit=7.0)
    gate = torch.tensor([7.0, -10.0, 1.0])
    lin = torch.tensor([7.0, -7.0, 0.5])
    want = (lin + 1) * gate * torch.sigmoid(1.702 * gate)
    assert torch.allclose(out[0], want, atol=1e-6)


def test_grouped_gemm_matches_per_group_matmuls_with_empty_groups_and_tail():
    torch.manual_seed(1)
    lhs = torch.randn(10, 4)
    rhs = torch.randn(4, 4, 6)
    bias = torch.randn(4, 6)
    sizes = torch.tensor([3, 0, 5, 1])                                    # one empty group, one unused tail row
    out = ref.grouped_gemm(lhs, rhs, sizes, bias)
    assert torch.allclose(out[:3], lhs[:3] @ rhs[0] + bias[0], atol=1e-6)
    assert torch.allclose(out[3:8], lhs[3:8] @ rhs[2] + bias[2], atol=1e-6)
    assert torch.allclose(out[8:9], lhs[8:9] @ rhs[3] + bias[3], atol=1e-6)
    assert (out[9:] == 0).all()
    assert torch.allclose(ref.grouped_gemm_autograd(lhs, rhs, sizes, bias), out, atol=1e-6)


def test_linear_cross_entropy_masks_the_vocabulary_padding_and_matches_torch():
    torch.manual_seed(2)
    T, C, V, pad = 37, 16, 50, 14
    x = torch.randn(T, C, requires_grad=True)
    w = torch.randn(V + pad, C, requires_grad=True)
    y = torch.randint(0, V, (T,))
    loss, lse = ref.linear_cross_entropy(x, w, y, V, reduction="mean", chunk=8)
    logits = x @ w[:V].t()
    want = torch.nn.functional.cross_entropy(logits, y)
    assert torch.allclose(loss, want, atol=1e-5)
    assert torch.allclose(lse, torch.logsumexp(logits, -1), atol=1e-5)
    (gw,) = torch.autograd.grad(loss, w)
    assert (gw[V:] == 0).all()                                            # padded rows of the output embedding get no gradient


def test_embedding_grad_sums_repeated_tokens_and_count_ids():
    tokens = torch.tensor([[1, 3, 1], [0, 3, 3]])
    grad = torch.arange(6 * 2, dtype=torch.float32).view(2, 3, 2)
    out = ref.embedding_grad(tokens, grad, vocab=5)
    flat = grad.view(6, 2)
    assert torch.equal(out[1], flat[0] + flat[2]) and torch.equal(out[3], flat[1] + flat[4] + flat[5])
    assert torch.equal(out[0], flat[3]) and (out[2] == 0).all() and (out[4] == 0).all()
    assert ref.count_ids(tokens.reshape(-1), 5).tolist() == [1, 2, 0, 3, 0]


def test_topk_breaks_ties_towards_the_lower_index():
    vals, idx = ref.softcap_free_topk(torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0]]), 3)
    assert idx.tolist() == [[1, 2, 4]] and vals.tolist() == [[3.0, 3.0, 3.0]]


def test_sink_is_a_softmax_column_without_a_value():
    torch.manual_seed(3)
    q, k, v = torch.randn(1, 2, 4, 8), torch.randn(1, 1, 4, 8), torch.randn(1, 1, 4, 8)
    big = ref.attention(q, k, v, torch.full((2,), 30.0), 8 ** -0.5)[0]     # a dominant sink absorbs the probability mass
    none = ref.attention(q, k, v, torch.full((2,), -30.0), 8 ** -0.5)[0]
    assert big.abs().max() < 1e-6 < none.abs().max()
    s = torch.einsum("bhtd,bsd->bhts", q, k[:, 0]) * 8 ** -0.5
    s = s.masked_fill(~torch.tril(torch.ones(4, 4, dtype=torch.bool)), float("-inf"))
    assert torch.allclose(none, torch.softmax(s, -1) @ v[:, 0], atol=1e-5)
