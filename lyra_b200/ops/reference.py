"""Plain PyTorch statements of every op: the CPU path, the oracle of the CUDA kernels' tests and the
``implementation="torch"`` baseline mode. Semantics follow the reference's ``*_reference`` functions
(lyra/kernels/flash_attention.py:706-747, cross_entropy.py, gemm.py:477-499, common.py:98-114).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 RMS normalisation, result in the input dtype (lyra/model.py:189-191)."""
    t = x.float()
    return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * scale.float()).to(x.dtype)


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotary embedding (lyra/model.py:183-186). ``cos``/``sin`` broadcast against ``x[..., :hd/2]``."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def swiglu(x: torch.Tensor, beta: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """Clamped SwiGLU over ``x[..., 2, H]`` (gate half, linear half): ``(lin + 1) * gate * sigmoid(beta * gate)``
    with ``gate = min(g, limit)`` and ``lin = clip(l, -limit, limit)`` (lyra/kernels/common.py:98-114)."""
    gate, lin = x[..., 0, :], x[..., 1, :]
    gate = gate.clamp(max=limit)
    lin = lin.clamp(min=-limit, max=limit)
    return (lin + 1.0) * gate * torch.sigmoid(beta * gate)


def attention_mask(q_len: int, kv_len: int, window: int, q_start, device) -> torch.Tensor:
    """Boolean ``[q_len, kv_len]``: causal, and for sliding layers ``col > row - window``
    (lyra/kernels/flash_attention.py:189-205). ``q_start`` is the absolute position of query row 0."""
    rows = torch.arange(q_len, device=device)[:, None] + q_start
    cols = torch.arange(kv_len, device=device)[None, :]
    mask = cols <= rows
    if window > 0:
        mask &= cols > rows - window
    return mask


def attention(q, k, v, sinks, scale: float, window: int = 0, q_start=0):
    """GQA attention with a learned sink per query head.

    ``q [B, Nq, T, D]``, ``k, v [B, Nkv, S, D]``, ``sinks [Nq]``. The softmax denominator includes
    ``exp(sink_h)`` with no value contribution. Returns ``(out [B, Nq, T, D] in q.dtype, lse [B, Nq, T] fp32)``.
    """
    B, Nq, T, D = q.shape
    Nkv, S = k.shape[1], k.shape[2]
    rep = Nq // Nkv
    qf = q.float().view(B, Nkv, rep, T, D)
    logits = torch.einsum("bkrtd,bksd->bkrts", qf, k.float()) * scale
    mask = attention_mask(T, S, window, q_start, q.device)
    logits = logits.masked_fill(~mask, float("-inf"))
    sink = sinks.float().view(1, Nkv, rep, 1, 1).expand(B, Nkv, rep, T, 1)
    full = torch.cat([logits, sink], dim=-1)
    lse = torch.logsumexp(full, dim=-1)
    probs = torch.exp(logits - lse[..., None])
    out = torch.einsum("bkrts,bksd->bkrtd", probs, v.float())
    return out.view(B, Nq, T, D).to(q.dtype), lse.view(B, Nq, T)


def linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, vocab_size: int, reduction: str = "sum",
                         chunk: int = 4096):
    """Cross entropy of ``x [T, C] @ w[V, C]^T`` against ``y [T]`` without keeping ``[T, V]`` logits alive:
    rows are processed in chunks. Columns ``>= vocab_size`` (vocabulary padding) are excluded
    (lyra/kernels/cross_entropy.py:162-165). Differentiable through autograd; returns ``(loss, lse [T])``."""
    losses, lses = [], []
    wv = w[:vocab_size]
    for s in range(0, x.shape[0], chunk):
        logits = (x[s:s + chunk] @ wv.t().to(x.dtype)).float()
        lse = torch.logsumexp(logits, dim=-1)
        tgt = logits.gather(1, y[s:s + chunk, None].long())[:, 0]
        losses.append((lse - tgt).sum())
        lses.append(lse)
    loss = torch.stack(losses).sum()
    if reduction == "mean":
        loss = loss / x.shape[0]
    return loss, torch.cat(lses)


def grouped_gemm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``out[m] = lhs[m] @ rhs[g(m)]`` for rows sorted by group (lyra/kernels/gemm.py:477-499)."""
    out = lhs.new_empty(lhs.shape[0], rhs.shape[-1])
    start = 0
    for g, n in enumerate(group_sizes.tolist()):
        if n:
            seg = lhs[start:start + n] @ rhs[g].to(lhs.dtype)
            if bias is not None:
                seg = seg + bias[g].to(seg.dtype)
            out[start:start + n] = seg
        start += n
    if start < lhs.shape[0]:
        out[start:] = 0
    return out


def grouped_gemm_autograd(lhs, rhs, group_sizes, bias=None):
    """Differentiable version of :func:`grouped_gemm` (list of per-group matmuls concatenated)."""
    outs, start = [], 0
    for g, n in enumerate(group_sizes.tolist()):
        seg = lhs[start:start + n] @ rhs[g].to(lhs.dtype)
        if bias is not None:
            seg = seg + bias[g].to(seg.dtype)
        outs.append(seg)
        start += n
    if start < lhs.shape[0]:
        outs.append(lhs.new_zeros(lhs.shape[0] - start, rhs.shape[-1]))
    return torch.cat(outs, dim=0)


def combine(experts_out: torch.Tensor, scores: torch.Tensor, unpermute_map: torch.Tensor) -> torch.Tensor:
    """``out[f] = sum_k scores[f, k] * experts_out[unpermute_map[f*K + k]]`` (lyra/model.py:557)."""
    F_, K = scores.shape
    rows = experts_out[unpermute_map.long()].view(F_, K, -1)
    return torch.einsum("fkc,fk->fc", rows.float(), scores.float()).to(experts_out.dtype)


def embedding_grad(tokens: torch.Tensor, grad: torch.Tensor, vocab: int) -> torch.Tensor:
    """Deterministic embedding gradient: sort token ids, segment-sum in fp32 (lyra/kernels/embs.py:22-29)."""
    flat = tokens.reshape(-1).long()
    g = grad.reshape(flat.shape[0], -1).float()
    order = torch.argsort(flat, stable=True)
    out = torch.zeros(vocab, g.shape[1], dtype=torch.float32, device=g.device)
    out.index_add_(0, flat[order], g[order])
    return out


def softcap_free_topk(logits: torch.Tensor, k: int):
    """``lax.top_k`` semantics: values descending, ties resolved towards the lower index."""
    vals, idx = torch.sort(logits, dim=-1, descending=True, stable=True)
    return vals[..., :k], idx[..., :k]


def yarn_concentration(rope_scale: float) -> float:
    return 0.1 * math.log(rope_scale) + 1.0 if rope_scale > 1.0 else 1.0


def count_ids(ids: torch.Tensor, n: int) -> torch.Tensor:
    """``bincount(ids, minlength=n)`` without the device-to-host synchronisation ``torch.bincount`` needs to size its
    output (integer scatter-add: exact and order-independent)."""
    out = torch.zeros(n, dtype=torch.int64, device=ids.device)
    return out.scatter_add_(0, ids.reshape(-1).long(), torch.ones(ids.numel(), dtype=torch.int64, device=ids.device))
