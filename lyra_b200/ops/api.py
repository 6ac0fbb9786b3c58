"""Op dispatch: one entry per logical op, resolved to the sm_100a kernel or the PyTorch statement.

``implementation``:
  * ``"auto"``  - hand-written kernels when the tensors are on a CUDA device, PyTorch otherwise;
  * ``"b200"``  - kernels only (an unsupported shape is an error);
  * ``"torch"`` / ``"nccl"`` - PyTorch library ops (and NCCL collectives in the parallel layer): the
    oracle and the stand-in baseline.

Like the reference's ``dispatch_kernel`` (lyra/kernels/common.py:117-155) every resolution is logged once
per (op, shape, implementation) on stderr; ``LYRA_LOG_KERNELS=0`` silences it.
"""

from __future__ import annotations

import os
import sys

import torch

from lyra_b200.ops import native
from lyra_b200.ops import reference as ref

_LOG_SEEN: set[str] = set()


def log_kernel_resolution(op: str, shape: str, impl: str, tiling: str | None = None) -> None:
    if os.environ.get("LYRA_LOG_KERNELS", "1") == "0":
        return
    key = f"{op}|{shape}|{impl}|{tiling}"
    if key in _LOG_SEEN:
        return
    _LOG_SEEN.add(key)
    detail = impl if tiling is None else f"{impl:<6} {tiling}"
    print(f"[kernel] {op:<15} {shape:<26} -> {detail}", file=sys.stderr)


def use_kernels(t: torch.Tensor, implementation: str) -> bool:
    if implementation in ("torch", "nccl"):
        return False
    if not t.is_cuda:
        if implementation == "b200":
            raise ValueError("implementation='b200' needs CUDA tensors")
        return False
    return native.kernels_available()


def _cuda():
    from lyra_b200.ops import cuda_ops

    return cuda_ops


# --------------------------------------------------------------------------- ops
def rms_norm(x, scale, eps: float, implementation: str = "auto"):
    if use_kernels(x, implementation):
        return _cuda().rms_norm(x, scale, eps)
    return ref.rms_norm(x, scale, eps)


def linear(x, w, bias=None, implementation: str = "auto", *, residual=None, alpha: float = 1.0, out_dtype=None):
    """``alpha * (x @ w + bias) + residual`` with ``w`` stored ``[in, out]`` (fp32 master or bf16)."""
    if use_kernels(x, implementation):
        return _cuda().linear(x, w, bias, residual=residual, alpha=alpha, out_dtype=out_dtype)
    y = x @ w.to(x.dtype)
    if bias is not None:
        y = y + bias.to(y.dtype)
    if alpha != 1.0:
        y = y * alpha
    if residual is not None:
        y = residual + y
    return y.to(out_dtype) if out_dtype is not None else y


def linear_swiglu(x, w_up, bias, beta: float, limit: float, implementation: str = "auto"):
    """Dense up-projection fused with the clamped SwiGLU. ``w_up [C, 2, H]`` -> ``[..., H]``."""
    if use_kernels(x, implementation):
        return _cuda().linear_swiglu(x, w_up, bias, beta, limit)
    C, _, H = w_up.shape
    t = x @ w_up.reshape(C, 2 * H).to(x.dtype)
    if bias is not None:
        t = t + bias.reshape(2 * H).to(t.dtype)
    return ref.swiglu(t.reshape(*t.shape[:-1], 2, H), beta, limit).to(x.dtype)


def qk_norm_rope(q, k, qscale, kscale, cos, sin, eps: float, implementation: str = "auto"):
    """Optional per-head RMS norm of q and k, then rotary embedding; ``q,k [B, T, N, D]``."""
    if use_kernels(q, implementation):
        return _cuda().qk_norm_rope(q, k, qscale, kscale, cos, sin, eps)
    if qscale is not None:
        q = ref.rms_norm(q, qscale, eps)
        k = ref.rms_norm(k, kscale, eps)
    return ref.rotate(q, cos, sin), ref.rotate(k, cos, sin)


def attention(q, k, v, sinks, scale: float, window: int, q_start=0, implementation: str = "auto"):
    """Training / prefill attention, ``q [B, Nq, T, D]``, ``k, v [B, Nkv, S, D]`` -> ``[B, Nq, T, D]``."""
    if use_kernels(q, implementation):
        return _cuda().flash_attention(q, k, v, sinks, scale, window, q_start)
    return ref.attention(q, k, v, sinks, scale, window, q_start)[0]


def decode_attention(q, k_cache, v_cache, sinks, scale: float, window: int, pos, implementation: str = "auto", *, pos_dev=None):
    """Attention of ``T`` new query tokens (usually 1) starting at position ``pos`` over a KV cache
    (dense bf16 or fp8 ``QArray`` with one scale per (sequence, head, position))."""
    from lyra_b200.nn.quant import QArray, dequantize

    if use_kernels(q, implementation):
        return _cuda().decode_attention(q, k_cache, v_cache, sinks, scale, window, pos, pos_dev=pos_dev)
    if pos_dev is not None:
        pos = int(pos_dev.item())
    k = dequantize(k_cache, q.dtype) if isinstance(k_cache, QArray) else k_cache
    v = dequantize(v_cache, q.dtype) if isinstance(v_cache, QArray) else v_cache
    return ref.attention(q, k, v, sinks, scale, window, pos)[0]


def gate_xsa(t, h, w_gate, v, xsa_alpha, implementation: str = "auto"):
    """SDPA output gate ``t *= 2*sigmoid(h @ W_gate)`` (per token and query head, fp32 logits) followed by
    tanh-XSA ``t -= tanh(alpha_head) * (t . v_hat) * v_hat`` with ``v_hat`` the token's own unit value vector
    shared by the GQA group (lyra/model.py:343-360). ``t [B, Nq, T, D]``, ``h [B, T, C]``, ``v [B, Nkv, T, D]``."""
    if use_kernels(t, implementation):
        return _cuda().gate_xsa(t, h, w_gate, v, xsa_alpha)
    dtype = t.dtype
    if w_gate is not None:
        gate = 2.0 * torch.sigmoid(h.float() @ w_gate.float())  # [B, T, Nq]
        t = t * gate.transpose(1, 2)[..., None].to(dtype)
    if xsa_alpha is not None:
        B, Nq, T, D = t.shape
        Nkv = v.shape[1]
        rep = Nq // Nkv
        v32 = v.float()
        vn = (v32 * torch.rsqrt((v32 * v32).sum(-1, keepdim=True) + 1e-10)).to(dtype)
        t_g = t.reshape(B, Nkv, rep, T, D)
        vn_g = vn[:, :, None]
        coef = (t_g * vn_g).float().sum(-1, keepdim=True)
        alpha = torch.tanh(xsa_alpha.float()).reshape(1, Nkv, rep, 1, 1).to(dtype)
        t = (t_g - alpha * coef.to(dtype) * vn_g).reshape(B, Nq, T, D)
    return t


def linear_cross_entropy(x, w, y, vocab_size: int, reduction: str = "sum", implementation: str = "auto"):
    """Fused output head + cross entropy; never materialises ``[T, V]`` logits. Returns ``(loss, lse)``."""
    if use_kernels(x, implementation):
        return _cuda().linear_cross_entropy(x, w, y, vocab_size, reduction)
    return ref.linear_cross_entropy(x, w, y, vocab_size, reduction)


def embedding(emb, tokens, implementation: str = "auto", presorted: bool = True):
    """Row gather with a deterministic (sorted segment-sum, fp32) gradient (lyra/kernels/embs.py)."""
    if use_kernels(emb, implementation):
        return _cuda().embedding(emb, tokens)
    if presorted:
        return _EmbeddingRef.apply(emb, tokens)
    return emb[tokens]


class _EmbeddingRef(torch.autograd.Function):
    @staticmethod
    def forward(ctx, emb, tokens):
        ctx.save_for_backward(tokens)
        ctx.vocab = emb.shape[0]
        ctx.dtype = emb.dtype
        return emb[tokens]

    @staticmethod
    def backward(ctx, g):
        (tokens,) = ctx.saved_tensors
        return ref.embedding_grad(tokens, g, ctx.vocab).to(ctx.dtype), None


def moe_experts(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta: float, limit: float, implementation: str = "auto"):
    """Routed (+ shared) expert MLP on one rank: permute rows into expert order, grouped up-projection + SwiGLU,
    grouped down-projection, weighted top-k combine. ``xn [F, C]``, ``scores, indices [F, K]``,
    ``w_up [E, C, 2, H]``, ``w_down [E, H, C]`` -> ``[F, C]``."""
    if use_kernels(xn, implementation):
        return _cuda().moe_experts(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit)
    F_, K = indices.shape
    E, C, _, H = w_up.shape
    flat = indices.reshape(-1)
    order = torch.argsort(flat, stable=True)  # permute_map: sorted position -> assignment
    groups = torch.bincount(flat, minlength=E)
    t = xn[order // K]
    ub = up_bias.reshape(E, 2 * H) if up_bias is not None else None
    t = ref.grouped_gemm_autograd(t, w_up.reshape(E, C, 2 * H), groups, ub)
    t = ref.swiglu(t.reshape(-1, 2, H), beta, limit).to(xn.dtype)
    t = ref.grouped_gemm_autograd(t, w_down, groups, down_bias)
    unpermute = torch.empty_like(order)
    unpermute[order] = torch.arange(order.numel(), device=order.device)
    rows = t[unpermute].reshape(F_, K, C)
    return torch.einsum("fkc,fk->fc", rows.float(), scores.float()).to(xn.dtype)
