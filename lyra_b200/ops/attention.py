"""Python face of the sm_100a attention kernels (``csrc/attn``). Tensors are token-major ``[B, T, N, D]``;
heads-first views (``x.transpose(1, 2)``) of such tensors are accepted without a copy."""

from __future__ import annotations

import torch

from lyra_b200.ops import native
from lyra_b200.ops.native import c_float, c_int, c_ll, ptr


def _btnd(x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """``x`` is heads-first ``[B, N, T, D]`` (any strides with unit inner stride). Returns (tensor, (sb, st, sn))."""
    if x.stride(-1) != 1 or x.data_ptr() % 16 or any(s % 8 for s in x.stride()[:-1]):
        x = x.transpose(1, 2).contiguous().transpose(1, 2)
    return x, (x.stride(0), x.stride(2), x.stride(1))


def flash_fwd(q, k, v, sinks, scale: float, window: int, q_start: int = 0):
    """``q [B, Nq, T, D]``, ``k, v [B, Nkv, S, D]`` bf16 -> ``(out [B, Nq, T, D] (token-major storage), lse [B, Nq, T] fp32)``."""
    B, Nq, T, D = q.shape
    Nkv, S = k.shape[1], k.shape[2]
    q, qs = _btnd(q)
    k, ks = _btnd(k)
    v, vs = _btnd(v)
    out = torch.empty(B, T, Nq, D, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, Nq, T, dtype=torch.float32, device=q.device)
    fn = native.kernels().lyra_flash_fwd
    fn.restype = c_int
    rc = fn(ptr(q), c_ll(qs[0]), c_ll(qs[1]), c_ll(qs[2]), ptr(k), c_ll(ks[0]), c_ll(ks[1]), c_ll(ks[2]),
            ptr(v), c_ll(vs[0]), c_ll(vs[1]), c_ll(vs[2]), ptr(sinks.float().contiguous()), ptr(out), ptr(lse),
            c_int(B), c_int(T), c_int(S), c_int(Nq), c_int(Nkv), c_int(D), c_float(scale), c_int(window), c_int(int(q_start)),
            ptr(native.status_word()), native.stream_ptr())
    native.check(rc, "lyra_flash_fwd")
    native.count_launch()
    return out.transpose(1, 2), lse


def _strides3(x: torch.Tensor):
    import ctypes

    return (ctypes.c_longlong * 3)(x.stride(0), x.stride(2), x.stride(1))


def flash_bwd(q, k, v, out, d_out, lse, sinks, scale: float, window: int, q_start: int = 0):
    """Gradients of :func:`flash_fwd`. All tensors heads-first views; ``out`` must be the forward's output.
    Returns ``(dq, dk, dv, dsinks)`` (heads-first views of token-major storage, dsinks fp32 ``[Nq]``)."""
    B, Nq, T, D = q.shape
    Nkv, S = k.shape[1], k.shape[2]
    q, _ = _btnd(q)
    k, _ = _btnd(k)
    v, _ = _btnd(v)
    d_out, _ = _btnd(d_out)
    out_t = out.transpose(1, 2)
    if not out_t.is_contiguous():
        out_t = out_t.contiguous()
    dq = torch.empty(B, T, Nq, D, dtype=torch.bfloat16, device=q.device)
    dk = torch.empty(B, S, Nkv, D, dtype=torch.bfloat16, device=q.device)
    dv = torch.empty(B, S, Nkv, D, dtype=torch.bfloat16, device=q.device)
    delta = torch.empty(B, Nq, T, dtype=torch.float32, device=q.device)
    fn = native.kernels().lyra_flash_bwd
    fn.restype = c_int
    rc = fn(ptr(q), _strides3(q), ptr(k), _strides3(k), ptr(v), _strides3(v), ptr(out_t), ptr(d_out), _strides3(d_out),
            ptr(lse), ptr(delta), ptr(dq), ptr(dk), ptr(dv),
            c_int(B), c_int(T), c_int(S), c_int(Nq), c_int(Nkv), c_int(D), c_float(scale), c_int(window), c_int(int(q_start)),
            ptr(native.status_word()), native.stream_ptr())
    native.check(rc, "lyra_flash_bwd")
    native.count_launch(3)
    # dsink_h = -sum_{b,t} exp(sink_h - lse) * delta  (lyra/kernels/flash_attention.py:653-659)
    dsinks = -(torch.exp(sinks.float()[None, :, None] - lse) * delta).sum(dim=(0, 2))
    return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2), dsinks


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sinks, scale, window, q_start):
        out, lse = flash_fwd(q, k, v, sinks, scale, window, q_start)
        ctx.save_for_backward(q, k, v, out, lse, sinks)
        ctx.args = (scale, window, q_start)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse, sinks = ctx.saved_tensors
        scale, window, q_start = ctx.args
        dq, dk, dv, dsinks = flash_bwd(q, k, v, out, d_out, lse, sinks, scale, window, q_start)
        return dq, dk, dv, dsinks.to(sinks.dtype), None, None, None


def flash_attention(q, k, v, sinks, scale: float, window: int, q_start: int = 0):
    return FlashAttention.apply(q, k, v, sinks, scale, window, q_start)
