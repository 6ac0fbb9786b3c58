"""Decode-mode ops: attention of a few new query tokens over the KV cache and the small-M expert MLP
(roles of lyra/kernels/decode_attention.py and decode_gemm.py).

``decode_attention`` runs the split-KV single-query kernel (``csrc/attn/decode_attn.cu``) when it is built and the
query has one token; otherwise the tcgen05 prefill kernel with ``q_start = pos`` on the (dequantised) cache.
fp8 caches carry one fp32 scale per (sequence, kv head, position) and are dequantised inside the decode kernel."""

from __future__ import annotations

import torch

from lyra_b200.nn.quant import QArray, dequantize
from lyra_b200.ops import attention as attn_k
from lyra_b200.ops import native
from lyra_b200.ops.native import c_float, c_int, c_ll, ptr

BF16 = torch.bfloat16


def decode_attention(q, k_cache, v_cache, sinks, scale: float, window: int, pos: int):
    """``q [B, Nq, T, D]`` (T new tokens starting at ``pos``), caches ``[B, Nkv, S, D]``; keys ``<= pos + t`` are visible."""
    B, Nq, T, D = q.shape
    lib = native.kernels()
    quant = isinstance(k_cache, QArray)
    kq = k_cache.qval if quant else k_cache
    if T == 1 and hasattr(lib, "lyra_decode_attention") and D in (64, 128) and kq.is_contiguous():
        Nkv, S = kq.shape[1], kq.shape[2]
        out = torch.empty(B, Nq, 1, D, dtype=BF16, device=q.device)
        qc = q.to(BF16).contiguous()
        vq = v_cache.qval if quant else v_cache
        ks = k_cache.scale.contiguous() if quant else None
        vs = v_cache.scale.contiguous() if quant else None
        lib.lyra_decode_attention.restype = c_int
        rc = lib.lyra_decode_attention(ptr(qc), ptr(kq), ptr(vq), ptr(ks), ptr(vs), c_int(int(quant)), ptr(sinks.float().contiguous()), ptr(out),
                                       c_int(B), c_int(Nq), c_int(Nkv), c_int(S), c_int(D), c_float(scale), c_int(window), c_int(int(pos)),
                                       native.stream_ptr())
        native.check(rc, "lyra_decode_attention")
        native.count_launch()
        return out
    k = dequantize(k_cache, BF16) if quant else k_cache
    v = dequantize(v_cache, BF16) if quant else v_cache
    S = min(k.shape[2], (int(pos) + T + 127) // 128 * 128)
    out, _ = attn_k.flash_fwd(q.to(BF16), k[:, :, :S], v[:, :, :S], sinks, scale, window, int(pos))
    return out


def decode_moe(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit):
    """Expert MLP for a handful of tokens: weight-streaming small-M kernel when built, else the grouped-GEMM path."""
    from lyra_b200.ops import cuda_ops

    if isinstance(w_up, QArray) or isinstance(w_down, QArray):
        C = xn.shape[1]
        if isinstance(w_up, QArray):
            w_up = dequantize(w_up, BF16).reshape(w_up.shape[0], C, 2, -1)
        if isinstance(w_down, QArray):
            w_down = dequantize(w_down, BF16)
    return cuda_ops.moe_experts(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit)
