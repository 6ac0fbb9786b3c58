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


def decode_splits(batch: int, n_kv: int, n_keys: int) -> int:
    """Key splits so that the grid covers the 148 SMs about twice, with at least 128 keys per split."""
    return max(1, min((n_keys + 127) // 128, (2 * 148 + batch * n_kv - 1) // (batch * n_kv)))


_scratch: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _split_scratch(device, B: int, Nq: int, splits: int, D: int):
    key = (device, B, Nq, splits, D)
    if key not in _scratch:
        _scratch[key] = (torch.empty(B, Nq, splits, D, dtype=torch.float32, device=device),
                         torch.empty(B, Nq, splits, 2, dtype=torch.float32, device=device))
    return _scratch[key]


def decode_attention(q, k_cache, v_cache, sinks, scale: float, window: int, pos, *, pos_dev: torch.Tensor | None = None,
                     out: torch.Tensor | None = None):
    """``q [B, Nq, T, D]`` (T new tokens starting at ``pos``), caches ``[B, Nkv, S, D]``; keys ``<= pos + t`` are visible.

    With ``pos_dev`` (int32 device scalar) the single-token kernel reads the position on the device, so that a recorded
    sequence of launches can be replayed for later positions; ``pos`` then only bounds the number of key splits."""
    B, Nq, T, D = q.shape
    lib = native.kernels()
    quant = isinstance(k_cache, QArray)
    kq = k_cache.qval if quant else k_cache
    Nkv, S = kq.shape[1], kq.shape[2]
    fast = (T == 1 and hasattr(lib, "lyra_decode_attention") and D in (64, 128) and kq.is_contiguous() and Nq % Nkv == 0 and Nq // Nkv <= 16
            and kq.dtype in (BF16, torch.float8_e4m3fn))
    if fast:
        vq = v_cache.qval if quant else v_cache
        assert vq.is_contiguous() and vq.dtype == kq.dtype
        if out is None:
            out = torch.empty(B, Nq, 1, D, dtype=BF16, device=q.device)
        qc = q.to(BF16).contiguous()
        ks = k_cache.scale.float().contiguous() if quant else None
        vs = v_cache.scale.float().contiguous() if quant else None
        n_keys = S if pos_dev is not None else (min(int(pos) + 1, window) if window else int(pos) + 1)
        if pos_dev is not None and window:
            n_keys = min(S, window)
        splits = decode_splits(B, Nkv, n_keys)
        part_o, part_ml = _split_scratch(q.device, B, Nq, splits, D) if splits > 1 else (None, None)
        sk = sinks.float().contiguous() if sinks is not None else None
        lib.lyra_decode_attention.restype = c_int
        rc = lib.lyra_decode_attention(ptr(qc), ptr(kq), ptr(vq), ptr(ks), ptr(vs), c_int(int(quant)), ptr(sk), ptr(out), ptr(part_o), ptr(part_ml),
                                       c_int(splits), ptr(pos_dev), c_int(B), c_int(Nq), c_int(Nkv), c_int(S), c_int(D), c_float(scale),
                                       c_int(int(window)), c_int(int(pos)), native.stream_ptr())
        native.check(rc, "lyra_decode_attention")
        native.count_launch(2 if splits > 1 else 1)
        return out
    k = dequantize(k_cache, BF16) if quant else k_cache
    v = dequantize(v_cache, BF16) if quant else v_cache
    S = min(k.shape[2], (int(pos) + T + 127) // 128 * 128)
    o, _ = attn_k.flash_fwd(q.to(BF16), k[:, :, :S], v[:, :, :S], sinks, scale, window, int(pos))
    return o


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
