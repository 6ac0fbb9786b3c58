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
    if pos_dev is not None:
        raise ValueError("a device-resident position needs the single-token kernel (T == 1, head dim 64 or 128, bf16 or e4m3 cache)")
    k = dequantize(k_cache, BF16) if quant else k_cache
    v = dequantize(v_cache, BF16) if quant else v_cache
    S = min(k.shape[2], (int(pos) + T + 127) // 128 * 128)
    o, _ = attn_k.flash_fwd(q.to(BF16), k[:, :, :S], v[:, :, :S], sinks, scale, window, int(pos))
    return o


def _gemm_panel(n_cols: int) -> int:
    """Columns per CTA: 128 when it divides N, else 64 (measured on B200: 128 reads 4.4 TB/s, 64 and 192 about 4.0)."""
    import os

    forced = int(os.environ.get("LYRA_DECODE_PANEL", "0"))
    if forced in (64, 128, 192) and n_cols % forced == 0:
        return forced
    return 128 if n_cols % 128 == 0 else 64


def _gemm_splits(n_cols: int, panel: int, groups_with_rows: int, k_chunks: int) -> int:
    """K splits so that a layer with few column panels still spreads over the SMs (about two CTAs per SM)."""
    ctas = max(1, (n_cols // panel) * max(1, groups_with_rows))
    want = max(1, (2 * 148 + ctas - 1) // ctas)
    best = 1
    for s in range(1, k_chunks + 1):
        if k_chunks % s == 0 and s <= want:
            best = s
    return best


def decode_gemm(x: torch.Tensor, w, *, offsets: torch.Tensor | None = None, counts: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                swiglu: bool = False,
                swiglu_beta: float = 1.702, swiglu_limit: float = 7.0, active_groups: int | None = None,
                max_group_rows: int | None = None, residual: torch.Tensor | None = None, alpha: float = 1.0,
                typical_group_rows: int | None = None) -> torch.Tensor:
    """``x [R, K]`` (rows sorted by group) times ``w [G, K, N]`` (bf16 tensor, or QArray of e4m3 values with 2-D block
    scales) -> bf16 ``[R, N]`` (``[R, N/2]`` with SwiGLU). ``offsets [G+1]`` int32 row offsets on the device; ``None``
    means one group (a dense layer, ``w [K, N]`` or ``[1, K, N]``). ``counts [G]`` int32 gives the real rows per group when
    ``offsets`` describe a padded layout (the expert-parallel receive buffer); ``max_group_rows`` bounds the rows any group
    can hold (default: all ``R``), which sizes the launch. Rows per group beyond 64 cost another pass over that
    group's weights, so this is the path for a few rows per expert."""
    lib = native.kernels()
    quant = isinstance(w, QArray)
    wq = w.qval if quant else w
    if wq.ndim == 2:
        wq = wq.unsqueeze(0)
    G, K, N = wq.shape
    R = x.shape[0]
    assert x.shape[1] == K and x.dtype == BF16 and x.is_contiguous() and wq.is_contiguous()
    assert wq.dtype == (torch.float8_e4m3fn if quant else BF16), wq.dtype
    bk = bn = 0
    scale = None
    if quant:
        bk, bn = w.block[-2], w.block[-1]
        scale = w.scale.float().contiguous()
        if F8_TENSOR_CORES and f8_gemm_supported(K, N, bk, bn) and hasattr(lib, "lyra_decode_gemm_f8"):
            return _decode_gemm_f8(lib, x, wq, scale, bk, bn, offsets, counts, bias, swiglu, swiglu_beta, swiglu_limit, active_groups,
                                   max_group_rows, residual, alpha, typical_group_rows)
    panel = _gemm_panel(N)
    splits = _gemm_splits(N, panel, min(G, R) if active_groups is None else active_groups, K // 64)
    part = torch.empty(splits, R, N, dtype=torch.float32, device=x.device)
    out = torch.empty(R, N // 2 if swiglu else N, dtype=BF16, device=x.device)
    b = bias.detach().float().contiguous() if bias is not None else None
    if residual is not None:
        assert not swiglu and residual.dtype == BF16 and residual.shape == (R, N) and residual.is_contiguous()
    lib.lyra_decode_gemm.restype = c_int
    rc = lib.lyra_decode_gemm(ptr(x), ptr(wq), ptr(scale), c_int(int(quant)), c_int(bk), c_int(bn), ptr(offsets), ptr(counts), ptr(b), ptr(part), ptr(out),
                              c_int(R), c_int(K), c_int(N), c_int(G), c_int(splits), c_int(int(swiglu)), c_float(swiglu_beta),
                              c_float(swiglu_limit), c_int(panel), c_int(min(R, max_group_rows) if max_group_rows else R), ptr(residual), c_float(alpha), native.stream_ptr())
    native.check(rc, "lyra_decode_gemm")
    native.count_launch(2)
    return out




def f8_gemm_supported(K: int, N: int, bk: int, bn: int) -> bool:
    """Shapes the e4m3 x e4m3 tcgen05 kernel takes: K blocks of 32..., column blocks of 64 or multiples of 128."""
    return (bk >= 32 and bk % 32 == 0 and (128 % bk == 0 or bk % 128 == 0) and K % bk == 0 and (bn == 64 or bn % 128 == 0) and N % bn == 0
            and N % 16 == 0 and K % 16 == 0 and K // bk <= 64)


def _decode_gemm_f8(lib, x, wq, wscale, bk, bn, offsets, counts, bias, swiglu, swiglu_beta, swiglu_limit, active_groups, max_group_rows, residual, alpha,
                    typical_group_rows=None):
    """e4m3 weights x e4m3 activations on the tensor cores (``decode_gemm_f8_kernel``). The activations are quantised here with
    one scale per (row, K block of ``bk``), the (1 x scale_k) block of the reference's quantised grouped GEMM
    (lyra/kernels/gemm.py:1551-1556); the weights stream once, as stored."""
    from lyra_b200.nn.quant import quantize

    G, K, N = wq.shape
    R = x.shape[0]
    xq = quantize(x, torch.float8_e4m3fn, (1, bk))
    most = min(R, max_group_rows) if max_group_rows else R
    # token columns per tile: sized for the rows a group usually has, not for the worst case - a CTA takes a larger group in
    # several passes, and the narrow tiles read their accumulators back four at a time
    usual = min(most, typical_group_rows) if typical_group_rows else most
    ntok = 16 if usual <= 16 else 32 if usual <= 32 else 64
    groups = min(G, R) if active_groups is None else active_groups
    ctas = max(1, (N + 127) // 128 * max(1, groups))
    splits = 1
    for cand in range(1, K // 128 + 1):            # K splits for layers with few column panels (about two CTAs per SM)
        if K % (cand * 128) == 0 and (K // bk) % cand == 0 and cand * ctas <= 2 * 148:
            splits = cand
    part = torch.empty(splits, R, N, dtype=torch.float32, device=x.device)
    out = torch.empty(R, N // 2 if swiglu else N, dtype=BF16, device=x.device)
    b = bias.detach().float().contiguous() if bias is not None else None
    if residual is not None:
        assert not swiglu and residual.dtype == BF16 and residual.shape == (R, N) and residual.is_contiguous()
    lib.lyra_decode_gemm_f8.restype = c_int
    rc = lib.lyra_decode_gemm_f8(ptr(xq.qval), ptr(xq.scale), ptr(wq), ptr(wscale), c_int(bk), c_int(bn), ptr(offsets), ptr(counts), ptr(b), ptr(part),
                                 ptr(out), c_int(R), c_int(K), c_int(N), c_int(G), c_int(splits), c_int(int(swiglu)), c_float(swiglu_beta),
                                 c_float(swiglu_limit), c_int(ntok), c_int(most), ptr(residual), c_float(alpha), ptr(native.status_word()),
                                 native.stream_ptr())
    native.check(rc, "lyra_decode_gemm_f8")
    native.count_launch(2)
    return out


def decode_gemm_supported(K: int, N: int, w) -> bool:
    if K % 64 or N % 64:
        return False
    if isinstance(w, QArray):
        return (w.qval.dtype == torch.float8_e4m3fn and len(w.block) == 2 and w.block[0] % 64 == 0 and w.block[1] % 64 == 0
                and K % w.block[0] == 0 and N % w.block[1] == 0)
    return True


import os as _os

F8_TENSOR_CORES = _os.environ.get("LYRA_DECODE_F8_TC", "1") != "0"   # quantised weights: e4m3 x e4m3 tcgen05 kernel (0: dequantise in flight, mma.sync)
DECODE_GEMM_MAX_ROWS = int(_os.environ.get("LYRA_DECODE_GEMM_MAX_ROWS", "512"))   # assignments (tokens x experts per token); above this the 128-row-tile tcgen05 grouped GEMM takes over


def decode_moe(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit, plan=None):
    """Expert MLP for a handful of tokens (role of lyra/kernels/decode_gemm.py): rows sorted by expert without padding,
    two weight-streaming products (SwiGLU fused into the first one's finishing pass), weighted combine. ``plan``: the routing
    kernels' counts / offsets / expert-sorted order for exactly these ``indices`` (no shared experts appended), which replaces
    the sort-and-count glue below by one gather launch."""
    from lyra_b200.ops import cuda_ops
    from lyra_b200.ops import elementwise as ew
    from lyra_b200.ops import reference as ref

    F_, K = indices.shape
    C = xn.shape[1]
    E = (w_up.qval if isinstance(w_up, QArray) else w_up).shape[0]
    up_q, down_q = isinstance(w_up, QArray), isinstance(w_down, QArray)
    wu = w_up if up_q else cuda_ops.bf16_weight(w_up).view(E, C, -1)
    wd = w_down if down_q else cuda_ops.bf16_weight(w_down)
    N_up = (wu.qval if up_q else wu).shape[-1]
    H = N_up // 2
    # Measured on gpt-oss-20b shapes (batch 64, CUDA-graph replay): for bf16 experts the tcgen05 tile GEMM on 128-row padded
    # groups is faster than the small-M kernel (15.9 vs 17.0 ms per step), so bf16 experts take the tile path below;
    # quantised experts take the small-M kernel, which dequantises in flight. LYRA_DECODE_MOE_SMALL_M=1 forces it for bf16 too.
    force = _os.environ.get("LYRA_DECODE_MOE_SMALL_M", "0") == "1"
    small = F_ * K <= DECODE_GEMM_MAX_ROWS and (up_q or down_q or force)
    if small and decode_gemm_supported(C, N_up, wu) and decode_gemm_supported(H, C, wd):
        if plan is not None and plan.counts.numel() == E and plan.order.numel() == F_ * K and C % 8 == 0:
            from lyra_b200.ops import routing

            offsets = plan.starts
            x_sorted, dest = routing.gather_by_plan(xn.to(BF16).contiguous(), plan, K)
        else:
            flat = indices.reshape(-1)
            counts = ref.count_ids(flat, E)
            offsets = torch.zeros(E + 1, dtype=torch.int32, device=xn.device)
            offsets[1:] = torch.cumsum(counts, 0)
            order = torch.argsort(flat, stable=True)
            dest = torch.empty_like(order)
            dest[order] = torch.arange(order.numel(), device=order.device)
            x_sorted = xn.to(BF16)[order // K].contiguous()
        ub = cuda_ops.fp32_param(up_bias).reshape(E, N_up) if up_bias is not None else None
        db = cuda_ops.fp32_param(down_bias).reshape(E, C) if down_bias is not None else None
        usual = -(-2 * F_ * K // E)                            # twice the balanced rows per expert
        act = decode_gemm(x_sorted, wu, offsets=offsets, bias=ub, swiglu=True, swiglu_beta=beta, swiglu_limit=limit, active_groups=min(E, F_ * K),
                          typical_group_rows=usual)
        down = decode_gemm(act, wd, offsets=offsets, bias=db, active_groups=min(E, F_ * K), typical_group_rows=usual)
        return ew.combine_rows(down, dest, scores.float().contiguous(), F_, K)
    if up_q:
        w_up = dequantize(w_up, BF16).reshape(E, C, 2, -1)
    if down_q:
        w_down = dequantize(w_down, BF16)
    return cuda_ops.moe_experts(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit)
