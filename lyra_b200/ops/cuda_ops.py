"""Autograd wrappers that route the model's ops to the sm_100a kernels.

Every function here assumes CUDA tensors and a built kernel library; ``lyra_b200.ops.api`` decides when to
call them. Saved-for-backward state is kept minimal: pre-activations of SwiGLU MLPs are recomputed in the
backward pass (the reference rematerialises the whole MLP block, lyra/model.py:648-660), attention saves
only its output and log-sum-exp, the output head never stores logits.

Weight gradients are accumulated in place into ``param.grad`` by the GEMM epilogue (``C = A^T B + C``), so
gradient accumulation over microbatches costs no extra pass over the gradient buffers.
"""

from __future__ import annotations

import math
import weakref

import torch

from lyra_b200.ops import attention as attn_k
from lyra_b200.ops import elementwise as ew
from lyra_b200.ops import gemm as G
from lyra_b200.ops import native
from lyra_b200.ops import reference as ref
from lyra_b200.ops.native import c_float, c_int, c_ll, ptr

BF16 = torch.bfloat16

# --------------------------------------------------------------------------- bf16 shadows of fp32 masters
_SHADOW: dict[int, tuple[int, torch.Tensor, weakref.ref]] = {}
KEEP_SHADOWS = True  # False: cast at every use instead (for models whose bf16 copy does not fit beside the optimizer state)
GRAD_DTYPE = torch.float32
SAVE_PREACT = True   # keep SwiGLU pre-activations for backward; False recomputes them (one more up-projection GEMM, less memory)


def set_memory_mode(keep_shadows: bool, grad_dtype: torch.dtype = torch.float32, save_preact: bool | None = None) -> None:
    global KEEP_SHADOWS, GRAD_DTYPE, SAVE_PREACT
    KEEP_SHADOWS, GRAD_DTYPE = keep_shadows, grad_dtype
    SAVE_PREACT = keep_shadows if save_preact is None else save_preact
    if not keep_shadows:
        _SHADOW.clear()


def bf16_weight(w: torch.Tensor) -> torch.Tensor:
    """bf16 compute copy of a master weight. Cached per parameter and refreshed when the master changed."""
    if w.dtype == BF16:
        return w
    if not KEEP_SHADOWS:
        return w.detach().to(BF16)
    key = id(w)
    hit = _SHADOW.get(key)
    if hit is not None and hit[2]() is not w:      # the id was recycled by a different tensor
        hit = None
    if hit is not None and hit[0] == w._version:
        return hit[1]
    if hit is not None:
        hit[1].copy_(w.detach())
        shadow = hit[1]
    else:
        shadow = w.detach().to(BF16)
        if len(_SHADOW) > 4096:
            for k in [k for k, v in _SHADOW.items() if v[2]() is None]:
                del _SHADOW[k]
    _SHADOW[key] = (w._version, shadow, weakref.ref(w))
    return shadow


def shadow_of(w: torch.Tensor) -> torch.Tensor | None:
    hit = _SHADOW.get(id(w))
    return hit[1] if hit is not None and hit[2]() is w else None


_WEIGHTS_EPOCH = 0


def weights_changed() -> None:
    """Tells the derived-weight caches below (fused projections, fp32 copies) that parameters were rewritten behind PyTorch's
    version counters: the optimizer kernels update masters and bf16 copies through raw pointers."""
    global _WEIGHTS_EPOCH
    _WEIGHTS_EPOCH += 1


def invalidate_shadows() -> None:
    """Marks every cached bf16 copy stale (call after the masters changed through an alias, e.g. the optimizer)."""
    weights_changed()
    for key, (_, shadow, ref) in list(_SHADOW.items()):
        _SHADOW[key] = (-1, shadow, ref)


_F32: dict[int, tuple] = {}


def fp32_param(p: torch.Tensor | None) -> torch.Tensor | None:
    """fp32 copy of a parameter that is stored in another dtype (biases and the router of a bf16 checkpoint), cached per parameter
    object until it changes: an inference step otherwise converts the same few tensors again in every layer call. Parameters that
    take part in a gradient computation are converted in the graph as before."""
    if p is None or p.dtype == torch.float32:
        return p
    if torch.is_grad_enabled() and p.requires_grad:
        return p.float()
    hit = _F32.get(id(p))
    if hit is not None and hit[2]() is p and hit[0] == (p._version, _WEIGHTS_EPOCH):
        return hit[1]
    copy = p.detach().float()
    if len(_F32) > 4096:
        for k in [k for k, v in _F32.items() if v[2]() is None]:
            del _F32[k]
    _F32[id(p)] = ((p._version, _WEIGHTS_EPOCH), copy, weakref.ref(p))
    return copy


_FUSED: dict[tuple, tuple] = {}


def pull_pending(*ws) -> bool:
    """True when the sharding runtime still has to pull one of these weights from its owner (the pull rides inside the first
    forward GEMM that is given the weight itself; a derived copy made before that would hold last step's values)."""
    return AG_HOOK is not None and any(w is not None and AG_HOOK(w) is not None for w in ws)


def fused_columns(ws, biases):
    """``[C, sum N_i]`` bf16 concatenation of the weights ``ws`` (and the fp32 concatenation of their biases, or None), cached
    until one of them changes: a decode step multiplies the same few rows with q, k and v, and one product of the fused
    matrix is two launches instead of six. Inference only (the copies do not follow the masters' gradients)."""
    key = tuple(id(w) for w in ws)
    versions = tuple(w._version for w in ws) + tuple(-1 if b is None else b._version for b in biases) + (_WEIGHTS_EPOCH,)
    hit = _FUSED.get(key)
    if hit is not None and hit[0] == versions and all(r() is w for r, w in zip(hit[3], ws)):
        return hit[1], hit[2]
    fused = torch.cat([bf16_weight(w).reshape(w.shape[0], -1) for w in ws], dim=1).contiguous()
    fb = None
    if any(b is not None for b in biases):
        fb = torch.cat([(b.detach().float().reshape(-1) if b is not None else torch.zeros(w.shape[1], device=w.device)) for w, b in zip(ws, biases)])
    if len(_FUSED) > 1024:
        for k in [k for k, v in _FUSED.items() if any(r() is None for r in v[3])]:
            del _FUSED[k]
    _FUSED[key] = (versions, fused, fb, tuple(weakref.ref(w) for w in ws))
    return fused, fb


AG_HOOK = None  # set by the sharding runtime: callable(weight) -> pending fused all-gather description or None


def _forward_gemm(x2: torch.Tensor, w: torch.Tensor, wb2d: torch.Tensor, **kw) -> torch.Tensor:
    """``x2 @ wb2d`` for a forward pass. If ``w`` is a sharded weight whose rows still sit on its owner, the pull over
    NVLink is fused into this GEMM (``gemm_allgather``) and the local copy is complete afterwards."""
    info = AG_HOOK(w) if AG_HOOK is not None else None
    if info is None:
        return G.gemm(x2, wb2d, b_mn=True, **kw)
    y = G.gemm_allgather(x2, wb2d, info["src"], info["my_rank"], wb2d.shape[0], info["flags"], info["epoch"], **kw)
    info["done"]()
    return y


def _accumulate_wgrad(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0) -> None:
    """``w.grad += alpha * a^T @ b`` with ``a [M, K_in]``, ``b [M, N_out]`` (both MN-major operands), in the GEMM epilogue."""
    shape2d = (a.shape[1], b.shape[1])
    if w.grad is None:
        w.grad = torch.empty(w.shape, dtype=GRAD_DTYPE, device=w.device)
        G.gemm(a, b, a_mn=True, b_mn=True, out=w.grad.view(shape2d), alpha=alpha)
    else:
        g = w.grad.view(shape2d)
        G.gemm(a, b, a_mn=True, b_mn=True, out=g, alpha=alpha, beta=1.0, c_in=g)


def _add_grad(p: torch.Tensor | None, g: torch.Tensor) -> None:
    if p is None:
        return
    if p.grad is None:
        p.grad = g.to(p.dtype if p.dtype == torch.float32 else torch.float32).reshape(p.shape).clone()
    else:
        p.grad += g.reshape(p.shape).to(p.grad.dtype)


# --------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual, alpha):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != BF16:
            x2 = x2.to(BF16)
        wb = bf16_weight(w)
        res2 = residual.reshape(-1, w.shape[1]) if residual is not None else None
        b = None
        if bias is not None:
            b = bias.detach().float().reshape(-1)
            if alpha != 1.0:
                b = b * alpha
        y = _forward_gemm(x2.contiguous(), w, wb, alpha=alpha, beta=1.0 if res2 is not None else 0.0,
                          c_in=res2.contiguous() if res2 is not None else None, bias=b)
        ctx.save_for_backward(x2, w)
        ctx.alpha, ctx.has_res, ctx.bias = alpha, residual is not None, bias
        ctx.lead = lead
        return y.reshape(*lead, w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        wb = bf16_weight(w)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm(dy2, wb, alpha=ctx.alpha).reshape(*ctx.lead, w.shape[0])
        if w.requires_grad:
            _accumulate_wgrad(w, x2, dy2, ctx.alpha)
        if ctx.bias is not None and ctx.bias.requires_grad:
            _add_grad(ctx.bias, dy2.float().sum(0) * ctx.alpha)
        return dx, None, None, (dy if ctx.has_res else None), None


SMALL_M_ROWS = 64   # at most this many rows (and no autograd): the weight-streaming small-M kernel, all SMs busy via K splits


def linear(x, w, bias=None, *, residual=None, alpha: float = 1.0, out_dtype=None):
    N = w.shape[1]
    rows = x.numel() // x.shape[-1]
    if (rows <= SMALL_M_ROWS and N % 64 == 0 and w.shape[0] % 64 == 0 and w.ndim == 2
            and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or (residual is not None and residual.requires_grad)))
            and (AG_HOOK is None or AG_HOOK(w) is None)):
        from lyra_b200.ops import decode as dec

        x2 = x.reshape(rows, x.shape[-1]).to(BF16).contiguous()
        res2 = residual.reshape(rows, N).to(BF16).contiguous() if residual is not None else None
        y = dec.decode_gemm(x2, bf16_weight(w), bias=fp32_param(bias).reshape(1, N) if bias is not None else None, residual=res2,
                            alpha=alpha).reshape(*x.shape[:-1], N)
    elif N % 8 or w.shape[0] % 8:
        y = ref_linear(x, w, bias, residual, alpha)
    else:
        y = _Linear.apply(x, w, bias, residual, alpha)
    return y.to(out_dtype) if out_dtype is not None else y


def ref_linear(x, w, bias, residual, alpha):
    y = x @ w.to(x.dtype)
    if bias is not None:
        y = y + bias.to(y.dtype)
    if alpha != 1.0:
        y = y * alpha
    return y if residual is None else residual + y


# --------------------------------------------------------------------------- dense up-projection + SwiGLU
class _LinearSwiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_up, bias, beta, limit):
        C, _, H = w_up.shape
        lead = x.shape[:-1]
        x2 = x.reshape(-1, C).contiguous()
        wb = bf16_weight(w_up).view(C, 2 * H)
        b = bias.detach().float().reshape(2 * H) if bias is not None else None
        if SAVE_PREACT and x.requires_grad:
            pre = _forward_gemm(x2, w_up, wb, bias=b)
            y = ew.swiglu_fwd(pre, beta, limit)
            ctx.save_for_backward(x2, w_up, pre)
        else:
            if AG_HOOK is not None and AG_HOOK(w_up) is not None:   # land the weight first; the SwiGLU-epilogue GEMM has no fused pull
                _forward_gemm(x2[:128], w_up, wb)
            y = G.gemm_swiglu(x2, wb, bias=b, swiglu_beta=beta, swiglu_limit=limit)
            ctx.save_for_backward(x2, w_up)
        ctx.bias, ctx.beta, ctx.limit, ctx.lead = bias, beta, limit, lead
        return y.reshape(*lead, H)

    @staticmethod
    def backward(ctx, dy):
        x2, w_up, *saved = ctx.saved_tensors
        C, _, H = w_up.shape
        wb = bf16_weight(w_up).view(C, 2 * H)
        b = ctx.bias.detach().float().reshape(2 * H) if ctx.bias is not None else None
        pre = saved[0] if saved else G.gemm(x2, wb, b_mn=True, bias=b)   # kept, or recomputed [M, 2H]
        dpre = ew.swiglu_bwd(pre, dy.reshape(-1, H).contiguous(), ctx.beta, ctx.limit)
        del pre
        dx = G.gemm(dpre, wb).reshape(*ctx.lead, C) if ctx.needs_input_grad[0] else None
        if w_up.requires_grad:
            _accumulate_wgrad(w_up, x2, dpre)
        if ctx.bias is not None and ctx.bias.requires_grad:
            _add_grad(ctx.bias, dpre.float().sum(0))
        return dx, None, None, None, None


def linear_swiglu(x, w_up, bias, beta, limit):
    C, _, H = w_up.shape
    if H % 8 or C % 8:
        # widths the tile kernels do not take (TMA rows must be multiples of 16 bytes), e.g. 1080 / 2 hidden units per rank under
        # tensor parallelism: the PyTorch statement of the same op, differentiable
        pre = x @ w_up.reshape(C, 2 * H).to(x.dtype)
        if bias is not None:
            pre = pre + bias.reshape(2 * H).to(pre.dtype)
        return ref.swiglu(pre.float().reshape(*pre.shape[:-1], 2, H), beta, limit).to(x.dtype)
    return _LinearSwiglu.apply(x, w_up, bias, beta, limit)


# --------------------------------------------------------------------------- norms / rope / gate (fused elementwise kernels)
def rms_norm(x, scale, eps):
    return ew.RMSNorm.apply(x, scale, eps)


def qk_norm_rope(q, k, qscale, kscale, cos, sin, eps):
    return ew.qk_norm_rope(q, k, qscale, kscale, cos, sin, eps)


def gate_xsa(t, h, w_gate, v, xsa_alpha):
    return ew.gate_xsa(t, h, w_gate, v, xsa_alpha)


def embedding(emb, tokens):
    return ew.Embedding.apply(emb, tokens)


# --------------------------------------------------------------------------- attention
def flash_attention(q, k, v, sinks, scale, window, q_start):
    if q.dtype != BF16:
        q, k, v = q.to(BF16), k.to(BF16), v.to(BF16)
    return attn_k.flash_attention(q, k, v, sinks, scale, window, int(q_start))


def decode_attention(q, k_cache, v_cache, sinks, scale, window, pos, pos_dev=None):
    from lyra_b200.ops import decode as dec

    return dec.decode_attention(q, k_cache, v_cache, sinks, scale, window, int(pos), pos_dev=pos_dev)


def decode_moe(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit, plan=None):
    from lyra_b200.ops import decode as dec

    return dec.decode_moe(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit, plan)


# --------------------------------------------------------------------------- fused linear cross-entropy
_CE_CHUNK = 8192  # rows of dZ materialised at a time (bf16 [chunk, vocab] = 3.3 GB at the full vocabulary)


def _ce_forward(x2, wb, y32, vocab):
    M, K = x2.shape
    lib = native.kernels()
    n_tiles = (vocab + 255) // 256
    part_m = torch.empty(n_tiles, M, dtype=torch.float32, device=x2.device)
    part_l = torch.empty_like(part_m)
    tgt = torch.zeros(M, dtype=torch.float32, device=x2.device)
    lib.lyra_ce_gemm.restype = c_int
    rc = lib.lyra_ce_gemm(ptr(x2), c_ll(x2.stride(0)), ptr(wb), c_ll(wb.stride(0)), ptr(y32), c_int(M), c_int(vocab), c_int(K), c_int(0),
                          ptr(part_m), ptr(part_l), ptr(tgt), ptr(None), ptr(None), ptr(None), c_ll(0),
                          ptr(native.status_word()), native.stream_ptr())
    native.check(rc, "lyra_ce_gemm fwd")
    lse = torch.empty(M, dtype=torch.float32, device=x2.device)
    row_loss = torch.empty_like(lse)
    lib.lyra_ce_merge.restype = c_int
    native.check(lib.lyra_ce_merge(ptr(part_m), ptr(part_l), ptr(tgt), ptr(lse), ptr(row_loss), c_int(M), c_int(n_tiles),
                                   native.stream_ptr()), "lyra_ce_merge")
    native.count_launch(2)
    return lse, row_loss


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, y, vocab, reduction):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y32 = y.reshape(-1).to(torch.int32).contiguous()
        wb = bf16_weight(w)
        lse, row_loss = _ce_forward(x2, wb, y32, vocab)
        loss = row_loss.sum()
        if reduction == "mean":
            loss = loss / x2.shape[0]
        ctx.save_for_backward(x2, w, y32, lse)
        ctx.vocab, ctx.reduction = vocab, reduction
        ctx.mark_non_differentiable(lse)
        return loss, lse

    @staticmethod
    def backward(ctx, dloss, _dlse):
        x2, w, y32, lse = ctx.saved_tensors
        vocab = ctx.vocab
        M, K = x2.shape
        wb = bf16_weight(w)
        g = dloss.detach().float().reshape(1)
        if ctx.reduction == "mean":
            g = g / M
        g = g.contiguous()
        lib = native.kernels()
        lib.lyra_ce_gemm.restype = c_int
        dx = torch.empty(M, K, dtype=BF16, device=x2.device) if ctx.needs_input_grad[0] else None
        chunk = min(_CE_CHUNK, M)
        dz = torch.empty(chunk, vocab, dtype=BF16, device=x2.device)
        if w.requires_grad and w.grad is None:
            w.grad = torch.zeros(w.shape, dtype=GRAD_DTYPE, device=w.device)
        for s in range(0, M, chunk):
            n = min(chunk, M - s)
            xs, dzs = x2[s:s + n], dz[:n]
            rc = lib.lyra_ce_gemm(ptr(xs), c_ll(xs.stride(0)), ptr(wb), c_ll(wb.stride(0)), ptr(y32[s:s + n]), c_int(n), c_int(vocab),
                                  c_int(K), c_int(1), ptr(None), ptr(None), ptr(None), ptr(lse[s:s + n]), ptr(g), ptr(dzs),
                                  c_ll(dzs.stride(0)), ptr(native.status_word()), native.stream_ptr())
            native.check(rc, "lyra_ce_gemm dz")
            native.count_launch()
            if dx is not None:  # dX = dZ @ W[:vocab]   (A = dZ K-major over the vocabulary, B = W MN-major)
                G.gemm(dzs, wb[:vocab], b_mn=True, out=dx[s:s + n])
            if w.requires_grad:  # dW[:vocab] += dZ^T @ X
                gw = w.grad[:vocab]
                G.gemm(dzs, xs, a_mn=True, b_mn=True, out=gw, beta=1.0, c_in=gw)
        return dx, None, None, None, None


def linear_cross_entropy(x, w, y, vocab_size, reduction="sum"):
    """``w`` is ``[padded vocabulary, C]`` (row v = output embedding of token v); only the first ``vocab_size`` rows are read."""
    shape = x.shape
    if w.ndim != 2 or w.shape[1] != shape[-1] or w.shape[0] < vocab_size:
        raise ValueError(f"linear_cross_entropy: weight {tuple(w.shape)} does not match x {tuple(shape)} / vocab {vocab_size}")
    loss, lse = _LinearCE.apply(x.reshape(-1, shape[-1]), w, y, vocab_size, reduction)
    return loss, lse


# --------------------------------------------------------------------------- single-rank MoE experts
def moe_routing_layout(indices: torch.Tensor, n_experts: int):
    """Expert-sorted padded layout for ``indices [F, K]``: every expert's rows start at a multiple of 128.

    Returns ``(dest [F*K] int64 row of each assignment, tile_group [R/128] int32, offsets [E+1] int32 padded, R)``.
    ``R`` is a static upper bound so no host synchronisation is needed: ``F*K`` rounded up plus one tile per expert."""
    F_, K = indices.shape
    flat = indices.reshape(-1)
    R = ((F_ * K + 127) // 128 + n_experts) * 128
    counts = ref.count_ids(flat, n_experts)
    padded = (counts + 127) // 128 * 128
    offsets = torch.zeros(n_experts + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = torch.cumsum(padded, 0)
    order = torch.argsort(flat, stable=True)
    starts = torch.cumsum(counts, 0) - counts
    rank_in_group = torch.arange(flat.numel(), device=flat.device) - starts[flat[order]]
    dest = torch.empty_like(order)
    dest[order] = offsets[flat[order]] + rank_in_group
    tile_start = torch.arange(R // 128, device=flat.device) * 128
    tile_group = torch.searchsorted(offsets[1:], tile_start, right=True)
    tile_group = torch.where(tile_start < offsets[-1], tile_group, torch.full_like(tile_group, -1)).to(torch.int32)
    return dest, tile_group, offsets.to(torch.int32), R


class _MoEExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit):
        F_, K = indices.shape
        E, C, _, H = w_up.shape
        dest, tile_group, offsets, R = moe_routing_layout(indices, E)
        x_perm = ew.scatter_rows(xn, dest, K, R)                                   # [R, C], pad rows zero
        wu = bf16_weight(w_up).view(E, C, 2 * H)
        wd = bf16_weight(w_down)
        ub = up_bias.detach().float().reshape(E, 2 * H) if up_bias is not None else None
        db = down_bias.detach().float().reshape(E, C) if down_bias is not None else None
        pre = None
        if SAVE_PREACT and (xn.requires_grad or w_up.requires_grad):
            # memory to spare: keep the pre-activations (and the permuted rows) so that backward skips the up-projection recompute
            pre = G.grouped_gemm(x_perm, wu, tile_group, bias=ub, out=torch.zeros(R, 2 * H, dtype=BF16, device=xn.device))
            act = ew.swiglu_fwd(pre, beta, limit)
        else:
            act = G.grouped_gemm(x_perm, wu, tile_group, bias=ub, swiglu=True, swiglu_beta=beta, swiglu_limit=limit,
                                 out=torch.zeros(R, H, dtype=BF16, device=xn.device))
        down = G.grouped_gemm(act, wd, tile_group, bias=db, out=torch.zeros(R, C, dtype=BF16, device=xn.device))
        out = ew.combine_rows(down, dest, scores, F_, K)
        ctx.save_for_backward(xn, scores, dest, tile_group, offsets, w_up, w_down, down)
        ctx.cfg = (beta, limit, R, up_bias, down_bias)
        ctx.kept = (x_perm, pre) if pre is not None else None
        return out

    @staticmethod
    def backward(ctx, dout):
        xn, scores, dest, tile_group, offsets, w_up, w_down, down = ctx.saved_tensors
        beta, limit, R, up_bias, down_bias = ctx.cfg
        F_, K = scores.shape
        E, C, _, H = w_up.shape
        dout = dout.contiguous()
        wu = bf16_weight(w_up).view(E, C, 2 * H)
        wd = bf16_weight(w_down)
        ub = up_bias.detach().float().reshape(E, 2 * H) if up_bias is not None else None
        # d(down rows) = score * dout[token]; dscore = <down row, dout[token]>
        d_down, dscores = ew.combine_rows_bwd(down, dout, dest, scores, R)
        del down
        if ctx.kept is not None:
            x_perm, pre = ctx.kept
            ctx.kept = None
        else:
            x_perm = ew.scatter_rows(xn, dest, K, R)
            pre = G.grouped_gemm(x_perm, wu, tile_group, bias=ub, out=torch.zeros(R, 2 * H, dtype=BF16, device=xn.device))
        act = ew.swiglu_fwd(pre, beta, limit)
        if w_down.requires_grad:
            if w_down.grad is None:
                w_down.grad = G.grouped_wgrad(act, d_down, offsets, E).to(GRAD_DTYPE)
            else:
                G.grouped_wgrad(act, d_down, offsets, E, out=w_down.grad, accumulate=True)
        d_act = G.grouped_gemm(d_down, wd, tile_group, w_kmajor=True, out=torch.zeros(R, H, dtype=BF16, device=xn.device))
        del act
        d_pre = ew.swiglu_bwd(pre, d_act, beta, limit)
        del pre, d_act
        if w_up.requires_grad:
            if w_up.grad is None:
                w_up.grad = G.grouped_wgrad(x_perm, d_pre, offsets, E).view(w_up.shape).to(GRAD_DTYPE)
            else:
                G.grouped_wgrad(x_perm, d_pre, offsets, E, out=w_up.grad.view(E, C, 2 * H), accumulate=True)
        dx_perm = G.grouped_gemm(d_pre, wu, tile_group, w_kmajor=True, out=torch.zeros(R, C, dtype=BF16, device=xn.device))
        dxn = ew.gather_sum_rows(dx_perm, dest, F_, K)
        if up_bias is not None and up_bias.requires_grad:
            _add_grad(up_bias, _segment_sum(d_pre, offsets, E))
        if down_bias is not None and down_bias.requires_grad:
            _add_grad(down_bias, _segment_sum(d_down, offsets, E))
        return dxn, dscores, None, None, None, None, None, None, None


def _segment_sum(rows: torch.Tensor, offsets: torch.Tensor, E: int) -> torch.Tensor:
    off = offsets.tolist()
    return torch.stack([rows[off[e]:off[e + 1]].float().sum(0) for e in range(E)])


def moe_experts(xn, scores, indices, w_up, up_bias, w_down, down_bias, beta, limit):
    return _MoEExperts.apply(xn.contiguous(), scores.float().contiguous(), indices.contiguous(), w_up, up_bias, w_down, down_bias, beta, limit)
