"""Bandwidth-bound fused ops around the GEMMs and attention: RMSNorm, QK-norm + RoPE, output gate + XSA,
SwiGLU, embedding gather / deterministic gradient, and the MoE row movement (scatter into the padded
expert-sorted layout, weighted combine and their gradients). CUDA kernels live in ``csrc/elementwise`` and
``csrc/moe``; each function falls back to the equivalent PyTorch expression when its kernel is not available
for the given dtype or shape."""

from __future__ import annotations

import torch

from lyra_b200.ops import native
from lyra_b200.ops import reference as ref
from lyra_b200.ops.native import c_float, c_int, c_ll, ptr

BF16 = torch.bfloat16


def _lib():
    return native.kernels()


def _has(name: str) -> bool:
    return hasattr(_lib(), name)


# --------------------------------------------------------------------------- RMSNorm
class RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, eps):
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        if x2.dtype == BF16 and x2.is_contiguous() and _has("lyra_rmsnorm_fwd") and C % 8 == 0:
            y = torch.empty_like(x2)
            rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
            sc = scale.detach().float().contiguous()
            native.check(_lib().lyra_rmsnorm_fwd(ptr(x2), ptr(sc), ptr(y), ptr(rstd), c_int(x2.shape[0]), c_int(C), c_float(eps),
                                                 native.stream_ptr()), "rmsnorm_fwd")
            native.count_launch()
        else:
            xf = x2.float()
            rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
            y = (xf * rstd[:, None] * scale.float()).to(x.dtype)
        ctx.save_for_backward(x2, scale, rstd)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, scale, rstd = ctx.saved_tensors
        C = x2.shape[-1]
        dy2 = dy.reshape(-1, C)
        if x2.dtype == BF16 and dy2.dtype == BF16 and _has("lyra_rmsnorm_bwd") and C % 8 == 0:
            dy2 = dy2.contiguous()
            dx = torch.empty_like(x2)
            rows = x2.shape[0]
            nblk = min(1024, max(1, (rows + 31) // 32))
            partial = torch.empty(nblk, C, dtype=torch.float32, device=x2.device)
            sc = scale.detach().float().contiguous()
            native.check(_lib().lyra_rmsnorm_bwd(ptr(x2), ptr(sc), ptr(rstd), ptr(dy2), ptr(dx), ptr(partial), c_int(rows), c_int(C),
                                                 c_int(nblk), native.stream_ptr()), "rmsnorm_bwd")
            native.count_launch()
            dscale = partial.sum(0)
        else:
            xf, dyf = x2.float(), dy2.float()
            xhat = xf * rstd[:, None]
            g = dyf * scale.float()
            dx = ((g - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd[:, None]).to(x2.dtype)
            dscale = (dyf * xhat).sum(0)
        return dx.reshape(dy.shape), dscale.to(scale.dtype).reshape(scale.shape), None


# --------------------------------------------------------------------------- QK-norm + RoPE
class _QKNormRope(torch.autograd.Function):
    """Per-head RMS norm (optional) followed by the half-split rotation, applied to q and k in one pass."""

    @staticmethod
    def forward(ctx, x, scale, cos, sin, eps):
        # x [B, T, N, D]; cos/sin [1, T, 1, D/2]
        xf = x.float()
        if scale is not None:
            rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            xn = xf * rstd * scale.float()
        else:
            rstd = None
            xn = xf
        y = ref.rotate(xn, cos, sin).to(x.dtype)
        ctx.save_for_backward(x, scale, rstd, cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, scale, rstd, cos, sin = ctx.saved_tensors
        d1, d2 = dy.float().chunk(2, dim=-1)
        # inverse rotation (transpose of the rotation matrix)
        dxn = torch.cat([d1 * cos + d2 * sin, d2 * cos - d1 * sin], dim=-1)
        if scale is None:
            return dxn.to(x.dtype), None, None, None, None
        xf = x.float()
        xhat = xf * rstd
        g = dxn * scale.float()
        dx = (g - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd
        dscale = (dxn * xhat).sum(dim=(0, 1, 2))
        return dx.to(x.dtype), dscale.to(scale.dtype), None, None, None


def qk_norm_rope(q, k, qscale, kscale, cos, sin, eps):
    if q.dtype == BF16 and _has("lyra_qknorm_rope_fwd") and not (q.requires_grad or k.requires_grad) and q.is_contiguous() and k.is_contiguous():
        return _qknorm_rope_kernel(q, qscale, cos, sin, eps), _qknorm_rope_kernel(k, kscale, cos, sin, eps)
    return _QKNormRope.apply(q, qscale, cos, sin, eps), _QKNormRope.apply(k, kscale, cos, sin, eps)


def _qknorm_rope_kernel(x, scale, cos, sin, eps):
    B, T, N, D = x.shape
    y = torch.empty_like(x)
    sc = scale.detach().float().contiguous() if scale is not None else None
    c2, s2 = cos.reshape(-1, D // 2).contiguous(), sin.reshape(-1, D // 2).contiguous()
    native.check(_lib().lyra_qknorm_rope_fwd(ptr(x), ptr(sc), ptr(c2), ptr(s2), ptr(y), c_int(B), c_int(T), c_int(N), c_int(D), c_float(eps),
                                             native.stream_ptr()), "qknorm_rope_fwd")
    native.count_launch()
    return y


# --------------------------------------------------------------------------- output gate + XSA
def gate_xsa(t, h, w_gate, v, xsa_alpha):
    """See ``ops.api.gate_xsa``. Autograd-differentiable composition; heads-first ``t [B, Nq, T, D]``."""
    dtype = t.dtype
    if w_gate is not None:
        from lyra_b200.ops import cuda_ops

        B, T, C = h.shape
        nq = w_gate.shape[1]
        if nq % 8 == 0:
            logits = cuda_ops.linear(h, w_gate, None, out_dtype=None).float()
        else:
            logits = h.float() @ w_gate.float()
        gate = 2.0 * torch.sigmoid(logits)                    # [B, T, Nq]
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


# --------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(pre: torch.Tensor, beta: float, limit: float) -> torch.Tensor:
    """``pre [M, 2H]`` (gate columns then linear columns) -> ``[M, H]``."""
    M, H2 = pre.shape
    H = H2 // 2
    if pre.dtype == BF16 and _has("lyra_swiglu_fwd") and H % 8 == 0:
        out = torch.empty(M, H, dtype=BF16, device=pre.device)
        native.check(_lib().lyra_swiglu_fwd(ptr(pre), ptr(out), c_ll(M), c_int(H), c_float(beta), c_float(limit), native.stream_ptr()), "swiglu_fwd")
        native.count_launch()
        return out
    return ref.swiglu(pre.float().view(M, 2, H), beta, limit).to(pre.dtype)


def swiglu_bwd(pre: torch.Tensor, dact: torch.Tensor, beta: float, limit: float) -> torch.Tensor:
    """Gradient w.r.t. ``pre [M, 2H]`` given ``dact [M, H]``; clamped regions pass no gradient."""
    M, H2 = pre.shape
    H = H2 // 2
    if pre.dtype == BF16 and dact.dtype == BF16 and _has("lyra_swiglu_bwd") and H % 8 == 0:
        out = torch.empty_like(pre)
        native.check(_lib().lyra_swiglu_bwd(ptr(pre), ptr(dact.contiguous()), ptr(out), c_ll(M), c_int(H), c_float(beta), c_float(limit),
                                            native.stream_ptr()), "swiglu_bwd")
        native.count_launch()
        return out
    g, l = pre[:, :H].float(), pre[:, H:].float()
    gc, lc = g.clamp(max=limit), l.clamp(-limit, limit)
    sig = torch.sigmoid(beta * gc)
    d = dact.float()
    dg = d * (lc + 1.0) * (sig + gc * beta * sig * (1 - sig)) * (g <= limit)
    dl = d * gc * sig * ((l >= -limit) & (l <= limit))
    return torch.cat([dg, dl], dim=1).to(pre.dtype)


# --------------------------------------------------------------------------- embedding
class Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, emb, tokens):
        ctx.save_for_backward(tokens)
        ctx.emb = emb
        return emb.detach()[tokens]

    @staticmethod
    def backward(ctx, g):
        (tokens,) = ctx.saved_tensors
        emb = ctx.emb
        flat = tokens.reshape(-1).long()
        g2 = g.reshape(flat.shape[0], -1)
        # deterministic: sorted segment-sum in fp32 (lyra/kernels/embs.py:22-29), accumulated into the gradient buffer
        order = torch.argsort(flat, stable=True)
        sorted_ids = flat[order]
        uniq, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
        seg = torch.repeat_interleave(torch.arange(uniq.numel(), device=flat.device), counts)
        sums = torch.zeros(uniq.numel(), g2.shape[1], dtype=torch.float32, device=g.device)
        sums.index_add_(0, seg, g2[order].float())
        if emb.grad is None:
            from lyra_b200.ops import cuda_ops

            emb.grad = torch.zeros(emb.shape, dtype=cuda_ops.GRAD_DTYPE, device=emb.device)
        emb.grad.index_add_(0, uniq, sums.to(emb.grad.dtype))
        return None, None


# --------------------------------------------------------------------------- MoE row movement
def scatter_rows(xn: torch.Tensor, dest: torch.Tensor, K: int, R: int) -> torch.Tensor:
    """``out[dest[f*K + k]] = xn[f]`` into a zeroed ``[R, C]`` buffer (expert-sorted, padded layout)."""
    out = torch.zeros(R, xn.shape[1], dtype=xn.dtype, device=xn.device)
    if _has("lyra_scatter_rows") and xn.dtype == BF16:
        native.check(_lib().lyra_scatter_rows(ptr(xn), ptr(dest), ptr(out), c_int(xn.shape[0]), c_int(K), c_int(xn.shape[1]),
                                              native.stream_ptr()), "scatter_rows")
        native.count_launch()
        return out
    out[dest] = xn.repeat_interleave(K, dim=0)
    return out


def combine_rows(rows: torch.Tensor, dest: torch.Tensor, scores: torch.Tensor, F_: int, K: int) -> torch.Tensor:
    """``out[f] = sum_k scores[f, k] * rows[dest[f*K + k]]`` with fp32 accumulation in a fixed order."""
    if _has("lyra_combine_rows") and rows.dtype == BF16:
        out = torch.empty(F_, rows.shape[1], dtype=BF16, device=rows.device)
        native.check(_lib().lyra_combine_rows(ptr(rows), ptr(dest), ptr(scores), ptr(out), c_int(F_), c_int(K), c_int(rows.shape[1]),
                                              native.stream_ptr()), "combine_rows")
        native.count_launch()
        return out
    g = rows[dest].view(F_, K, -1).float()
    return (g * scores.float()[..., None]).sum(1).to(rows.dtype)


def combine_rows_bwd(rows, dout, dest, scores, R: int):
    """Returns ``(d_rows [R, C] with pad rows zero, dscores [F, K])``."""
    F_, K = scores.shape
    C = rows.shape[1]
    if _has("lyra_combine_rows_bwd") and rows.dtype == BF16:
        d_rows = torch.zeros(R, C, dtype=BF16, device=rows.device)
        dscores = torch.empty(F_, K, dtype=torch.float32, device=rows.device)
        native.check(_lib().lyra_combine_rows_bwd(ptr(rows), ptr(dout), ptr(dest), ptr(scores), ptr(d_rows), ptr(dscores), c_int(F_), c_int(K),
                                                  c_int(C), native.stream_ptr()), "combine_rows_bwd")
        native.count_launch()
        return d_rows, dscores
    g = rows[dest].view(F_, K, C).float()
    dscores = (g * dout.float()[:, None, :]).sum(-1)
    d_rows = torch.zeros(R, C, dtype=rows.dtype, device=rows.device)
    d_rows[dest] = (scores.float()[..., None] * dout.float()[:, None, :]).to(rows.dtype).view(F_ * K, C)
    return d_rows, dscores


def gather_sum_rows(rows: torch.Tensor, dest: torch.Tensor, F_: int, K: int) -> torch.Tensor:
    """``out[f] = sum_k rows[dest[f*K + k]]`` (gradient of :func:`scatter_rows`)."""
    if _has("lyra_combine_rows") and rows.dtype == BF16:
        ones = torch.ones(F_, K, dtype=torch.float32, device=rows.device)
        return combine_rows(rows, dest, ones, F_, K)
    return rows[dest].view(F_, K, -1).float().sum(1).to(rows.dtype)
