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
            # rows of the partial-sum buffer: one per block of the block-per-row kernel, one per warp of the warp-per-row
            # kernel that serves C % 256 == 0, C <= 2048 (148 SMs x 8 warps)
            nblk = min(1184, max(1, rows // 4)) if (C % 256 == 0 and C <= 2048) else min(1024, max(1, (rows + 31) // 32))
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


class _QKNormRopeKernel(torch.autograd.Function):
    """Kernel-backed version of :class:`_QKNormRope` for contiguous bf16 ``[B, T, N, D]`` inputs."""

    @staticmethod
    def forward(ctx, x, scale, cos, sin, eps):
        D = x.shape[-1]
        c2, s2 = cos.reshape(-1, D // 2).contiguous(), sin.reshape(-1, D // 2).contiguous()
        ctx.save_for_backward(x, scale, c2, s2)
        ctx.eps = eps
        return _qknorm_rope_kernel(x, scale, c2, s2, eps)

    @staticmethod
    def backward(ctx, dy):
        x, scale, c2, s2 = ctx.saved_tensors
        B, T, N, D = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        max_blocks = 1184
        partial = torch.empty(max_blocks, D, dtype=torch.float32, device=x.device) if scale is not None else None
        sc = scale.detach().float().contiguous() if scale is not None else None
        lib = _lib()
        lib.lyra_qknorm_rope_bwd.restype = c_int
        used = lib.lyra_qknorm_rope_bwd(ptr(x), ptr(sc), ptr(c2), ptr(s2), ptr(dy), ptr(dx), ptr(partial), c_int(B), c_int(T), c_int(N), c_int(D),
                                        c_float(ctx.eps), c_int(max_blocks), native.stream_ptr())
        if used < 0:
            raise native.NativeError(f"qknorm_rope_bwd failed with code {used}")
        native.count_launch()
        dscale = partial[:used].sum(0).to(scale.dtype) if scale is not None else None
        return dx, dscale, None, None, None


def _token_strided(x) -> bool:
    """``[B, T, N, D]`` whose heads are contiguous inside a token and whose tokens are evenly spaced (a slice of a fused projection)."""
    B, T, N, D = x.shape
    return x.stride(3) == 1 and x.stride(2) == D and x.stride(1) >= N * D and (B == 1 or x.stride(0) == T * x.stride(1))


def qk_norm_rope(q, k, qscale, kscale, cos, sin, eps):
    ok = (q.dtype == BF16 and k.dtype == BF16 and _has("lyra_qknorm_rope_bwd") and q.shape[-1] in (64, 128) and q.dim() == 4)
    if ok and not (q.is_contiguous() and k.is_contiguous()):
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad) or not (_token_strided(q) and _token_strided(k)):
            q, k = q.contiguous(), k.contiguous()          # the backward kernel takes contiguous inputs only
    if ok:
        return _QKNormRopeKernel.apply(q, qscale, cos, sin, eps), _QKNormRopeKernel.apply(k, kscale, cos, sin, eps)
    return _QKNormRope.apply(q, qscale, cos, sin, eps), _QKNormRope.apply(k, kscale, cos, sin, eps)


def _qknorm_rope_kernel(x, scale, c2, s2, eps):
    B, T, N, D = x.shape
    y = torch.empty(B, T, N, D, dtype=x.dtype, device=x.device)
    sc = scale.detach().float().contiguous() if scale is not None else None
    native.check(_lib().lyra_qknorm_rope_fwd(ptr(x), ptr(sc), ptr(c2), ptr(s2), ptr(y), c_int(B), c_int(T), c_int(N), c_int(D), c_float(eps),
                                             c_ll(x.stride(1)), native.stream_ptr()), "qknorm_rope_fwd")
    native.count_launch()
    return y


# --------------------------------------------------------------------------- output gate + XSA
class _GateXSAKernel(torch.autograd.Function):
    """``t, v`` token-major ``[B, T, N, D]`` bf16; ``logits [B, T, Nq]`` bf16 or None; ``alpha [Nq]`` or None."""

    @staticmethod
    def forward(ctx, t, logits, v, alpha):
        B, T, Nq, D = t.shape
        Nkv = v.shape[2]
        out = torch.empty_like(t)
        al = alpha.detach().float().contiguous() if alpha is not None else None
        native.check(_lib().lyra_gate_xsa_fwd(ptr(t), ptr(logits), ptr(v), ptr(al), ptr(out), c_ll(B * T), c_int(Nq), c_int(Nkv), c_int(D),
                                              native.stream_ptr()), "gate_xsa_fwd")
        native.count_launch()
        ctx.save_for_backward(t, logits, v, alpha)
        return out

    @staticmethod
    def backward(ctx, d_out):
        t, logits, v, alpha = ctx.saved_tensors
        B, T, Nq, D = t.shape
        Nkv = v.shape[2]
        d_out = d_out.contiguous()
        d_t = torch.empty_like(t)
        d_logits = torch.empty_like(logits) if logits is not None else None
        d_v = torch.empty_like(v) if alpha is not None else None
        max_blocks = 1184
        partial = torch.empty(max_blocks, Nq, dtype=torch.float32, device=t.device) if alpha is not None else None
        al = alpha.detach().float().contiguous() if alpha is not None else None
        lib = _lib()
        lib.lyra_gate_xsa_bwd.restype = c_int
        used = lib.lyra_gate_xsa_bwd(ptr(t), ptr(logits), ptr(v), ptr(al), ptr(d_out), ptr(d_t), ptr(d_logits), ptr(d_v), ptr(partial), c_ll(B * T),
                                     c_int(Nq), c_int(Nkv), c_int(D), c_int(max_blocks), native.stream_ptr())
        if used < 0:
            raise native.NativeError(f"gate_xsa_bwd failed with code {used}")
        native.count_launch()
        d_alpha = partial[:used].sum(0).to(alpha.dtype) if alpha is not None else None
        return d_t, d_logits, d_v, d_alpha


def gate_xsa(t, h, w_gate, v, xsa_alpha):
    """See ``ops.api.gate_xsa``. Heads-first ``t [B, Nq, T, D]``; fused kernel when the storage is token-major bf16."""
    dtype = t.dtype
    tt, vt = t.transpose(1, 2), v.transpose(1, 2)
    if (dtype == BF16 and _has("lyra_gate_xsa_fwd") and tt.is_contiguous() and vt.is_contiguous() and t.shape[-1] in (64, 128)
            and (w_gate is None or w_gate.shape[1] % 8 == 0)):
        logits = None
        if w_gate is not None:
            from lyra_b200.ops import cuda_ops

            logits = cuda_ops.linear(h, w_gate, None).contiguous()
        return _GateXSAKernel.apply(tt, logits, vt, xsa_alpha).transpose(1, 2)
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
def swiglu_fwd(pre: torch.Tensor, beta: float, limit: float, rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """``pre [M, 2H]`` (gate columns then linear columns) -> ``[M, H]``. With ``rows_dev`` (int32 device scalar) only that
    many leading rows are computed and the rest of the output is left uninitialised."""
    M, H2 = pre.shape
    H = H2 // 2
    if pre.dtype == BF16 and _has("lyra_swiglu_fwd") and H % 8 == 0:
        out = torch.empty(M, H, dtype=BF16, device=pre.device)
        if rows_dev is not None:
            native.check(_lib().lyra_swiglu_fwd_rows(ptr(pre), ptr(out), c_ll(M), c_int(H), c_float(beta), c_float(limit), ptr(rows_dev),
                                                     native.stream_ptr()), "swiglu_fwd_rows")
            native.count_launch()
            return out
        native.check(_lib().lyra_swiglu_fwd(ptr(pre), ptr(out), c_ll(M), c_int(H), c_float(beta), c_float(limit), native.stream_ptr()), "swiglu_fwd")
        native.count_launch()
        return out
    return ref.swiglu(pre.float().view(M, 2, H), beta, limit).to(pre.dtype)


def swiglu_bwd(pre: torch.Tensor, dact: torch.Tensor, beta: float, limit: float, rows_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Gradient w.r.t. ``pre [M, 2H]`` given ``dact [M, H]``; clamped regions pass no gradient. ``rows_dev`` as in ``swiglu_fwd``."""
    M, H2 = pre.shape
    H = H2 // 2
    if pre.dtype == BF16 and dact.dtype == BF16 and _has("lyra_swiglu_bwd") and H % 8 == 0:
        out = torch.empty_like(pre)
        if rows_dev is not None:
            native.check(_lib().lyra_swiglu_bwd_rows(ptr(pre), ptr(dact.contiguous()), ptr(out), c_ll(M), c_int(H), c_float(beta), c_float(limit),
                                                     ptr(rows_dev), native.stream_ptr()), "swiglu_bwd_rows")
            native.count_launch()
            return out
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
        return emb.detach()[tokens].to(BF16)  # bf16 activations, so the incoming gradient is bf16 too

    @staticmethod
    def backward(ctx, g):
        (tokens,) = ctx.saved_tensors
        emb = ctx.emb
        flat = tokens.reshape(-1).long()
        g2 = g.reshape(flat.shape[0], -1)
        if emb.grad is None:
            from lyra_b200.ops import cuda_ops

            emb.grad = torch.zeros(emb.shape, dtype=cuda_ops.GRAD_DTYPE, device=emb.device)
        # deterministic: sorted segment-sum in fp32 (lyra/kernels/embs.py:22-29), accumulated into the gradient buffer
        sorted_ids, order = torch.sort(flat, stable=True)
        if g2.dtype == BF16 and _has("lyra_embedding_grad") and g2.shape[1] % 8 == 0 and emb.grad.dtype in (BF16, torch.float32):
            g2 = g2.contiguous()
            native.check(_lib().lyra_embedding_grad(ptr(sorted_ids), ptr(order), ptr(g2), ptr(emb.grad), c_int(int(emb.grad.dtype == BF16)),
                                                    c_int(flat.shape[0]), c_int(g2.shape[1]), native.stream_ptr()), "embedding_grad")
            native.count_launch()
        else:
            uniq, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
            seg = torch.repeat_interleave(torch.arange(uniq.numel(), device=flat.device), counts)
            sums = torch.zeros(uniq.numel(), g2.shape[1], dtype=torch.float32, device=g.device)
            sums.index_add_(0, seg, g2[order].float())
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


def combine_rows_bwd(rows, dout, dest, scores, R: int, dense: bool = False):
    """Returns ``(d_rows [R, C] with pad rows zero, dscores [F, K])``. ``dense``: ``dest`` covers every one of the ``R`` rows
    (no padding rows), so the output needs no zero fill."""
    F_, K = scores.shape
    C = rows.shape[1]
    if _has("lyra_combine_rows_bwd") and rows.dtype == BF16:
        d_rows = (torch.empty if dense and R == F_ * K else torch.zeros)(R, C, dtype=BF16, device=rows.device)
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
