"""Block-scaled fp8 arrays: ``QArray(qval, scale, block)`` with the reference's semantics
(lyra/nn/quant.py:14-113): block absmax over the trailing ``len(block)`` dims, fp32 scale
``amax / fmax`` (1.0 for an all-zero block), values clipped to the format's finite range.
This module is the oracle; the CUDA kernels in ``csrc/quant`` implement the hot cases
(KV-cache append with ``(1, head_dim)`` blocks, weight quantisation).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def is_scaled(dtype: torch.dtype) -> bool:
    return dtype in FP8_DTYPES


@dataclass(frozen=True)
class QArray:
    qval: torch.Tensor
    scale: torch.Tensor
    block: tuple[int, ...]

    @property
    def dtype(self):
        return self.qval.dtype

    @property
    def shape(self):
        return tuple(self.qval.shape)

    @property
    def ndim(self):
        return self.qval.ndim

    @property
    def stype(self):
        return self.scale.dtype

    @property
    def ldim(self) -> int:
        return self.qval.ndim - len(self.block)

    def eff_block(self, axis: int) -> int:
        return 1 if axis < self.ldim else self.block[axis - self.ldim]

    def to(self, device) -> "QArray":
        return QArray(self.qval.to(device), self.scale.to(device), self.block)


def tile(x: torch.Tensor, block: tuple[int, ...]) -> torch.Tensor:
    n = len(block)
    lead, tail = x.shape[: x.ndim - n], x.shape[x.ndim - n:]
    bad = [(d, b) for d, b in zip(tail, block) if d % b]
    if bad:
        raise ValueError(f"block {block} does not divide trailing dims {tuple(tail)}")
    return x.reshape(*lead, *(v for d, b in zip(tail, block) for v in (d // b, b)))


def block_axes(ldim: int, sdim: int) -> tuple[int, ...]:
    return tuple(ldim + 2 * i + 1 for i in range(sdim))


def quantize(x, dtype: torch.dtype, block: tuple[int, ...] = (128, 128), scale_dtype: torch.dtype = torch.float32) -> QArray:
    if isinstance(x, QArray):
        if x.block != tuple(block) or x.dtype != dtype:
            raise ValueError(f"already quantized as {x.dtype}/{x.block}; requested {dtype}/{block}")
        return x
    if not is_scaled(dtype):
        raise ValueError(f"quantize target must be fp8, got {dtype}")
    if is_scaled(scale_dtype):
        raise ValueError("scale dtype must be unscaled (fp32/bf16)")
    block = tuple(block)
    fast = _quantize_kernel(x, dtype, block, scale_dtype)
    if fast is not None:
        return fast
    sdim = len(block)
    ldim = x.ndim - sdim
    axes = block_axes(ldim, sdim)
    tiled = tile(x, block).float()
    fmax = float(torch.finfo(dtype).max)
    amax = tiled.abs().amax(dim=axes)
    scale = torch.where(amax > 0, amax / fmax, torch.ones_like(amax)).to(scale_dtype)
    qinv = 1.0 / scale.float()
    for a in axes:
        qinv = qinv.unsqueeze(a)
    qval = (tiled * qinv).clamp(-fmax, fmax).to(dtype).reshape(x.shape)
    return QArray(qval, scale, block)


def _kernel_lib(t: torch.Tensor):
    """The CUDA kernel library when ``t`` lives on a GPU, else None (CPU tensors use the PyTorch formulas below)."""
    if not t.is_cuda:
        return None
    from lyra_b200.ops import native

    return native.kernels() if native.kernels_available() else None


def _quantize_kernel(x: torch.Tensor, dtype, block: tuple[int, ...], scale_dtype) -> "QArray | None":
    """CUDA path of ``quantize`` for e4m3 with a 2-D block over the last two axes (weights; KV rows when the block is (1, D))."""
    if dtype != torch.float8_e4m3fn or scale_dtype != torch.float32 or len(block) != 2 or x.ndim < 2:
        return None
    if x.dtype not in (torch.float32, torch.bfloat16) or x.numel() == 0:
        return None
    lib = _kernel_lib(x)
    if lib is None:
        return None
    # a strided view (e.g. the value slice of a fused q | k | v projection) is copied rather than sent down the PyTorch path: that
    # path divides by the scale where the kernels multiply by its rounded reciprocal, and the two round a few values differently
    x = x.contiguous()
    import ctypes

    from lyra_b200.ops import native

    R, C = x.shape[-2], x.shape[-1]
    br, bc = block
    if R % br or C % bc:
        return None
    L = x.numel() // (R * C)
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty(*x.shape[:-2], R // br, C // bc, dtype=torch.float32, device=x.device)
    is_bf16 = ctypes.c_int(int(x.dtype == torch.bfloat16))
    if br == 1 and bc % 32 == 0 and bc <= 1024:
        # one scale per (row, run of bc values): the runs are contiguous, so the array is a list of L * R * C / bc rows of bc values
        # (KV-cache rows with bc == C; activations of the e4m3 products with bc = the K block of the weights' scales)
        rc = lib.lyra_fp8_quantize_rows(native.ptr(x), is_bf16, native.ptr(q), native.ptr(scale), ctypes.c_longlong(L * R * (C // bc)), ctypes.c_int(bc),
                                        ctypes.c_longlong(bc), ctypes.c_longlong(bc), native.stream_ptr())
    elif L <= 65535 and R // br <= 65535:
        rc = lib.lyra_fp8_quantize_2d(native.ptr(x), is_bf16, native.ptr(q), native.ptr(scale), ctypes.c_int(L), ctypes.c_int(R), ctypes.c_int(C),
                                      ctypes.c_int(br), ctypes.c_int(bc), native.stream_ptr())
    else:
        return None
    native.check(rc, "fp8 quantize")
    native.count_launch()
    return QArray(q, scale, block)


def _dequantize_kernel(qx: "QArray", dtype) -> "torch.Tensor | None":
    if dtype != torch.bfloat16 or qx.qval.dtype != torch.float8_e4m3fn or len(qx.block) != 2 or qx.qval.ndim < 2:
        return None
    if qx.scale.dtype != torch.float32 or not qx.qval.is_contiguous() or not qx.scale.is_contiguous() or qx.qval.numel() == 0:
        return None
    R, C = qx.qval.shape[-2], qx.qval.shape[-1]
    br, bc = qx.block
    if R % br or C % bc or bc % 16:
        return None
    lib = _kernel_lib(qx.qval)
    if lib is None:
        return None
    import ctypes

    from lyra_b200.ops import native

    out = torch.empty(qx.qval.shape, dtype=torch.bfloat16, device=qx.qval.device)
    L = qx.qval.numel() // (R * C)
    rc = lib.lyra_fp8_dequantize_2d(native.ptr(qx.qval), native.ptr(qx.scale), native.ptr(out), ctypes.c_int(L), ctypes.c_int(R), ctypes.c_int(C),
                                    ctypes.c_int(br), ctypes.c_int(bc), native.stream_ptr())
    native.check(rc, "fp8 dequantize")
    native.count_launch()
    return out


def dequantize(qx: QArray, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    fast = _dequantize_kernel(qx, dtype)
    if fast is not None:
        return fast
    axes = block_axes(qx.ldim, len(qx.block))
    tiled = tile(qx.qval.float(), qx.block)
    scale = qx.scale.float()
    for a in axes:
        scale = scale.unsqueeze(a)
    return (tiled * scale).reshape(qx.shape).to(dtype)


def qupdate(qx: QArray, x: torch.Tensor, start: tuple) -> QArray:
    """Writes ``x`` (quantised with ``qx``'s format) at ``start`` - values and scales (lyra/nn/quant.py:89-98).
    The update is in place on ``qx``'s storage; the returned QArray aliases it."""
    for axis, s in enumerate(start):
        b = qx.eff_block(axis)
        if isinstance(s, int) and s % b:
            raise ValueError(f"start {s} on axis {axis} is not aligned to block {b}")
    qnew = quantize(x, qx.dtype, qx.block, qx.stype)
    idx = tuple(slice(int(s), int(s) + n) for s, n in zip(start, qnew.qval.shape))
    qx.qval[idx] = qnew.qval
    sidx = tuple(slice(int(s) // qx.eff_block(axis), int(s) // qx.eff_block(axis) + n)
                 for axis, (s, n) in enumerate(zip(start, qnew.scale.shape)))
    qx.scale[sidx] = qnew.scale
    return QArray(qx.qval, qx.scale, qx.block)


def maybe_dequant(x, dtype: torch.dtype) -> torch.Tensor:
    return dequantize(x, dtype) if isinstance(x, QArray) else x


def dot(lhs: torch.Tensor, rhs) -> torch.Tensor:
    """``lhs @ rhs`` with a possibly quantised right operand (dequantise-then-matmul, lyra/nn/quant.py:106-108)."""
    return lhs @ maybe_dequant(rhs, lhs.dtype).to(lhs.dtype)
