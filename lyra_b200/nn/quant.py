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


def dequantize(qx: QArray, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
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
