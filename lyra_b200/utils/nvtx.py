"""Named regions. The region names equal the reference's ``jax.named_scope`` names (lyra/model.py:284-775,
lyra/training/steps.py:31-189) and show up as NVTX ranges in profiler timelines when ``LYRA_NVTX=1`` and a CUDA device is present."""

from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("LYRA_NVTX", "0") == "1"


def enable(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = flag


@contextlib.contextmanager
def _range(name: str):
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def scope(name: str):
    if _ENABLED and torch.cuda.is_available():
        return _range(name)
    return _NULL
