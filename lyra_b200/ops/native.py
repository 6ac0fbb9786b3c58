"""ctypes bindings of the in-tree native libraries.

``kernels()`` returns the sm_100a kernel library, ``io()`` the host runtime. On a machine with a
GPU a missing kernel library is an error (the CUDA path must be the one that runs); on a CPU-only
machine ``kernels_available()`` is False and callers use the PyTorch reference implementations.
"""

from __future__ import annotations

import ctypes
import functools
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class NativeError(RuntimeError):
    pass


@functools.cache
def _load(name: str) -> ctypes.CDLL | None:
    path = _LIB_DIR / name
    if not path.exists():
        try:
            from lyra_b200 import build

            build.build_all()
        except Exception:
            return None
    if not path.exists():
        return None
    return ctypes.CDLL(str(path))


def kernels() -> ctypes.CDLL:
    lib = _load("liblyra_b200_kernels.so")
    if lib is None:
        raise NativeError("liblyra_b200_kernels.so is not built; run `python -m lyra_b200.build`")
    return lib


def io() -> ctypes.CDLL:
    lib = _load("liblyra_b200_io.so")
    if lib is None:
        raise NativeError("liblyra_b200_io.so is not built; run `python -m lyra_b200.build`")
    return lib


@functools.cache
def kernels_available() -> bool:
    """True when a CUDA device is present. A GPU box without the library raises instead."""
    if not torch.cuda.is_available():
        return False
    kernels()
    return True


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> c_void_p:
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


_status: dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait gives up."""
    dev = torch.cuda.current_device()
    if dev not in _status:
        _status[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _status[dev]


STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free stage",
    3: "timeout waiting for an accumulator",
    4: "timeout waiting for a peer flag",
    5: "bad argument",
    6: "expert-parallel receive buffer overflow (raise LYRA_EP_CAPACITY)",
    7: "timeout waiting for the rows of a tile that other GPUs store (expert dispatch)",
    8: "timeout waiting for dispatched rows to come back from the experts' GPUs",
}


def check_status() -> None:
    """Reads the status word (synchronises) and raises if any kernel reported a failed wait."""
    if not _status:
        return
    for dev, word in _status.items():
        code = int(word.item())
        if code != 0:
            word.zero_()
            raise NativeError(f"device {dev}: kernel reported '{STATUS_NAMES.get(code, code)}'")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


_launches = 0


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    return _launches
