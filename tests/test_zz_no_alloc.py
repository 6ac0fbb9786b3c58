"""Allocation-free RMSNorm backward (``lyra_rmsnorm_bwd_noalloc``), called through its exported C symbol.

Some users of the library cannot allocate device memory when they call it: a host program whose own pool already holds
all device memory, a latency-critical loop that must avoid the synchronisation an allocation can bring, or a plain C
caller without PyTorch's allocator. For them the scratch of the kernel lives in a fixed array inside the library. The
test checks the entry point against the regular one (which takes caller-allocated scratch) on two calls in a row -
the second with fewer rows and a different width, so left-over scratch contents from the first call would show - and
that a width beyond the built-in scratch is refused without launching anything. This file sorts last so that a
``pytest -x`` run has already run every other test before it.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(lib, rows, C, seed):
    from lyra_b200.ops.native import c_float, c_int, ptr, stream_ptr

    torch.manual_seed(seed)
    x = torch.randn(rows, C, device="cuda").bfloat16()
    dy = torch.randn(rows, C, device="cuda").bfloat16()
    scale = torch.rand(C, device="cuda") + 0.5
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    # regular entry point: the caller allocates the per-block partial sums and adds them up
    nblk = min(1024, max(1, (rows + 31) // 32))
    partial = torch.empty(nblk, C, dtype=torch.float32, device="cuda")
    dx_ref = torch.empty_like(x)
    assert lib.lyra_rmsnorm_bwd(ptr(x), ptr(scale), ptr(rstd), ptr(dy), ptr(dx_ref), ptr(partial), c_int(rows), c_int(C), c_int(nblk), stream_ptr()) == 0
    dscale_ref = partial.sum(0)
    # allocation-free entry point: inputs and outputs only
    dx = torch.empty_like(x)
    dscale = torch.full((C,), float("nan"), device="cuda")
    fn = lib.lyra_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    assert fn(ptr(x), ptr(scale), ptr(rstd), ptr(dy), ptr(dx), ptr(dscale), c_int(rows), c_int(C), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert (dx.float() - dx_ref.float()).abs().max().item() <= 1e-2 * dx_ref.float().abs().max().item()
    rel = ((dscale - dscale_ref).norm() / dscale_ref.norm()).item()
    assert rel < 1e-3, rel


def test_noalloc_entry_point_matches_regular_one_twice_in_a_row():
    from lyra_b200.ops import native

    lib = native.kernels()
    assert hasattr(lib, "lyra_rmsnorm_bwd_noalloc")
    _run_both(lib, 3000, 4096, seed=0)
    _run_both(lib, 77, 2880, seed=1)      # fewer blocks and a narrower row than the call before


def test_noalloc_entry_point_rejects_widths_beyond_its_scratch():
    from lyra_b200.ops import native
    from lyra_b200.ops.native import c_int, ptr, stream_ptr

    lib = native.kernels()
    fn = lib.lyra_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    t = torch.zeros(8, device="cuda")
    assert fn(ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), c_int(1), c_int(8192 + 8), stream_ptr()) == -70
    assert fn(ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), c_int(1), c_int(12), stream_ptr()) == -71
