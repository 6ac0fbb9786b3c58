"""A peer that never answers: the bounded device-side wait gives up, reports a status code, and the context stays usable."""

import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_expires_with_status_and_context_survives():
    from lyra_b200.ops import gemm as G, native

    lib = native.kernels()
    native.check_status()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")       # nobody ever raises these
    t0 = time.perf_counter()
    native.check(lib.lyra_wait_limit(native.ptr(flags), ctypes.c_int(2), ctypes.c_int(1), native.ptr(native.status_word()), ctypes.c_int(200),
                                     native.stream_ptr()), "wait")
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.15 < waited < 1.5, waited                             # gave up after about 200 ms, not the 2 s default, not at once
    with pytest.raises(native.NativeError, match="peer flag"):
        native.check_status()
    native.check_status()                                          # the status word was cleared by the failed check
    # a flag that is already raised returns at once
    flags.fill_(1)
    native.check(lib.lyra_wait_limit(native.ptr(flags), ctypes.c_int(2), ctypes.c_int(1), native.ptr(native.status_word()), ctypes.c_int(200),
                                     native.stream_ptr()), "wait")
    native.check_status()
    # and the device still computes
    a = torch.randn(256, 128, device="cuda").bfloat16()
    b = torch.randn(128, 128, device="cuda").bfloat16()
    y = G.gemm(a, b)
    assert (y.float() - a.float() @ b.float().t()).abs().max().item() < 0.5
