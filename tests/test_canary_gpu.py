"""Out-of-bounds writes, caught without a sanitizer: every kernel output that takes a caller-provided buffer is placed in
the middle of a larger allocation filled with a bit pattern; after the launch the guard regions before and behind the
output (and, where the contract says so, the untouched rows inside it) must still hold the pattern. Shapes are the
awkward ones: ragged groups, empty groups, extents that are no multiple of a tile."""

import pytest
import torch

pytestmark = pytest.mark.gpu
GUARD = 4096          # elements on either side
PATTERN = -7.625      # exactly representable in bf16 / fp32; never produced by the tests' data in whole rows


class Guarded:
    """A tensor of ``shape`` inside a larger flat buffer pre-filled with ``PATTERN``."""

    def __init__(self, shape, dtype):
        n = 1
        for d in shape:
            n *= d
        self.flat = torch.full((n + 2 * GUARD,), PATTERN, dtype=dtype, device="cuda")
        self.view = self.flat[GUARD:GUARD + n].view(shape)
        self.n = n

    def intact(self) -> bool:
        return bool((self.flat[:GUARD] == PATTERN).all() and (self.flat[GUARD + self.n:] == PATTERN).all())


def _padded_layout(sizes, device):
    offsets, tile_group, row = [0], [], 0
    for g, n in enumerate(sizes):
        tiles = (n + 127) // 128
        tile_group += [g] * tiles
        row += tiles * 128
        offsets.append(row)
    tile_group += [-1, -1]                       # two unused tiles at the end
    R = row + 256
    return (torch.tensor(tile_group, dtype=torch.int32, device=device), torch.tensor(offsets, dtype=torch.int32, device=device), R)


@pytest.mark.parametrize("shape", [(200, 136, 72), (129, 264, 200), (1, 8, 64), (300, 520, 4104)])
def test_dense_gemm_stays_inside_its_output(shape):
    from lyra_b200.ops import gemm as G, native

    M, N, K = shape
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    for dtype in (torch.bfloat16, torch.float32):
        out = Guarded((M, N), dtype)
        G.gemm(a, b, b_mn=True, out=out.view)
        torch.cuda.synchronize()
        native.check_status()
        assert out.intact()
        assert ((out.view.float() - a.float() @ b.float()).norm() / (a.float() @ b.float()).norm()).item() < 2e-2


def test_grouped_gemms_leave_unused_tiles_and_neighbours_alone():
    from lyra_b200.ops import gemm as G, native

    sizes = [130, 0, 5, 256, 77]
    K, N = 192, 320
    tile_group, offsets, R = _padded_layout(sizes, "cuda")
    x = torch.randn(R, K, device="cuda").bfloat16()
    w = (torch.randn(len(sizes), K, N, device="cuda") / 8).bfloat16()
    used = int(offsets[-1])
    for kw, cols in ((dict(), N), (dict(swiglu=True), N // 2)):
        out = Guarded((R, cols), torch.bfloat16)
        G.grouped_gemm(x, w, tile_group, out=out.view, **kw)
        torch.cuda.synchronize()
        native.check_status()
        assert out.intact()
        assert bool((out.view[used:] == PATTERN).all())          # rows of unused tiles are not written
    dw = Guarded((len(sizes), K, N), torch.float32)
    G.grouped_wgrad(x, torch.randn(R, N, device="cuda").bfloat16(), offsets, len(sizes), out=dw.view)
    torch.cuda.synchronize()
    assert dw.intact() and float(dw.view[1].abs().max()) == 0.0     # the empty group's gradient is zero-filled, nothing beyond


def test_row_limited_elementwise_kernels_respect_the_row_count():
    from lyra_b200.ops import elementwise as ew

    M, H, live = 640, 264, 301
    pre = torch.randn(M, 2 * H, device="cuda").bfloat16()
    rows = torch.tensor([live], dtype=torch.int32, device="cuda")
    act = ew.swiglu_fwd(pre, 1.702, 7.0, rows_dev=rows)
    full = ew.swiglu_fwd(pre, 1.702, 7.0)
    assert torch.equal(act[:live], full[:live])
    d = ew.swiglu_bwd(pre, torch.randn(M, H, device="cuda").bfloat16(), 1.702, 7.0, rows_dev=rows)
    assert torch.isfinite(d[:live].float()).all()


def test_decode_gemm_and_routing_outputs_have_no_overrun():
    """These ops allocate their own outputs; the check is that neighbouring allocations made right before and after survive."""
    from lyra_b200.nn.quant import quantize
    from lyra_b200.ops import decode, native, routing

    before = torch.full((1 << 16,), PATTERN, device="cuda")
    G_, K, N, rows = 6, 320, 192, 5
    x = torch.randn(G_ * rows, K, device="cuda").bfloat16()
    w8 = quantize(torch.randn(G_, K, N, device="cuda") / K ** 0.5, torch.float8_e4m3fn, block=(64, 64))
    offsets = torch.arange(G_ + 1, device="cuda", dtype=torch.int32) * rows
    y = decode.decode_gemm(x, w8, offsets=offsets, max_group_rows=rows)
    s, idx, aux, plan = routing.route(torch.randn(333, 31, device="cuda"), None, 3, 1e-2, 1e-4)
    after = torch.full((1 << 16,), PATTERN, device="cuda")
    torch.cuda.synchronize()
    native.check_status()
    assert bool((before == PATTERN).all()) and bool((after == PATTERN).all())
    assert torch.isfinite(y.float()).all() and int(plan.counts.sum()) == 333 * 3
