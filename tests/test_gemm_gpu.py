"""tcgen05 GEMM family against fp32 PyTorch references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 512, 128), (384, 264, 192), (1000, 2880, 2880)])
def test_gemm_layouts(a_mn, b_mn, shape):
    from lyra_b200.ops import gemm as G, native

    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    a_st = a.t().contiguous() if a_mn else a
    b_st = b.t().contiguous() if b_mn else b
    out = G.gemm(a_st, b_st, a_mn=a_mn, b_mn=b_mn)
    native.check_status()
    assert _rel(out, ref) < 1e-2
    out32 = G.gemm(a_st, b_st, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert _rel(out32, ref) < 1e-5 * 300
    assert torch.equal(out, G.gemm(a_st, b_st, a_mn=a_mn, b_mn=b_mn))  # run-to-run bit equality


def test_gemm_epilogue_alpha_beta_bias():
    from lyra_b200.ops import gemm as G

    torch.manual_seed(1)
    M, N, K = 300, 520, 320
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    c = torch.randn(M, N, device="cuda")
    bias = torch.randn(N, device="cuda")
    ref = 0.5 * (a.float() @ b.float()) + 2.0 * c + bias
    out = G.gemm(a, b, b_mn=True, out_dtype=torch.float32, alpha=0.5, beta=2.0, c_in=c, bias=bias)
    assert _rel(out, ref) < 1e-3
    acc = c.clone()
    G.gemm(a, b, b_mn=True, out=acc, beta=1.0, c_in=acc)
    assert _rel(acc, a.float() @ b.float() + c) < 1e-3


def test_gemm_swiglu():
    from lyra_b200.ops import gemm as G
    from lyra_b200.ops.reference import swiglu

    torch.manual_seed(2)
    M, K, H = 260, 256, 384
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(K, 2 * H, device="cuda") / 16).bfloat16()
    ref = swiglu((x.float() @ w.float()).view(M, 2, H))
    out = G.gemm_swiglu(x, w)
    assert _rel(out, ref) < 1e-2


def _padded_layout(sizes, device):
    tile_group, offsets, row = [], [0], 0
    for g, n in enumerate(sizes):
        tiles = (n + 127) // 128
        tile_group += [g] * tiles
        row += tiles * 128
        offsets.append(row)
    tile_group.append(-1)  # one unused trailing tile
    return (torch.tensor(tile_group, dtype=torch.int32, device=device), torch.tensor(offsets, dtype=torch.int32, device=device), row + 128)


def test_grouped_gemm_and_wgrad():
    from lyra_b200.ops import gemm as G
    from lyra_b200.ops.reference import swiglu

    torch.manual_seed(3)
    sizes = [130, 0, 5, 256, 77]
    K, N = 192, 320
    tile_group, offsets, R = _padded_layout(sizes, "cuda")
    x = torch.zeros(R, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.zeros(R, N, device="cuda", dtype=torch.bfloat16)
    for g, n in enumerate(sizes):
        s = int(offsets[g])
        x[s:s + n] = torch.randn(n, K, device="cuda").bfloat16()
        dy[s:s + n] = torch.randn(n, N, device="cuda").bfloat16()
    w = (torch.randn(len(sizes), K, N, device="cuda") / 8).bfloat16()
    out = G.grouped_gemm(x, w, tile_group, out=torch.zeros(R, N, device="cuda", dtype=torch.bfloat16))
    sw = G.grouped_gemm(x, w, tile_group, swiglu=True, out=torch.zeros(R, N // 2, device="cuda", dtype=torch.bfloat16))
    dx = G.grouped_gemm(dy, w, tile_group, w_kmajor=True, out=torch.zeros(R, K, device="cuda", dtype=torch.bfloat16))
    dw = G.grouped_wgrad(x, dy, offsets, len(sizes))
    for g, n in enumerate(sizes):
        s = int(offsets[g])
        xs, ds = x[s:s + n].float(), dy[s:s + n].float()
        if n:
            assert _rel(out[s:s + n], xs @ w[g].float()) < 1e-2
            assert _rel(sw[s:s + n], swiglu((xs @ w[g].float()).view(n, 2, N // 2))) < 1e-2
            assert _rel(dx[s:s + n], ds @ w[g].float().t()) < 1e-2
            assert _rel(dw[g], xs.t() @ ds) < 1e-3
        else:
            assert dw[g].abs().max().item() == 0.0
    assert out[R - 128:].abs().max().item() == 0.0  # unused tile untouched


def test_batched_gemm():
    from lyra_b200.ops import gemm as G

    torch.manual_seed(4)
    g, m, n = 3, 192, 320
    x = torch.randn(g, m, n, device="cuda").bfloat16()
    a = G.batched_gemm(x, x)  # X X^T
    assert _rel(a, x.float() @ x.float().transpose(1, 2)) < 1e-2
    y = G.batched_gemm(a, x, b_mn=True, alpha=0.5, beta=2.0, c_in=x)  # 0.5 A X + 2 X
    assert _rel(y, 0.5 * (a.float() @ x.float()) + 2 * x.float()) < 1e-2


@pytest.mark.parametrize("shape", [(2, 1024, 1536), (1, 2048, 512), (3, 640, 640)])
def test_symmetric_products_skip_lower_tiles(shape):
    """X X^T and X^T X declared symmetric: upper-triangle tiles computed, lower ones mirrored; equals the full product."""
    from lyra_b200.ops import gemm as G, native

    Gn, m, n = shape
    torch.manual_seed(0)
    X = (torch.randn(Gn, m, n, device="cuda") / n ** 0.5).bfloat16()
    full = G.batched_gemm(X, X)
    sym = torch.full_like(full, float("nan"))
    G.batched_gemm(X, X, out=sym, symmetric=True)
    native.check_status()
    assert torch.isfinite(sym.float()).all()
    assert torch.equal(sym, sym.transpose(1, 2)) or (sym.float() - sym.float().transpose(1, 2)).abs().max().item() < 1e-2
    assert (sym.float() - full.float()).abs().max().item() < 2e-2
    full_t = G.batched_gemm(X, X, a_mn=True, b_mn=True)
    sym_t = torch.full_like(full_t, float("nan"))
    G.batched_gemm(X, X, a_mn=True, b_mn=True, out=sym_t, symmetric=True)
    assert (sym_t.float() - full_t.float()).abs().max().item() < 2e-2
    # B = c A A + b A with A symmetric
    A = sym.clone()
    ref = 0.5 * (A.float() @ A.float()) - 1.5 * A.float()
    B = torch.full_like(A, float("nan"))
    G.batched_gemm(A, A, out=B, alpha=0.5, beta=-1.5, c_in=A, symmetric=True)
    assert (B.float() - ref).abs().max().item() < 5e-2 * max(1.0, ref.abs().max().item())


def test_newton_schulz_gemm_matches_torch():
    from lyra_b200.training.optimizer_cuda import _ns_unnormalised, newtonschulz_gemm

    torch.manual_seed(1)
    for shape in [(2, 1024, 2048), (1, 2048, 1024)]:
        X = torch.randn(*shape, device="cuda")
        X = (X / (X.norm(dim=(1, 2), keepdim=True) * 1.01)).bfloat16()
        ref = _ns_unnormalised(X.float())
        got = newtonschulz_gemm(X.clone()).float()      # the iteration ping-pongs between its input buffer and a scratch one
        assert (got - ref).abs().max().item() < 0.05, (got - ref).abs().max().item()


@pytest.mark.parametrize("N", [512, 2880])
def test_grouped_gemm_scattered_epilogue(N):
    """The epilogue that stores result rows to per-row destinations (the expert-parallel return leg) on one GPU: the
    "peer" buffer is a local tensor, the row map a permutation with some rows dropped."""
    from lyra_b200.ops import gemm as G, native

    torch.manual_seed(3)
    R, K, E = 1024, 256, 4
    x = torch.randn(R, K, device="cuda").bfloat16()
    w = (torch.randn(E, K, N, device="cuda") / K ** 0.5).bfloat16()
    bias = torch.randn(E, N, device="cuda")
    tile_group = torch.tensor([0, 0, 1, 2, 2, 2, 3, -1], dtype=torch.int32, device="cuda")
    ref = G.grouped_gemm(x, w, tile_group, bias=bias, out=torch.zeros(R, N, dtype=torch.bfloat16, device="cuda"))
    perm = torch.randperm(R, device="cuda")
    row_dest = perm.to(torch.int32).clone()                 # rank 0 << 24 | slot
    dropped = torch.arange(R, device="cuda") % 7 == 3
    row_dest[dropped] = -1
    out = torch.full((R, N), 7.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm(x, w, tile_group, bias=bias, row_dest=row_dest, peer_out=[out.data_ptr()])
    torch.cuda.synchronize()
    native.check_status()
    live = (~dropped) & (torch.arange(R, device="cuda") < 7 * 128)       # the last tile belongs to no expert: nothing is stored
    assert torch.equal(out[perm[live]], ref[live])
    untouched = torch.ones(R, dtype=torch.bool, device="cuda")
    untouched[perm[live]] = False
    assert (out[untouched] == 7.0).all()
