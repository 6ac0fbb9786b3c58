"""Python face of the tcgen05 GEMM family (``csrc/gemm/gemm.cu``).

Operands are described by how they are *stored*: a K-major operand is ``[rows, K]``, an MN-major
operand is ``[K, rows]``. With weights kept in the reference's ``[in, out]`` layout
(lyra/model.py:252-274) the three products of a linear layer need no transposes:

* forward  ``y = x @ W``        -> A = x (K-major),  B = W (MN-major)
* dgrad    ``dx = dy @ W^T``    -> A = dy (K-major), B = W (K-major)
* wgrad    ``dW = x^T @ dy``    -> A = x (MN-major), B = dy (MN-major)
"""

from __future__ import annotations

import torch

from lyra_b200.ops import native
from lyra_b200.ops.native import c_float, c_int, c_ll, c_void_p, ptr

GROUP_NONE, GROUP_M, GROUP_K, GROUP_BATCH = 0, 1, 2, 3
EPI_STORE, EPI_SWIGLU = 0, 1
TILE_M = 128


def _raw(
    a, lda, a_gs, a_mn, b, ldb, b_gs, b_mn, c, c_in, ldc, c_gs, out_fp32, M, N, K, alpha, beta, bias, bias_gs,
    group_mode, num_groups, tile_group, group_offsets, total_rows, epilogue, n_split, swiglu_beta, swiglu_limit, sym_upper=False, row_dest=None, peer_out=None,
    row_scale=None, peer_count=None, tile_perm=None, arrive=None, expect=None,
):
    import ctypes

    lib = native.kernels()
    fn = lib.lyra_gemm_bf16
    fn.restype = c_int
    peers = (ctypes.c_longlong * len(peer_out))(*peer_out) if peer_out else None
    counters = (ctypes.c_longlong * len(peer_count))(*peer_count) if peer_count else None
    rc = fn(
        ptr(a), c_ll(lda), c_ll(a_gs), c_int(int(a_mn)),
        ptr(b), c_ll(ldb), c_ll(b_gs), c_int(int(b_mn)),
        ptr(c), ptr(c_in), c_ll(ldc), c_ll(c_gs), c_int(int(out_fp32)),
        c_int(M), c_int(N), c_int(K), c_float(alpha), c_float(beta),
        ptr(bias), c_ll(bias_gs),
        c_int(group_mode), c_int(num_groups), ptr(tile_group), ptr(group_offsets), c_int(total_rows),
        c_int(epilogue), c_int(n_split), c_float(swiglu_beta), c_float(swiglu_limit), c_int(int(sym_upper)),
        ptr(row_dest), peers, c_int(len(peer_out) if peer_out else 0),
        ptr(row_scale), counters, ptr(tile_perm), ptr(arrive), ptr(expect),
        ptr(native.status_word()), native.stream_ptr(),
    )
    native.check(rc, "lyra_gemm_bf16")
    native.count_launch()


def _check2d(t: torch.Tensor) -> None:
    assert t.dtype == torch.bfloat16 and t.is_cuda and t.stride(-1) == 1, (t.dtype, t.device, t.stride())
    assert t.data_ptr() % 16 == 0


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    alpha: float = 1.0,
    beta: float = 0.0,
    c_in: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out = alpha * A @ B^T + beta * c_in (+ bias)`` with 2-D bf16 operands (see module docstring)."""
    _check2d(a)
    _check2d(b)
    K, M = a.shape if a_mn else a.shape[::-1]
    Kb, N = b.shape if b_mn else b.shape[::-1]
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if c_in is not None:
        assert c_in.dtype == out.dtype and c_in.stride() == out.stride()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _raw(a, a.stride(0), 0, a_mn, b, b.stride(0), 0, b_mn, out, c_in, out.stride(0), 0, out.dtype == torch.float32,
         M, N, K, alpha, beta, bias, 0, GROUP_NONE, 1, None, None, 0, EPI_STORE, 0, 0.0, 0.0)
    return out


def gemm_swiglu(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None, swiglu_beta: float = 1.702,
                swiglu_limit: float = 7.0) -> torch.Tensor:
    """``swiglu(x @ W)`` with ``W`` stored ``[K, 2H]`` (gate columns then linear columns) -> ``[M, H]``."""
    _check2d(x)
    _check2d(w)
    M, K = x.shape
    H = w.shape[1] // 2
    out = torch.empty(M, H, dtype=torch.bfloat16, device=x.device)
    _raw(x, x.stride(0), 0, False, w, w.stride(0), 0, True, out, None, out.stride(0), 0, False, M, 2 * H, K, 1.0, 0.0,
         bias, 0, GROUP_NONE, 1, None, None, 0, EPI_SWIGLU, H, swiglu_beta, swiglu_limit)
    return out


def batched_gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn=False, b_mn=False, out=None, alpha=1.0, beta=0.0, c_in=None,
                 symmetric: bool = False) -> torch.Tensor:
    """Stacked independent products, ``a``/``b`` are ``[G, rows, cols]`` bf16 with the per-matrix meaning of ``gemm``.

    ``symmetric=True`` declares the result symmetric (``X X^T``, ``X^T X``, ``A A`` with ``A`` symmetric, and ``c_in``
    symmetric too): the tiles wholly below the diagonal (47 % of them at 4096 x 4096) are not computed but mirrored from the
    upper triangle (by the epilogue of the upper tiles for bf16 results, by a second kernel for fp32 ones)."""
    G = a.shape[0]
    K, M = a.shape[1:] if a_mn else a.shape[1:][::-1]
    Kb, N = b.shape[1:] if b_mn else b.shape[1:][::-1]
    assert K == Kb and b.shape[0] == G
    if out is None:
        out = torch.empty(G, M, N, dtype=torch.bfloat16, device=a.device)
    _raw(a, a.stride(1), a.stride(0), a_mn, b, b.stride(1), b.stride(0), b_mn, out, c_in, out.stride(1), out.stride(0),
         out.dtype == torch.float32, M, N, K, alpha, beta, None, 0, GROUP_BATCH, G, None, None, 0, EPI_STORE, 0, 0.0, 0.0,
         sym_upper=symmetric and M == N and M >= 512)
    if symmetric and M == N and M >= 512 and out.dtype == torch.float32:   # bf16 results are mirrored inside the GEMM epilogue
        lib = native.kernels()
        native.check(lib.lyra_symmetrize(ptr(out), c_ll(out.stride(1)), c_ll(out.stride(0)), c_int(M), c_int(G), c_int(int(out.dtype == torch.float32)),
                                         native.stream_ptr()), "lyra_symmetrize")
        native.count_launch()
    return out


def grouped_gemm(
    x: torch.Tensor,
    w: torch.Tensor,
    tile_group: torch.Tensor,
    *,
    w_kmajor: bool = False,
    bias: torch.Tensor | None = None,
    swiglu: bool = False,
    swiglu_beta: float = 1.702,
    swiglu_limit: float = 7.0,
    out: torch.Tensor | None = None,
    row_dest: torch.Tensor | None = None,
    peer_out: list[int] | None = None,
    row_scale: torch.Tensor | None = None,
    peer_count: list[int] | None = None,
    tile_perm: torch.Tensor | None = None,
    arrive: torch.Tensor | None = None,
    expect: torch.Tensor | None = None,
) -> torch.Tensor | None:
    """Ragged grouped GEMM over rows sorted by group and padded so every 128-row tile has one group.

    With ``row_dest [R]`` (int32: ``rank << 24 | row``, negative = drop the row) and ``peer_out`` (one peer-mapped buffer
    address per rank, rows of ``N`` bf16) the epilogue stores every result row straight into that rank's buffer over
    NVLink instead of a local output: the return leg of the expert-parallel exchange fused into the product.

    Scattered mode extras: ``row_scale [R]`` fp32 multiplies each stored row (after the bias) - the routing score, so that the
    source rank's combine is a plain K-way sum; ``peer_count`` (one address per rank of an int32 counter in that rank's memory)
    makes every output tile add the number of rows it stored on a rank to that rank's counter, which the rank waits on
    (``lyra_wait_arrivals``) instead of an all-rank barrier.

    Tile-granular input (``arrive`` / ``expect`` int32 ``[R/128]``): other GPUs are still storing the rows of ``x`` while the
    kernel runs; the TMA producer waits until ``arrive[t] - expect[t] >= 0`` before it first reads 128-row tile ``t``.
    ``tile_perm [R/128]`` int32 lists the used tiles in the order in which they should be visited (-1 ends the list).

    ``x [R, K]``; ``tile_group [R/128]`` int32 (-1 marks unused tiles, whose output rows are left untouched);
    ``w [G, K, N]`` (forward, MN-major) or, with ``w_kmajor``, ``w [G, N, K]`` (data gradient of an ``[in, out]`` weight).
    """
    _check2d(x)
    R, K = x.shape
    assert R % TILE_M == 0 and tile_group.numel() == R // TILE_M and tile_group.dtype == torch.int32
    G = w.shape[0]
    if w_kmajor:
        N, Kw = w.shape[1], w.shape[2]
    else:
        Kw, N = w.shape[1], w.shape[2]
    assert Kw == K
    n_out = N // 2 if swiglu else N
    for t in (tile_perm, arrive, expect):
        assert t is None or (t.dtype == torch.int32 and t.numel() >= R // TILE_M and t.is_contiguous())
    waits = dict(tile_perm=tile_perm, arrive=arrive, expect=expect)
    if row_dest is not None:
        assert not swiglu and peer_out and row_dest.dtype == torch.int32 and row_dest.numel() >= R
        assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() >= R)
        assert peer_count is None or len(peer_count) == len(peer_out)
        _raw(x, x.stride(0), 0, False, w, w.stride(1), w.stride(0), not w_kmajor, x, None, N, 0, False,
             R, N, K, 1.0, 0.0, bias, (bias.stride(0) if bias is not None else 0), GROUP_M, G, tile_group, None, 0,
             EPI_STORE, 0, swiglu_beta, swiglu_limit, row_dest=row_dest, peer_out=peer_out, row_scale=row_scale, peer_count=peer_count, **waits)
        return None
    if out is None:
        out = torch.empty(R, n_out, dtype=torch.bfloat16, device=x.device)
    _raw(x, x.stride(0), 0, False, w, w.stride(1), w.stride(0), not w_kmajor, out, None, out.stride(0), 0, False,
         R, N, K, 1.0, 0.0, bias, (bias.stride(0) if bias is not None else 0), GROUP_M, G, tile_group, None, 0,
         EPI_SWIGLU if swiglu else EPI_STORE, N // 2 if swiglu else 0, swiglu_beta, swiglu_limit, **waits)
    return out


def grouped_wgrad(x: torch.Tensor, dy: torch.Tensor, group_offsets: torch.Tensor, num_groups: int, *,
                  out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Per-group weight gradient ``dW[g] = x[rows_g]^T @ dy[rows_g]`` -> fp32 ``[G, K, N]``.

    ``group_offsets [G+1]`` int32 padded row offsets (multiples of 128); pad rows of ``x`` must be zero.
    """
    _check2d(x)
    _check2d(dy)
    R, K = x.shape
    N = dy.shape[1]
    if out is None:
        out = torch.empty(num_groups, K, N, dtype=torch.float32, device=x.device)
        accumulate = False
    _raw(x, x.stride(0), 0, True, dy, dy.stride(0), 0, True, out, out if accumulate else None, out.stride(1), out.stride(0),
         out.dtype == torch.float32, K, N, 0, 1.0, 1.0, None, 0, GROUP_K, num_groups, None, group_offsets, R,
         EPI_STORE, 0, 0.0, 0.0)
    return out


def gemm_allgather(x: torch.Tensor, w_local: torch.Tensor, src_ptrs: list[int], my_rank: int, rows_per_rank: int, flags: torch.Tensor, epoch: int, *,
                   alpha: float = 1.0, beta: float = 0.0, c_in: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """``x [M, K] @ W [K, N]`` where the rows of ``W`` live in peer GPUs' memory: the all-gather is fused into the GEMM.

    ``w_local [K, N]`` is this rank's full-size bf16 buffer, filled by the kernel one 256-column panel after the other
    while the tensor cores already work on the panels that have landed; ``src_ptrs[r]`` is the peer-mapped address of rank r's rows
    (``rows_per_rank`` each; a single owner is ``rows_per_rank = K`` with the owner's address in slot 0). ``flags`` is an
    int32 tensor with at least ``ceil(N / 256)`` entries, zero before the first call; ``epoch`` is the number of this call on
    those flags (1, 2, ...), always with the same ``K`` and ``N``.
    After the call ``w_local`` holds the whole matrix and can be used by ordinary GEMMs."""
    import ctypes

    _check2d(x)
    M, K = x.shape
    Kw, N = w_local.shape
    assert K == Kw and w_local.dtype == torch.bfloat16 and w_local.stride(1) == 1
    assert flags.dtype == torch.int32 and flags.numel() >= (N + 255) // 256
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    lib = native.kernels()
    fn = lib.lyra_gemm_allgather_bf16
    fn.restype = c_int
    arr = (ctypes.c_longlong * len(src_ptrs))(*src_ptrs)
    rc = fn(ptr(x), c_ll(x.stride(0)), ptr(w_local), c_ll(w_local.stride(0)), arr, c_int(len(src_ptrs)), c_int(my_rank), c_int(rows_per_rank),
            ptr(out), ptr(c_in), c_ll(out.stride(0)), c_int(M), c_int(N), c_int(K), c_float(alpha), c_float(beta), ptr(bias), ptr(flags), c_int(epoch),
            ptr(native.status_word()), native.stream_ptr())
    native.check(rc, "lyra_gemm_allgather_bf16")
    native.count_launch()
    return out
