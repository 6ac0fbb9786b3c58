"""Index arithmetic of the GEMM kernels restated in Python and checked exhaustively on small grids (no GPU): the
upper-triangle tile enumeration of symmetric products, the mirror condition of their epilogue, the grouped raster, and the
piece order of the all-gather fused GEMM."""

import pytest

BM, BN = 128, 256


def sym_decode(local: int, m_tiles: int, n_tiles: int) -> tuple[int, int]:
    """csrc/gemm/gemm.cu decode_tile, sym_upper branch."""
    m, acc = 0, 0
    while True:
        cnt = n_tiles - min(n_tiles, m * BM // BN)
        if local < acc + cnt or m + 1 >= m_tiles:
            break
        acc += cnt
        m += 1
    return m, m * BM // BN + (local - acc)


def sym_tiles(m_tiles: int, n_tiles: int) -> int:
    return sum(n_tiles - min(n_tiles, m * BM // BN) for m in range(m_tiles))


@pytest.mark.parametrize("n", [512, 640, 1024, 2880, 4096, 4224])
def test_symmetric_enumeration_and_mirror_cover_the_matrix_exactly(n):
    m_tiles, n_tiles = -(-n // BM), -(-n // BN)
    total = sym_tiles(m_tiles, n_tiles)
    seen = set()
    for local in range(total):
        m, nb = sym_decode(local, m_tiles, n_tiles)
        assert 0 <= m < m_tiles and 0 <= nb < n_tiles
        assert (m, nb) not in seen
        seen.add((m, nb))
        assert (nb + 1) * BN > m * BM                     # the tile reaches the diagonal or lies above it
    # every tile that is not enumerated lies wholly below the diagonal
    for m in range(m_tiles):
        for nb in range(n_tiles):
            if (m, nb) not in seen:
                assert (nb + 1) * BN <= m * BM
    # element coverage: direct stores of enumerated tiles + mirrored 32-column chunks reach every element exactly where needed
    covered = [[False] * n for _ in range(n)]
    for (m, nb) in seen:
        r0, c0 = m * BM, nb * BN
        for r in range(r0, min(r0 + BM, n)):
            for c in range(c0, min(c0 + BN, n)):
                covered[r][c] = True
        for chunk in range(BN // 32):
            col = c0 + chunk * 32
            if col >= n:
                continue
            if BN * (r0 // BN + 1) <= BM * (col // BM):   # the epilogue's mirror condition for this chunk
                for r in range(r0, min(r0 + BM, n)):
                    for c in range(col, min(col + 32, n)):
                        # the target tile must be one that was skipped: nobody else writes it
                        assert (c // BM, r // BN) not in seen
                        covered[c][r] = True
    step = max(1, n // 97)
    assert all(covered[r][c] for r in range(0, n, step) for c in range(n))
    assert all(covered[r][c] for r in range(n) for c in range(0, n, step))


@pytest.mark.parametrize("m_tiles,n_tiles,group", [(64, 48, 8), (13, 40, 8), (7, 33, 4), (64, 32, 16)])
def test_grouped_raster_is_a_permutation(m_tiles, n_tiles, group):
    seen = set()
    for local in range(m_tiles * n_tiles):
        band = group * n_tiles
        grp, within = divmod(local, band)
        gm = min(group, m_tiles - grp * group)
        n_blk = within // gm
        m_blk = grp * group + (within - n_blk * gm)
        assert 0 <= m_blk < m_tiles and 0 <= n_blk < n_tiles
        seen.add((m_blk, n_blk))
    assert len(seen) == m_tiles * n_tiles


@pytest.mark.parametrize("K,N,ctas", [(4096, 4096, 148), (6144, 12288, 148), (2880, 2880, 148), (128, 512, 148)])
def test_allgather_pieces_cover_b_once_and_in_panel_order(K, N, ctas):
    n_slabs, n_panels = -(-K // 64), -(-N // BN)
    per_panel = [0] * n_panels
    first_round_panels = set()
    for cta in range(ctas):
        piece = cta
        while piece < n_slabs * n_panels:
            panel, slab = divmod(piece, n_slabs)
            per_panel[panel] += 1
            if piece < ctas:
                first_round_panels.add(panel)
            piece += ctas
    assert per_panel == [n_slabs] * n_panels               # the producer waits for exactly this count (times the epoch)
    assert first_round_panels == set(range(max(first_round_panels) + 1))   # the first wave of pieces fills the leading panels
