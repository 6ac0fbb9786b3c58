"""Index arithmetic of the GEMM kernels restated in Python and checked exhaustively on small grids (no GPU): the
upper-triangle tile enumeration of symmetric products, the mirror condition of their epilogue, the grouped raster, and the
piece order of the all-gather fused GEMM."""

import numpy as np
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


# ---------------------------------------------------------------------------------------------------------------------
# Layout arithmetic of the tile-granular expert exchange (csrc/comm/comm.cu: ep_layout_tiles_kernel,
# ep_dispatch_sorted_kernel), restated for every rank of a small world and checked against each other: what the senders
# compute as destination rows must tile the receivers' buffers exactly, and the receivers' expectations must equal what arrives.
def ep_layout(counts, world, rank, e_local, cap_rows):
    """The receiver / sender side tables of one rank. ``counts[s][e]``: rows rank ``s`` routes to expert ``e``."""
    E = world * e_local
    total = [sum(counts[s][e] for s in range(world)) for e in range(E)]
    base, offsets = [0] * E, []
    for d in range(world):
        off = 0
        for j in range(e_local):
            e = d * e_local + j
            base[e] = off
            if d == rank:
                offsets.append(min(off, cap_rows))
            off += (total[e] + 127) // 128 * 128
        if d == rank:
            offsets.append(min(off, cap_rows))
    send_base = [base[e] + sum(counts[s][e] for s in range(rank)) for e in range(E)]
    starts = [sum(counts[rank][:e]) for e in range(E + 1)]
    send_starts, run = [], 0
    for k in range(E):
        j, t = divmod(k, world)
        send_starts.append(run)
        run += counts[rank][((rank + t) % world) * e_local + j]
    send_starts.append(run)
    n_tiles = cap_rows // 128
    group, valid, key = [-1] * n_tiles, [0] * n_tiles, [-1] * n_tiles
    for t in range(n_tiles):
        row = t * 128
        g = next((j for j in range(e_local) if offsets[j] <= row < offsets[j + 1]), -1) if row < offsets[e_local] else -1
        if g >= 0:
            e = rank * e_local + g
            r0 = row - offsets[g]
            r1 = min(r0 + 128, total[e])
            lo, step = 0, -1
            for s in range(world):
                c = counts[s][e]
                if c > 0 and lo < r1 and lo + c > r0:
                    step = max(step, (rank - s + world) % world)
                lo += c
            group[t], valid[t], key[t] = g, max(r1 - r0, 0), g * world + step
    perm = [t for k in range(e_local * world) for t in range(n_tiles) if valid[t] > 0 and key[t] == k]
    return dict(offsets=offsets, send_base=send_base, starts=starts, send_starts=send_starts, group=group, valid=valid, perm=perm)


def ep_send_sequence(lay, world, rank, e_local):
    """(destination rank, destination row) of every block of ep_dispatch_sorted_kernel, in launch order."""
    E = world * e_local
    out = []
    for i in range(lay["send_starts"][E]):
        k = max(k for k in range(E) if lay["send_starts"][k] <= i)
        j, t = divmod(k, world)
        d = (rank + t) % world
        e = d * e_local + j
        out.append((d, lay["send_base"][e] + i - lay["send_starts"][k], j))
    return out


@pytest.mark.parametrize("world, e_local, seed", [(2, 2, 0), (4, 2, 1), (4, 4, 2), (8, 1, 3), (8, 4, 4), (3, 2, 5)])
def test_exchange_layout_senders_and_receivers_agree(world, e_local, seed):
    import random

    rng = random.Random(seed)
    E = world * e_local
    counts = [[rng.choice([0, 0, 1, 5, 130, 260, 77]) for _ in range(E)] for _ in range(world)]
    cap = (max(sum(counts[s][e] for s in range(world)) for e in range(E)) // 128 + 2) * 128 * e_local
    lays = [ep_layout(counts, world, r, e_local, cap) for r in range(world)]
    landed = [dict() for _ in range(world)]                 # per destination: row -> (source, local expert)
    for s in range(world):
        seq = ep_send_sequence(lays[s], world, s, e_local)
        assert len(seq) == sum(counts[s])
        assert [j for _, _, j in seq] == sorted(j for _, _, j in seq)          # all of local expert 0 first, then 1, ...
        for d, row, j in seq:
            assert row not in landed[d], "two assignments were given the same row"
            landed[d][row] = (s, j)
    for d in range(world):
        lay = lays[d]
        per_tile = [0] * len(lay["valid"])
        for row, (s, j) in landed[d].items():
            assert lay["offsets"][j] <= row < lay["offsets"][j + 1]            # inside its expert's (padded) range
            per_tile[row // 128] += 1
        assert per_tile == lay["valid"]                                        # the receiver expects exactly what arrives, tile by tile
        used = [t for t, v in enumerate(lay["valid"]) if v > 0]
        assert sorted(lay["perm"]) == used
        assert [lay["group"][t] for t in lay["perm"]] == sorted(lay["group"][t] for t in lay["perm"])   # visited expert by expert
        # inside an expert: rows are source-major, every source's rows contiguous and in source order
        for j in range(e_local):
            rows = sorted(r for r, (s, jj) in landed[d].items() if jj == j)
            assert [landed[d][r][0] for r in rows] == sorted(landed[d][r][0] for r in rows)
            assert rows == list(range(lay["offsets"][j], lay["offsets"][j] + len(rows)))


# ---------------------------------------------------------------------------------------------------------------------
# Persistent flash-attention forward (csrc/attn/flash_fwd.cu): the work items of a launch and how the CTAs share them.
def fwd_item(idx, n_qt, Nq, B, T, S, window, q_start):
    """Restates ``item_at``: (q0, head, b, first key tile, key tiles) of item ``idx``; late query tiles come first."""
    per_qt = Nq * B
    q0 = (n_qt - 1 - idx // per_qt) * 128
    rest = idx % per_qt
    qlo = q_start + q0
    qhi = min(q_start + min(q0 + 128, T) - 1, S - 1)
    klo = max(0, qlo - window + 1) if window > 0 else 0
    jt_begin = klo // 128
    jt_end = jt_begin if qhi < 0 else qhi // 128 + 1
    return q0, rest % Nq, rest // Nq, jt_begin, max(jt_end - jt_begin, 0)


def fwd_schedule(grid, n_items):
    """Items of every CTA in the order it takes them (serpentine over the rounds)."""
    out = [[] for _ in range(grid)]
    for cta in range(grid):
        r = 0
        while True:
            idx = r * grid + (grid - 1 - cta if r & 1 else cta)
            if idx >= n_items:
                break
            out[cta].append(idx)
            r += 1
    return out


@pytest.mark.parametrize("T,S,window,q_start,Nq,B,grid", [(4096, 4096, 0, 0, 32, 2, 148), (4096, 4096, 128, 0, 16, 4, 148), (1000, 1000, 0, 0, 4, 2, 148),
                                                       (128, 512, 128, 384, 4, 1, 4), (300, 300, 0, 0, 3, 1, 7), (4096, 4096, 0, 0, 32, 2, 1)])
def test_forward_items_are_visited_once_and_the_serpentine_balances_them(T, S, window, q_start, Nq, B, grid):
    n_qt = (T + 127) // 128
    n_items = n_qt * Nq * B
    grid = min(grid, n_items)
    sched = fwd_schedule(grid, n_items)
    seen = sorted(i for items in sched for i in items)
    assert seen == list(range(n_items))                                  # every item exactly once
    cover = set()
    for idx in range(n_items):
        q0, head, b, jt_begin, n_tiles = fwd_item(idx, n_qt, Nq, B, T, S, window, q_start)
        cover.add((q0, head, b))
        # the tiles are exactly those that intersect the band of the tile's queries
        qs = range(q_start + q0, q_start + min(q0 + 128, T))
        want = {k // 128 for q in qs for k in range(max(0, q - window + 1) if window else 0, min(q, S - 1) + 1)}
        assert set(range(jt_begin, jt_begin + n_tiles)) == want
    assert len(cover) == n_items
    work = [sum(fwd_item(i, n_qt, Nq, B, T, S, window, q_start)[4] for i in items) for items in sched]
    if grid == 148 and window == 0 and T == 4096:                         # the benchmark shape: CTAs finish within a few tiles of each other
        assert max(work) - min(work) <= 0.06 * max(work), (min(work), max(work))


# ---------------------------------------------------------------------------------------------------------------------
# e4m3 decode GEMM (csrc/gemm/decode_gemm.cu): the (group, block of token rows) units every CTA lists for itself.
def f8_units(offsets, counts, G, ntok, max_units=1024):
    """Restates the warp scan: lane l owns ``per`` consecutive groups; units are numbered by an exclusive scan over the lanes."""
    per = (G + 31) // 32
    mine = []
    for lane in range(32):
        n = 0
        for g in range(lane * per, min(G, (lane + 1) * per)):
            beg = offsets[g]
            end = beg + counts[g] if counts is not None else offsets[g + 1]
            n += (max(end - beg, 0) + ntok - 1) // ntok
        mine.append(n)
    units = {}
    for lane in range(32):
        at = sum(mine[:lane])
        for g in range(lane * per, min(G, (lane + 1) * per)):
            beg = offsets[g]
            end = beg + counts[g] if counts is not None else offsets[g + 1]
            r0 = beg
            while r0 < end and at < max_units:
                units[at] = (g, r0, min(ntok, end - r0))
                r0 += ntok
                at += 1
    return [units[i] for i in range(min(sum(mine), max_units))]


@pytest.mark.parametrize("G,ntok,seed", [(128, 16, 0), (32, 16, 1), (33, 32, 2), (1, 64, 3), (200, 16, 4), (64, 64, 5)])
def test_decode_gemm_units_cover_every_row_once_and_passes_are_balanced(G, ntok, seed):
    rng = np.random.default_rng(seed)
    real = np.where(rng.random(G) < 0.25, rng.integers(1, 3 * ntok, G), 0)            # most groups empty, some longer than a block
    padded = (real + 127) // 128 * 128 if seed % 2 else real                            # receive buffers pad every group to 128 rows
    offsets = np.concatenate([[0], np.cumsum(padded)]).astype(int)
    units = f8_units(offsets, real if seed % 2 else None, G, ntok)
    rows = [r for g, r0, cnt in units for r in range(r0, r0 + cnt)]
    want = [r for g in range(G) for r in range(offsets[g], offsets[g] + real[g])]
    assert rows == want                                                                # every real row once, in order; no empty unit
    assert all(1 <= cnt <= ntok for _, _, cnt in units)
    n_panels, splits, grid = 45, 1, 296
    n_passes = n_panels * len(units) * splits
    per_cta = [len(range(c, n_passes, grid)) for c in range(min(grid, max(n_passes, 1)))]
    assert max(per_cta) - min(per_cta) <= 1                                            # equal-cost passes dealt round-robin
