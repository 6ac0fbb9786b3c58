"""Host-side model of the expert-parallel exchange protocol (flags written by peers, epochs in per-rank device counters).

Each rank runs, per MoE layer call, the stream-ordered sequence of parallel/ep.py:

    push counts (+ flag64)   -> wait flag64     -> read counts
    dispatch rows to peers   -> signal flag128  -> wait flag128 -> expert GEMMs read the receive buffer
    return rows to peers     -> signal flag192  -> wait flag192 -> combine reads the return buffer

Ranks advance in a random interleaving (any rank that is not blocked may take its next step). The model checks what the
design relies on when ONE set of buffers serves every layer (inference): no deadlock, and no rank ever overwrites a peer's
counts / receive / return buffer while that peer has not yet consumed the previous exchange's contents. The counts live in
two slabs used by call parity, and an inference call reads its slab in place until its return kernel (no private copy), so
the slab of call n must survive until call n's last step while call n + 1 already uses the other one."""

import random

import pytest

STEPS = ["push_counts", "wait64", "read_counts", "dispatch", "signal128", "wait128", "gemm_reads_recv",
         "return", "signal192", "wait192", "combine_reads_ret"]
COUNT_SLABS = 2


class Rank:
    def __init__(self, r, world):
        self.r, self.world = r, world
        self.ctr = {64: 0, 128: 0, 192: 0}                 # device counters (epoch of the last signal sent)
        self.flags = {o: [0] * world for o in (64, 128, 192)}   # written by peers
        self.pc, self.call = 0, 0
        # generation (call index) of the data currently held in each buffer, per writer
        self.counts_gen = [[-1] * world for _ in range(COUNT_SLABS)]   # per slab (call parity), per writer
        self.recv_gen = [-1] * world
        self.ret_gen = [-1] * world
        self.consumed = {"counts": -1, "recv": -1, "ret": -1}   # last call whose contents this rank has finished reading


def run(world, calls, seed):
    rng = random.Random(seed)
    ranks = [Rank(r, world) for r in range(world)]
    done = 0
    guard = 0
    while done < world:
        guard += 1
        assert guard < 200000, "no progress: deadlock"
        rk = rng.choice([x for x in ranks if x.call < calls])
        step = STEPS[rk.pc]
        n = rk.call
        if step in ("wait64", "wait128", "wait192"):
            off = int(step[4:])
            if min(rk.flags[off]) < rk.ctr[off]:
                continue                                    # blocked: somebody has not signalled this epoch yet
        elif step == "push_counts":
            rk.ctr[64] += 1
            for p in ranks:
                # the slab being written last held call n - COUNT_SLABS, whose owner reads it until its return kernel
                assert p.consumed["counts"] >= n - COUNT_SLABS, f"rank {rk.r} overwrites counts of rank {p.r} still read by call {n - COUNT_SLABS}"
                p.counts_gen[n % COUNT_SLABS][rk.r] = n
                p.flags[64][rk.r] = rk.ctr[64]
        elif step == "read_counts":
            assert rk.counts_gen[n % COUNT_SLABS] == [n] * world
        elif step == "dispatch":
            for p in ranks:
                assert p.consumed["recv"] >= n - 1, f"rank {rk.r} overwrites receive buffer of rank {p.r} still in use by call {n - 1}"
                p.recv_gen[rk.r] = n
        elif step in ("signal128", "signal192"):
            off = int(step[6:])
            rk.ctr[off] += 1
            for p in ranks:
                p.flags[off][rk.r] = rk.ctr[off]
        elif step == "gemm_reads_recv":
            assert rk.recv_gen == [n] * world
            rk.consumed["recv"] = n
        elif step == "return":
            assert rk.counts_gen[n % COUNT_SLABS] == [n] * world     # the return kernel reads the counts in place: still this call's
            rk.consumed["counts"] = n
            for p in ranks:
                assert p.consumed["ret"] >= n - 1, f"rank {rk.r} overwrites return buffer of rank {p.r} still in use by call {n - 1}"
                p.ret_gen[rk.r] = n
        elif step == "combine_reads_ret":
            assert rk.ret_gen == [n] * world
            rk.consumed["ret"] = n
        rk.pc += 1
        if rk.pc == len(STEPS):
            rk.pc, rk.call = 0, rk.call + 1
            if rk.call == calls:
                done += 1
    return ranks


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_protocol_is_deadlock_free_and_never_overwrites_live_buffers(world):
    for seed in range(40):
        ranks = run(world, calls=6, seed=seed)
        assert all(r.ctr == {64: 6, 128: 6, 192: 6} for r in ranks)


def test_model_detects_a_missing_barrier():
    """Sanity of the model itself: without the return-phase wait a fast rank's next dispatch does hit a live receive buffer."""
    global STEPS
    saved = list(STEPS)
    try:
        STEPS = [s for s in saved if s not in ("wait192", "wait128")]
        with pytest.raises(AssertionError):
            for seed in range(200):
                run(4, calls=6, seed=seed)
    finally:
        STEPS = saved


def test_in_place_counts_reads_are_ordered_by_the_return_phase_even_with_one_slab():
    """The margin of the inference path: a call reads its counts slab in place until its return kernel, and every peer's next
    push waits (through the return phase) for that kernel, so even a single slab would never be overwritten while read."""
    global COUNT_SLABS
    try:
        COUNT_SLABS = 1
        for seed in range(60):
            run(4, calls=6, seed=seed)
    finally:
        COUNT_SLABS = 2


# ======================================================================================================================
# Tile-granular protocol (training path of parallel/ep.py): no phase barrier after the dispatch or the return.
#
#   forward of MoE layer l:
#     push counts (+ flag64) -> wait flag64 -> layout; expect_f[src] += rows(src)
#     store rows into every destination's layer-l receive buffer; each store bumps that rank's arrival counter of the tile
#     (modelled per source); grouped GEMM: a tile is read only once  arrive - expect >= 0  for it
#     down-projection epilogue stores result rows into the source rank's layer-l return buffer and bumps its "returned" counter
#     [shared expert] -> wait until returned - expected >= 0 -> combine reads the return buffer
#   backward of layer l (layers in reverse order, after all forwards of the microbatch):
#     combine-backward reads the layer-l return buffer; wait "scratch free" flags; expect_b += rows; store gradient rows into the
#     destinations' ONE receive scratch (shared by all layers); GEMMs read the scratch and the layer-l receive buffer; the
#     dgrad epilogue stores rows into the sources' ONE return scratch and bumps "returned_b"; signal "scratch free";
#     [shared expert backward] -> wait returned_b -> gather reads the return scratch
#
# A pair (source, destination) may exchange no rows at all in a call (random routing); then nothing orders the two ranks
# through data, which is the case the "scratch free" flag exists for.


class TRank:
    def __init__(self, r, world, layers):
        self.r, self.world = r, world
        self.pc = 0
        self.ctr64, self.flags64 = 0, [0] * world
        self.ctr_free, self.flags_free = 0, [0] * world
        self.counts_gen, self.counts_read = [[-1] * world, [-1] * world], -1   # two counts slabs, used by call parity
        self.arrive = {"f": [0] * world, "b": [0] * world}        # bumped by the sources' stores (cumulative, shared by all layers)
        self.expect = {"f": [0] * world, "b": [0] * world}        # this rank's running totals
        self.returned = {"f": 0, "b": 0}
        self.ret_expect = {"f": 0, "b": 0}
        # buffers: per layer for the forward (kept for the backward), one scratch for the backward; (generation per source, last generation read)
        self.recv = {("f", l): [[-1] * world, -1] for l in range(layers)} | {"b": [[-1] * world, -1]}
        self.ret = {("f", l): [[-1] * world, -1] for l in range(layers)} | {"b": [[-1] * world, -1]}


def _program(world, layers, microbatches, free_wait):
    """The stream-ordered list of steps every rank executes: (kind, way, layer, generation, call, k)."""
    prog = []
    q = 0                                                     # running number of backward exchanges (generation of the scratch buffers)
    for m in range(microbatches):
        for l in range(layers):
            n = m * layers + l
            prog += [("push", n), ("wait64", n), ("layout", n)]
            prog += [("send", "f", ("f", l), m, n, k) for k in range(world)]
            prog += [("tile", "f", ("f", l), m, n, k) for k in range(world)]
            prog += [("ret", "f", ("f", l), m, n, k) for k in range(world)]
            prog += [("wait_ret", "f", ("f", l), m, n)]
        for l in reversed(range(layers)):
            n = m * layers + l
            prog += [("read_ret_done", ("f", l), m)]           # combine-backward was the last reader of the layer's return buffer
            if free_wait:
                prog += [("wait_free",)]
            prog += [("bump_b", n)]
            prog += [("send", "b", "b", q, n, k) for k in range(world)]
            prog += [("tile", "b", "b", q, n, k) for k in range(world)]
            prog += [("recv_done", ("f", l), m), ("recv_done", "b", q)]
            prog += [("ret", "b", "b", q, n, k) for k in range(world)]
            prog += [("signal_free",), ("wait_ret", "b", "b", q, n), ("read_ret_done", "b", q)]
            q += 1
    return prog


def run_tiles(world, seed, layers=3, microbatches=2, density=0.6, free_wait=True):
    rng = random.Random(seed)
    prog = _program(world, layers, microbatches, free_wait)
    ranks = [TRank(r, world, layers) for r in range(world)]
    calls = layers * microbatches
    rows = [[[rng.random() < density for _ in range(world)] for _ in range(world)] for _ in range(calls)]   # rows[n][s][d]
    guard = 0
    while any(x.pc < len(prog) for x in ranks):
        guard += 1
        assert guard < 2000000, "no progress: deadlock"
        rk = rng.choice([x for x in ranks if x.pc < len(prog)])
        r, st = rk.r, prog[rk.pc]
        kind = st[0]
        if kind == "push":
            n = st[1]
            rk.ctr64 += 1
            for p in ranks:
                # without the phase barriers a rank may be a whole call ahead of a peer it exchanged no rows with: two slabs are needed
                assert p.counts_read >= n - 2, "counts slab overwritten before its previous contents were read"
                p.counts_gen[n & 1][r] = n
                p.flags64[r] = rk.ctr64
        elif kind == "wait64":
            if min(rk.flags64) < rk.ctr64:
                continue
        elif kind == "layout":
            n = st[1]
            assert rk.counts_gen[n & 1] == [n] * world
            rk.counts_read = n
            for s in range(world):
                rk.expect["f"][s] += int(rows[n][s][r])
        elif kind == "bump_b":
            for s in range(world):
                rk.expect["b"][s] += int(rows[st[1]][s][r])
        elif kind == "send":
            _, way, buf, gen, n, k = st
            d = (r + k) % world
            if rows[n][r][d]:
                slot = ranks[d].recv[buf]
                assert slot[1] >= gen - 1, f"rank {r} stores into receive buffer {buf} of rank {d}, which still reads generation {gen - 1}"
                slot[0][r] = gen
                ranks[d].arrive[way][r] += 1
        elif kind == "tile":
            _, way, buf, gen, n, k = st
            s = (r - k) % world
            if rows[n][s][r]:
                if rk.arrive[way][s] - rk.expect[way][s] < 0:
                    continue                                 # the GEMM's producer spins on this tile
                assert rk.recv[buf][0][s] == gen, "a tile was released before this call's rows landed in it"
        elif kind == "recv_done":
            rk.recv[st[1]][1] = st[2]
        elif kind == "ret":
            _, way, buf, gen, n, k = st
            s = (r + k) % world
            if rows[n][s][r]:
                slot = ranks[s].ret[buf]
                assert slot[1] >= gen - 1, f"rank {r} returns rows into buffer {buf} of rank {s}, which still reads generation {gen - 1}"
                slot[0][r] = gen
                ranks[s].returned[way] += 1
        elif kind == "wait_ret":
            _, way, buf, gen, n = st
            want = rk.ret_expect[way] + sum(rows[n][r])
            if rk.returned[way] - want < 0:
                continue
            rk.ret_expect[way] = want
            assert all(rk.ret[buf][0][d] == gen for d in range(world) if rows[n][r][d])
        elif kind == "read_ret_done":
            rk.ret[st[1]][1] = st[2]
        elif kind == "wait_free":
            if min(rk.flags_free) < rk.ctr_free:
                continue
        elif kind == "signal_free":
            rk.ctr_free += 1
            for p in ranks:
                p.flags_free[r] = rk.ctr_free
        rk.pc += 1
    return ranks


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tile_protocol_is_deadlock_free_and_never_overwrites_live_buffers(world):
    for seed in range(25):
        for density in (1.0, 0.5, 0.15):
            ranks = run_tiles(world, seed, density=density)
            assert all(x.arrive == x.expect and x.returned == x.ret_expect for x in ranks)


def test_tile_model_needs_the_scratch_free_flag():
    """Sanity of the model: with sparse routing and no "scratch free" wait, a fast rank's next backward dispatch does land in a
    receive scratch that its owner is still reading."""
    with pytest.raises(AssertionError):
        for seed in range(300):
            run_tiles(4, seed, density=0.3, free_wait=False)
