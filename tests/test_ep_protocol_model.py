"""Host-side model of the expert-parallel exchange protocol (flags written by peers, epochs in per-rank device counters).

Each rank runs, per MoE layer call, the stream-ordered sequence of parallel/ep.py:

    push counts (+ flag64)   -> wait flag64     -> read counts
    dispatch rows to peers   -> signal flag128  -> wait flag128 -> expert GEMMs read the receive buffer
    return rows to peers     -> signal flag192  -> wait flag192 -> combine reads the return buffer

Ranks advance in a random interleaving (any rank that is not blocked may take its next step). The model checks what the
design relies on when ONE set of buffers serves every layer (inference) and the counts slab is not double-buffered:
no deadlock, and no rank ever overwrites a peer's counts / receive / return buffer while that peer has not yet consumed the
previous exchange's contents."""

import random

import pytest

STEPS = ["push_counts", "wait64", "read_counts", "dispatch", "signal128", "wait128", "gemm_reads_recv",
         "return", "signal192", "wait192", "combine_reads_ret"]


class Rank:
    def __init__(self, r, world):
        self.r, self.world = r, world
        self.ctr = {64: 0, 128: 0, 192: 0}                 # device counters (epoch of the last signal sent)
        self.flags = {o: [0] * world for o in (64, 128, 192)}   # written by peers
        self.pc, self.call = 0, 0
        # generation (call index) of the data currently held in each buffer, per writer
        self.counts_gen = [-1] * world
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
                assert p.consumed["counts"] >= n - 1, f"rank {rk.r} overwrites counts of rank {p.r} before call {n - 1} was read"
                p.counts_gen[rk.r] = n
                p.flags[64][rk.r] = rk.ctr[64]
        elif step == "read_counts":
            assert rk.counts_gen == [n] * world
            rk.consumed["counts"] = n
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
