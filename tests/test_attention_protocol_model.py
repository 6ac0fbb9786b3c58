"""Host-side model of the synchronisation inside the persistent flash-attention forward kernel (csrc/attn/flash_fwd.cu).

Four agents run the kernel's role loops as written there - the TMA producer, the MMA issuer and the two softmax groups - plus
the tensor pipe, which retires the issued products and commits strictly in issue order. They advance in a random
interleaving. mbarriers are modelled with their phase parity (a wait on parity p passes once the phase of that parity has
completed; a fresh barrier passes waits on parity 1). Every buffer carries a tag of what it holds; each read checks the tag
and each write checks that the previous contents were consumed. The model therefore fails on a wrong parity, a missing wait
or a buffer reused too early, and on any deadlock."""

import random

import pytest


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier was initialised for"
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def done(self, parity):                      # has the phase with this parity completed?
        return (self.phase & 1) != parity


class Kernel:
    def __init__(self, items, rng):
        self.items, self.rng = items, rng       # items: key-tile counts of this CTA's work items, in order
        one = lambda: Bar(1)
        self.q_full, self.q_empty, self.o_full = one(), one(), one()
        self.k_full, self.k_empty, self.v_full, self.v_empty = [one(), one()], [one(), one()], [one(), one()], [one(), one()]
        self.s_full, self.p_full = [one(), one()], [one(), one()]      # a group counts as one arriving agent here
        self.l_full, self.o_empty = Bar(2), Bar(2)
        self.q = None                            # item whose Q is in shared memory
        self.k, self.v = [None, None], [None, None]      # (item, tile) per stage
        self.s = [None, None]                    # per group: ("S", item, tile) or ("P", item, tile)
        self.o = [None, None]                    # per group: (item, set of tiles accumulated)
        self.pipe = []                           # issued, not yet retired: closures
        self.k_read, self.v_read, self.q_reads = [True, True], [True, True], 0
        self.p_consumed = [True, True]
        self.o_read = [True, True]               # previous item's accumulator read by the epilogue of both groups
        self.outputs = []

    # ---------------------------------------------------------------- agents (generators yield a wait condition or None)
    def tma(self):
        t = n = 0
        for it, n_tiles in enumerate(self.items):
            if n_tiles == 0:
                continue
            yield lambda n=n: self.q_empty.done((n & 1) ^ 1)
            assert self.q is None or self.q_reads == 0, "Q overwritten while a product still has to read it"
            self.q = it
            self.q_full.arrive()
            n += 1
            for j in range(n_tiles):
                s, ph = t & 1, (t >> 1) & 1
                yield lambda s=s, ph=ph: self.k_empty[s].done(ph ^ 1)
                assert self.k_read[s], "K stage overwritten before its product retired"
                self.k[s], self.k_read[s] = (it, j), False
                self.k_full[s].arrive()
                yield lambda s=s, ph=ph: self.v_empty[s].done(ph ^ 1)
                assert self.v_read[s], "V stage overwritten before its product retired"
                self.v[s], self.v_read[s] = (it, j), False
                self.v_full[s].arrive()
                t += 1

    def mma(self):
        t = n = 0
        c = [0, 0]
        for it, n_tiles in enumerate(self.items):
            if n_tiles == 0:
                continue
            t0 = t

            def issue_s(j, it=it, t0=t0, n_tiles=n_tiles):
                g, s = j & 1, (t0 + j) & 1
                yield lambda: self.k_full[s].done(((t0 + j) >> 1) & 1)
                self.q_reads += 1

                def run():
                    assert self.q == it and self.k[s] == (it, j), (self.q, self.k[s], it, j)
                    assert self.s[g] is None or self.p_consumed[g], "scores written over probabilities that were not multiplied yet"
                    self.s[g] = ("S", it, j)
                    self.k_read[s] = True
                    self.q_reads -= 1
                self.pipe.append(run)
                self.pipe.append(self.s_full[g].arrive)
                self.pipe.append(self.k_empty[s].arrive)
                if j == n_tiles - 1:
                    self.pipe.append(self.q_empty.arrive)

            yield lambda n=n: self.q_full.done(n & 1)
            yield from issue_s(0)
            if n_tiles > 1:
                yield from issue_s(1)
            yield lambda n=n: self.o_empty.done((n & 1) ^ 1)
            for j in range(n_tiles):
                g, s = j & 1, (t0 + j) & 1
                yield lambda s=s, j=j: self.v_full[s].done(((t0 + j) >> 1) & 1)
                yield lambda g=g: self.p_full[g].done(c[g] & 1)
                c[g] += 1

                def run(g=g, s=s, j=j, it=it):
                    assert self.s[g] == ("P", it, j) and self.v[s] == (it, j), (self.s[g], self.v[s], it, j)
                    if j < 2:
                        assert self.o_read[g], "accumulator overwritten before the previous item's output was read"
                        self.o[g], self.o_read[g] = (it, set()), False
                    assert self.o[g][0] == it
                    self.o[g][1].add(j)
                    self.p_consumed[g] = True
                    self.v_read[s] = True
                self.pipe.append(run)
                self.pipe.append(self.v_empty[s].arrive)
                if j + 2 < n_tiles:
                    yield from issue_s(j + 2)
            self.pipe.append(self.o_full.arrive)
            t += n_tiles
            n += 1

    def group(self, g):
        n = cg = 0
        for it, n_tiles in enumerate(self.items):
            for j in range(g, n_tiles, 2):
                yield lambda cg=cg: self.s_full[g].done(cg & 1)
                assert self.s[g] == ("S", it, j), (self.s[g], it, j)
                if j >= 2:                          # a rescale may touch the accumulator: everything issued for it must have retired
                    assert self.o[g] == (it, set(range(g, j, 2))), (self.o[g], it, j)
                yield None                          # the exponentials take a while
                self.s[g], self.p_consumed[g] = ("P", it, j), False
                self.p_full[g].arrive()
                cg += 1
            if n_tiles == 0:
                self.outputs.append((it, g, "empty"))
                continue
            par = n & 1
            self.l_full.arrive()
            yield lambda par=par: self.o_full.done(par)
            yield lambda par=par: self.l_full.done(par)
            mine = set(range(g, n_tiles, 2))
            if mine:
                assert self.o[g] == (it, mine), (self.o[g], it, mine)
            other = set(range(g ^ 1, n_tiles, 2))
            if other:
                assert self.o[g ^ 1] == (it, other), (self.o[g ^ 1], it, other)
            yield None
            self.outputs.append((it, g, "written"))
            if g == 0:                              # both groups must be past their reads: modelled by the second arrival below
                pass
            self.o_read_pending = getattr(self, "o_read_pending", 0) + 1
            if self.o_read_pending == 2:
                self.o_read_pending = 0
                self.o_read = [True, True]
            self.o_empty.arrive()
            n += 1

    # ---------------------------------------------------------------- scheduler
    def run(self):
        agents = {"tma": self.tma(), "mma": self.mma(), "g0": self.group(0), "g1": self.group(1)}
        waiting = {}
        live = set(agents)
        idle = 0
        while live or self.pipe:
            choices = list(live) + (["pipe"] if self.pipe else [])
            who = self.rng.choice(choices)
            if who == "pipe":
                self.pipe.pop(0)()
                idle = 0
                continue
            cond = waiting.get(who)
            if cond is not None and not cond():
                idle += 1
                assert idle < 20000, f"deadlock: {sorted(live)} wait, pipe empty={not self.pipe}"
                continue
            waiting.pop(who, None)
            idle = 0
            try:
                nxt = next(agents[who])
                if nxt is not None:
                    waiting[who] = nxt
            except StopIteration:
                live.discard(who)
        return self.outputs


@pytest.mark.parametrize("seed", range(60))
def test_forward_kernel_protocol_has_no_deadlock_and_no_early_reuse(seed):
    rng = random.Random(seed)
    items = [rng.choice([0, 1, 1, 2, 3, 4, 5, 8]) for _ in range(rng.randint(1, 7))]
    out = Kernel(items, rng).run()
    assert sorted(out) == sorted((it, g, "written" if n else "empty") for it, n in enumerate(items) for g in (0, 1))


def test_the_model_sees_a_missing_output_wait():
    """Sanity of the model: without the wait for the previous item's output to be read, the next item's first product does
    overwrite an accumulator that is still being read."""
    class Broken(Kernel):
        def mma(self):
            for step in Kernel.mma(self):
                if step is not None and getattr(step, "__defaults__", None) and step.__code__.co_names[-2:] == ("o_empty", "done"):
                    continue                        # drop the o_empty wait
                yield step

    with pytest.raises(AssertionError):
        for seed in range(300):
            rng = random.Random(seed)
            Broken([rng.choice([1, 2, 3]) for _ in range(5)], rng).run()


# ======================================================================================================================
# dK/dV kernel (csrc/attn/flash_bwd.cu): four-stage (Q, dO) ring, two elementwise groups on alternate iterations, each with its
# own S^T / dP^T buffers that it turns in place into the operands of the accumulating products; statistics double-buffered.
class DkvKernel:
    STAGES = 4

    def __init__(self, n_iter, rng, stages=4):
        self.n, self.rng, self.STAGES = n_iter, rng, stages
        one = lambda: Bar(1)
        self.kv_full, self.acc_full = one(), one()
        self.qd_full, self.qd_empty = [one() for _ in range(stages)], [one() for _ in range(stages)]
        self.st_full, self.pt_full = [one(), one()], [one(), one()]
        self.stage = [None] * stages            # iteration whose (Q, dO) the stage holds
        self.stage_reads = [0] * stages         # issued products that still have to read the stage
        self.st = [None, None]                  # per group: ("S", it) or ("P", it)
        self.p_consumed = [True, True]
        self.acc = set()
        self.pipe = []

    def tma(self):
        self.kv_full.arrive()
        for it in range(self.n):
            s, ph = it % self.STAGES, (it // self.STAGES) & 1
            yield lambda s=s, ph=ph: self.qd_empty[s].done(ph ^ 1)
            assert self.stage_reads[s] == 0, "(Q, dO) stage overwritten while a product still has to read it"
            self.stage[s] = it
            self.qd_full[s].arrive()

    def mma(self):
        def issue_st(it):
            s, g = it % self.STAGES, it & 1
            yield lambda: self.qd_full[s].done((it // self.STAGES) & 1)
            self.stage_reads[s] += 1

            def run():
                assert self.stage[s] == it, (self.stage[s], it)
                assert self.st[g] is None or self.p_consumed[g], "S^T written over operands that were not multiplied yet"
                self.st[g] = ("S", it)
                self.stage_reads[s] -= 1
            self.pipe.append(run)
            self.pipe.append(self.st_full[g].arrive)

        if self.n == 0:
            return
        yield lambda: self.kv_full.done(0)
        yield from issue_st(0)
        if self.n > 1:
            yield from issue_st(1)
        for it in range(self.n):
            s, g = it % self.STAGES, it & 1
            yield lambda g=g, it=it: self.pt_full[g].done((it >> 1) & 1)
            self.stage_reads[s] += 1

            def run(it=it, s=s, g=g):
                assert self.st[g] == ("P", it) and self.stage[s] == it, (self.st[g], self.stage[s], it)
                self.acc.add(it)
                self.p_consumed[g] = True
                self.stage_reads[s] -= 1
            self.pipe.append(run)
            self.pipe.append(self.qd_empty[s].arrive)
            if it + 2 < self.n:
                yield from issue_st(it + 2)
        self.pipe.append(self.acc_full.arrive)

    def group(self, g):
        for it in range(g, self.n, 2):
            yield lambda it=it: self.st_full[g].done((it >> 1) & 1)
            assert self.st[g] == ("S", it), (self.st[g], it)
            yield None
            self.st[g], self.p_consumed[g] = ("P", it), False
            self.pt_full[g].arrive()
        if self.n:
            yield lambda: self.acc_full.done(0)
            assert self.acc == set(range(self.n))

    def run(self):
        agents = {"tma": self.tma(), "mma": self.mma(), "g0": self.group(0), "g1": self.group(1)}
        waiting, live, idle = {}, set(agents), 0
        while live or self.pipe:
            who = self.rng.choice(list(live) + (["pipe"] if self.pipe else []))
            if who == "pipe":
                self.pipe.pop(0)()
                idle = 0
                continue
            cond = waiting.get(who)
            if cond is not None and not cond():
                idle += 1
                assert idle < 20000, f"deadlock: {sorted(live)}"
                continue
            waiting.pop(who, None)
            idle = 0
            try:
                nxt = next(agents[who])
                if nxt is not None:
                    waiting[who] = nxt
            except StopIteration:
                live.discard(who)


@pytest.mark.parametrize("seed", range(40))
def test_dkv_kernel_protocol_has_no_deadlock_and_no_early_reuse(seed):
    rng = random.Random(seed)
    DkvKernel(rng.choice([0, 1, 2, 3, 4, 5, 8, 9, 17, 32]), rng).run()


def test_dkv_ring_needs_more_than_two_stages_to_run_ahead():
    """With two stages the load of iteration it + 2 can only start when the products of iteration it have retired - it still
    works (the ring protocol is the same), it just cannot run ahead; the model accepts any ring length of two or more."""
    for stages in (2, 3, 4, 6):
        for seed in range(10):
            DkvKernel(9, random.Random(seed), stages=stages).run()


# ======================================================================================================================
# dQ kernel: Q and dO are copied once into TMEM by the two elementwise groups (barrier a_full, 2 arrivals here), then the same
# alternation as above over 64-key tiles with a four-stage (K, V) ring; dS replaces dP in place.
class DqKernel(DkvKernel):
    def __init__(self, n_tiles, rng, stages=4):
        super().__init__(n_tiles, rng, stages)
        self.q_full, self.a_full = Bar(1), Bar(2)
        self.resident = 0                           # groups whose operand copy has landed in TMEM

    def tma(self):
        if self.n:
            self.q_full.arrive()
        yield from (step for step in super().tma() if True)

    def mma(self):
        if self.n == 0:
            return
        yield lambda: self.a_full.done(0)
        assert self.resident == 2, "a product was issued before both resident operands were in TMEM"
        yield from super().mma()

    def group(self, g):
        if self.n:
            yield lambda: self.q_full.done(0)
            yield None                              # shared memory -> registers -> TMEM
            self.resident += 1
            self.a_full.arrive()
        yield from super().group(g)


@pytest.mark.parametrize("seed", range(30))
def test_dq_kernel_protocol_has_no_deadlock_and_no_early_reuse(seed):
    rng = random.Random(seed)
    DqKernel(rng.choice([0, 1, 2, 3, 5, 8, 13, 64]), rng).run()
