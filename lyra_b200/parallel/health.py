"""Host-side liveness of the ranks of a job: a step-boundary heartbeat through the rendezvous store.

The reference has no failure detection beyond atomic checkpoints and the non-finite step skip. A job with one process per
GPU needs a little more: if a rank dies, the others would otherwise sit in their next peer wait (which gives up after two
seconds and reports a status code) or in a collective until its time-out. With a heartbeat every rank learns *on the host,
before its next launch,* that a peer is gone, and can stop cleanly (checkpoint, exit) instead of launching kernels that wait
for a dead peer. Ranks leave only between steps, with nothing in flight.

Usage (one ``Heartbeat`` per rank, any ``torch.distributed`` store: ``TCPStore``, ``FileStore``, the process group's)::

    hb = Heartbeat(store, rank, world)
    for step in range(steps):
        hb.beat(step)                 # "I am about to run step `step`"
        hb.check(step, timeout=30.0)  # raises PeerLost if some rank has not announced `step` in time or announced that it leaves
        train_step(...)
    hb.done()                         # ran every step: the others' remaining checks pass; hb.leave() = gone early, they stop
"""

from __future__ import annotations

import time


class PeerLost(RuntimeError):
    def __init__(self, rank: int, why: str):
        super().__init__(f"rank {rank} {why}")
        self.rank = rank


class Heartbeat:
    LEFT = -1
    DONE = 1 << 62                    # "past every step": a rank that finished never holds up, or alarms, a slower one

    def __init__(self, store, rank: int, world: int, prefix: str = "lyra/hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        self.store.set(self._key(self.rank), str(self.LEFT))

    def done(self) -> None:
        self.store.set(self._key(self.rank), str(self.DONE))

    def _read(self, rank: int) -> int | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return None
            return int(self.store.get(self._key(rank)).decode())
        except Exception:
            return None

    def check(self, step: int, timeout: float = 30.0, poll: float = 0.01) -> None:
        """Returns once every other rank has announced ``step`` (or a later one). Raises ``PeerLost`` when a rank announced
        that it leaves, or did not announce ``step`` within ``timeout`` seconds."""
        deadline = time.monotonic() + timeout
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                v = self._read(r)
                if v == self.LEFT:
                    raise PeerLost(r, "left the job")
                if v is None or v < step:
                    still.append(r)
            pending = still
            if pending:
                if time.monotonic() > deadline:
                    raise PeerLost(pending[0], f"did not reach step {step} within {timeout:.1f} s")
                time.sleep(poll)
