"""Device-time accounting of a training step by phase, with CUDA events on the launching stream.

Off by default (a span is then a no-op). ``collect()`` switches it on for the steps run inside it and returns, per phase,
the summed device time between the events that bracket its launches - not wall clock, so host launch gaps do not count.
Spans may nest (``ep_wait`` lies inside ``forward_backward``); the caller reports them side by side, not as a partition."""

from __future__ import annotations

import contextlib
from collections import defaultdict

import torch

_spans: dict[str, list] | None = None
_NULL = contextlib.nullcontext()


@contextlib.contextmanager
def _timed(name: str):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    try:
        yield
    finally:
        end.record()
        if _spans is not None:
            _spans[name].append((start, end))


def span(name: str):
    if _spans is None or not torch.cuda.is_available():
        return _NULL
    return _timed(name)


class collect:
    """``with collect() as p: step(); p.totals_ms()`` -> ``{phase: milliseconds}`` for everything run inside."""

    def __enter__(self):
        global _spans
        _spans = defaultdict(list)
        self._mine = _spans
        return self

    def __exit__(self, *exc):
        global _spans
        _spans = None

    def totals_ms(self) -> dict[str, float]:
        torch.cuda.synchronize()
        return {name: sum(a.elapsed_time(b) for a, b in pairs) for name, pairs in self._mine.items()}
