"""Expert placement by measured load (an addition; the reference places expert ``e`` on rank ``e // (E / ws)`` for good,
lyra/kernels/ep_moe.py:9-37, and takes whatever imbalance dropless routing produces).

Routing is dropless, so the rank whose experts draw the most tokens sets the pace of every MoE layer: the other ranks wait
for its rows at the return leg. Relabelling the experts of a layer is a symmetry of the model (permute the router's columns,
the router bias and the expert axis of the four expert leaves, together with their optimizer moments, and the function and
its training trajectory are unchanged), so the runtime may move experts between ranks at a step boundary without touching
the kernels, the expert-to-rank rule or the checkpoint format: slot ``s`` still lives on rank ``s // e_local``; what changes
is which expert sits in which slot.

* ``ExpertLoadMeter`` counts, on the device and without a host synchronisation, the tokens each routed slot of each MoE
  layer received (``route_tokens`` feeds it when ``Runtime.load_meter`` is set: in training forwards, or in every call when
  the meter was started for serving);
* ``plan_slots`` turns one layer's counts into a permutation of its routed slots: longest-processing-time assignment under
  the per-rank slot capacities (shared-expert slots stay where they are), rank labels chosen to keep as many experts as
  possible in place, refused unless the heaviest rank gets lighter by ``min_gain``;
* ``apply_slot_permutation`` carries it out: replicated router leaves are permuted locally, expert slabs travel point to
  point between the ranks (parameters and moments alike), in one fixed order on every rank;
* ``rebalance_experts`` does all layers and resets the meter. It is a collective: every rank calls it at the same step.
"""

from __future__ import annotations

from typing import Any, Sequence

import torch
import torch.distributed as dist

_EXPERT_LEAVES = ("mlp_up", "mlp_up_bias", "mlp_down", "mlp_down_bias")
_ROUTER_LEAVES = ("router", "router_bias")


class ExpertLoadMeter:
    """Per-layer token counts of the routed slots, accumulated on the device."""

    def __init__(self, moe_layers: Sequence[int], n_routed: int, device):
        self.layers = list(moe_layers)
        self._row = {layer: i for i, layer in enumerate(self.layers)}
        self.counts = torch.zeros(len(self.layers), n_routed, dtype=torch.int64, device=device)   # exact however long the window
        self.always = False                                   # False: training forwards only; True: inference calls too (serving)

    def add(self, layer: int, indices: torch.Tensor) -> None:
        row = self._row.get(layer)
        if row is None:
            return
        flat = indices.reshape(-1)
        self.counts[row].index_add_(0, flat, torch.ones_like(flat, dtype=torch.int64))   # no state of its own: safe inside a CUDA graph

    def add_counts(self, layer: int, counts: torch.Tensor) -> None:
        """The same with the per-expert counts already made (the routing kernels produce them)."""
        row = self._row.get(layer)
        if row is not None:
            self.counts[row] += counts[: self.counts.shape[1]]

    def reset(self) -> None:
        self.counts.zero_()


def rank_loads(load: Sequence[float], e_local: int, world: int) -> list[float]:
    out = [0.0] * world
    for s, v in enumerate(load):
        out[s // e_local] += float(v)
    return out


def plan_slots(load: Sequence[float], world: int, e_local: int, min_gain: float = 0.05) -> list[int] | None:
    """``load[s]``: tokens drawn by the expert that sits in routed slot ``s`` (``len(load)`` routed slots; the slots from
    there up to ``world * e_local`` hold shared experts and do not move). Returns ``perm`` with ``perm[new_slot] = old_slot``
    or ``None`` when no placement makes the heaviest rank at least ``min_gain`` lighter."""
    n = len(load)
    cap = [max(0, min(n, (r + 1) * e_local) - r * e_local) for r in range(world)]
    before = rank_loads(load, e_local, world)
    # longest processing time first, onto the lightest group that still has a free slot
    groups: list[list[int]] = [[] for _ in range(world)]
    weight = [0.0] * world
    for s in sorted(range(n), key=lambda i: (-float(load[i]), i)):
        home = s // e_local
        g = min((i for i in range(world) if len(groups[i]) < cap[i]), key=lambda i: (weight[i], i != home, i))
        groups[g].append(s)
        weight[g] += float(load[s])
    # local search: swap one expert of the heaviest group against a lighter one elsewhere while that lowers the pair's peak
    for _ in range(4 * n):
        h = max(range(world), key=lambda i: (weight[i], -i))
        best = None
        for g in range(world):
            if g == h:
                continue
            for a in groups[h]:
                for b in groups[g]:
                    d = float(load[a]) - float(load[b])
                    if d <= 0:
                        continue
                    peak = max(weight[h] - d, weight[g] + d)
                    if peak < weight[h] - 1e-9 and (best is None or peak < best[0]):
                        best = (peak, g, a, b)
        if best is None:
            break
        _, g, a, b = best
        groups[h][groups[h].index(a)] = b
        groups[g][groups[g].index(b)] = a
        d = float(load[a]) - float(load[b])
        weight[h] -= d
        weight[g] += d
    if max(weight) > (1.0 - min_gain) * max(before):
        return None
    # groups of equal capacity are interchangeable: label them so that most experts stay on their rank
    label: dict[int, int] = {}
    free = set(range(world))
    pairs = sorted(((sum(1 for s in groups[g] if s // e_local == r), -g, -r) for g in range(world) for r in range(world) if cap[g] == cap[r]),
                   reverse=True)
    for _, mg, mr in pairs:
        g, r = -mg, -mr
        if g not in label and r in free:
            label[g] = r
            free.discard(r)
    perm = [-1] * n
    for g, members in enumerate(groups):
        r = label[g]
        slots = list(range(r * e_local, r * e_local + cap[r]))
        stay = [s for s in members if s // e_local == r]
        for s in stay:
            perm[s] = s
        vacant = [s for s in slots if perm[s] < 0]
        for dst, s in zip(vacant, sorted(s for s in members if s // e_local != r)):
            perm[dst] = s
    assert sorted(perm) == list(range(n))
    return perm


def _tensors_of(path: str, params: dict[str, torch.Tensor], opt: Any) -> list[torch.Tensor]:
    out = []
    for tree in (params, opt.muon_moment, opt.adam_mu, opt.adam_nu):
        t = tree.get(path)
        if t is None:
            continue
        if not isinstance(t, torch.Tensor):               # block-quantised stack: values and scales both lead with the expert axis
            out.extend([t.qval, t.scale])
        elif t.numel() > 0:
            out.append(t)
    return out


@torch.no_grad()
def apply_slot_permutation(rt, layer: int, perm: Sequence[int], params: dict[str, torch.Tensor], opt: Any) -> int:
    """Moves the experts of MoE layer ``layer`` so that new slot ``s`` holds what old slot ``perm[s]`` held. Returns the
    number of expert slabs this rank received. Every rank calls it with the same ``perm``."""
    prefix = f"layers/{layer}/mlp/"
    n, e_local, rank = len(perm), rt.e_local, rt.rank
    index = torch.tensor(list(perm), dtype=torch.long)
    for leaf in _ROUTER_LEAVES:                              # replicated: every rank permutes its own copy
        for t in _tensors_of(prefix + leaf, params, opt):
            t.copy_(t.index_select(t.dim() - 1, index.to(t.device)))
    lo, hi = rank * e_local, min(n, (rank + 1) * e_local)
    local_moves = [(s - lo, perm[s] - lo) for s in range(lo, hi) if perm[s] != s and lo <= perm[s] < hi]
    recvs = [(s - lo, perm[s] // e_local) for s in range(lo, hi) if not lo <= perm[s] < hi]
    sends = [(perm[s] - lo, s // e_local) for s in range(n) if lo <= perm[s] < hi and not lo <= s < hi]   # ascending new slot
    received = 0
    for leaf in _EXPERT_LEAVES:
        for t in _tensors_of(prefix + leaf, params, opt):
            ops, landing = [], []
            # one global order (ascending new slot) on both ends of every pair, so the messages of a pair match up
            for src_local, peer in sends:
                ops.append(dist.P2POp(dist.isend, t[src_local].contiguous(), peer, group=rt.group))
            for dst_local, peer in recvs:
                buf = torch.empty_like(t[dst_local])
                landing.append((dst_local, buf))
                ops.append(dist.P2POp(dist.irecv, buf, peer, group=rt.group))
            if ops:
                for req in dist.batch_isend_irecv(ops):
                    req.wait()
            if local_moves:
                dst = torch.tensor([d for d, _ in local_moves], device=t.device)
                src = torch.tensor([s for _, s in local_moves], device=t.device)
                t[dst] = t[src]                               # the right-hand side is gathered into a new tensor first
            for dst_local, buf in landing:
                t[dst_local].copy_(buf)
            received += len(landing)
    return received


@torch.no_grad()
def rebalance_experts(rt, params: dict[str, torch.Tensor], opt: Any, *, min_gain: float = 0.05) -> dict:
    """Sums the metered loads over the ranks, re-places the experts of every MoE layer that gains from it and resets the
    meter. Returns ``{"layers_moved", "slabs_received", "max_share_before", "max_share_after"}`` (shares of the heaviest
    rank, averaged over the MoE layers; 1 / world is perfect balance)."""
    meter: ExpertLoadMeter = rt.load_meter
    counts = meter.counts.clone()
    dist.all_reduce(counts, group=rt.group)
    counts = counts.cpu().double()
    moved = slabs = 0
    before_share = after_share = 0.0
    for row, layer in enumerate(meter.layers):
        load = counts[row].tolist()
        total = max(sum(load), 1.0)
        before = max(rank_loads(load, rt.e_local, rt.world)) / total
        perm = plan_slots(load, rt.world, rt.e_local, min_gain)
        after = before
        if perm is not None:
            slabs += apply_slot_permutation(rt, layer, perm, params, opt)
            after = max(rank_loads([load[o] for o in perm], rt.e_local, rt.world)) / total
            moved += 1
        before_share += before
        after_share += after
    meter.reset()
    if moved and rt.device.type == "cuda":
        from lyra_b200.ops import cuda_ops

        cuda_ops.invalidate_shadows()                         # bf16 compute copies of the moved masters are stale
    k = max(1, len(meter.layers))
    return {"layers_moved": moved, "slabs_received": slabs, "max_share_before": before_share / k, "max_share_after": after_share / k}
