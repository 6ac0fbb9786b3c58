"""Sharding runtime for one NVSwitch node: one process per GPU, one flat group of ranks that is at once the
data-parallel, the parameter-sharding (ZeRO-3 style) and the expert-parallel axis.

What is sharded and how (the reference shards rows of every matrix over an ``fsdp`` axis and all-gathers the whole
model at the top of a step, lyra/nn/params.py:154-165, lyra/training/steps.py:75-91; here the unit is chosen for Muon):

* dense matrices and embeddings - each leaf is *owned* by one rank (greedy size balancing). The owner keeps the fp32
  master and the optimizer moments and runs Newton-Schulz on the whole matrix locally; every rank keeps a bf16 compute
  copy that it pulls from the owner over NVLink after the optimizer step, and accumulates its gradient into a
  peer-mapped buffer from which the owner pull-reduces (fixed rank order, deterministic) at the end of the step;
* expert stacks - sharded by expert over the ranks; tokens travel to the experts (dispatch) and results travel back
  (return + weighted combine). The shared expert is applied to local tokens from a replicated bf16 copy that its
  owning rank refreshes once per step - not broadcast on every call as in lyra/kernels/ep_moe.py:62-77;
* small leaves (norm scales, sinks, biases, router, gate) - replicated; their gradients are summed over ranks.

``implementation="b200"`` moves all of this with the kernels of ``csrc/comm`` over peer-mapped memory;
``implementation="nccl"`` uses torch.distributed collectives with the same data flow (the baseline mode, also the
mode that runs on CPU with gloo).
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

from lyra_b200.config import ModelConfig
from lyra_b200.nn.params import ArraySpec, ShardInfo, Tag, tree_dict

BF16 = torch.bfloat16
SMALL_LEAF = int(os.environ.get("LYRA_SMALL_LEAF", 1 << 16))  # leaves below this many elements are replicated


def _is_expert(spec: ArraySpec) -> bool:
    return spec.kind.startswith("moe_mlp")


@dataclass
class Plan:
    """Static placement of every parameter leaf."""

    owner: dict[str, int] = field(default_factory=dict)        # dense sharded leaves -> owning rank
    replicated: set = field(default_factory=set)
    expert: set = field(default_factory=set)
    specs: dict[str, ArraySpec] = field(default_factory=dict)

    @classmethod
    def build(cls, mcfg: ModelConfig, world: int) -> "Plan":
        from lyra_b200.model import ModelWeights

        plan = cls()
        plan.specs = tree_dict(ModelWeights.spec(mcfg))
        dense = []
        for path, spec in plan.specs.items():
            n = math.prod(spec.shape)
            if _is_expert(spec) and world > 1 and mcfg.n_experts % world == 0:
                plan.expert.add(path)
            elif world > 1 and n >= SMALL_LEAF and spec.tag in (Tag.MATRIX, Tag.EMBEDDING):
                dense.append((n, path))
            else:
                plan.replicated.add(path)
        # Owners are balanced by the estimated time of the owner's optimizer work, not by size: a Muon matrix costs five
        # Newton-Schulz iterations of tensor-core GEMMs (about 25k FLOP per element at 4096 x 4096), an Adam leaf (the
        # embeddings) only a few bytes of HBM traffic per element, so equal sizes would leave the embedding owners idle.
        load = [0.0] * world
        costed = [(_owner_cost(path, plan.specs[path]), n, path) for n, path in dense]
        for cost, n, path in sorted(costed, key=lambda x: (-x[0], x[2])):
            r = min(range(world), key=lambda i: (load[i], i))
            plan.owner[path] = r
            load[r] += cost
        return plan


def _owner_cost(path: str, spec: ArraySpec) -> float:
    """Seconds (nominal) the owning rank spends on one optimizer step of this leaf."""
    from lyra_b200.training.optimizer import is_mlp_up

    n = math.prod(spec.shape)
    if spec.tag != Tag.MATRIX:
        return n * 20.0 / 6.0e12                                   # Adam: parameter, gradient, two moments, bf16 copy
    if is_mlp_up(path):
        *lead, rows, two, cols = spec.shape
        mats = (math.prod(lead) if lead else 1) * two
    else:
        *lead, rows, cols = spec.shape
        mats = math.prod(lead) if lead else 1
    m, k = min(rows, cols), max(rows, cols)
    ns_flops = 5.0 * (4.0 * m * m * k + 2.0 * m ** 3) * mats
    return ns_flops / 1.3e15 + n * 14.0 / 6.0e12


class Runtime:
    def __init__(self, world_size: int, rank: int, device, implementation: str, mcfg: ModelConfig, group=None):
        self.world, self.rank, self.device = world_size, rank, torch.device(device)
        self.implementation = implementation if self.device.type == "cuda" else "nccl"
        self.mcfg = mcfg
        self.group = group
        self.plan = Plan.build(mcfg, world_size)
        self.ep_size = world_size if self.plan.expert else 1
        self.tp_size = 1
        self.data_size, self.data_rank = world_size, rank
        self.owns_optimizer = False
        self.e_local = mcfg.n_experts // self.ep_size
        self._path_of: dict[int, str] = {}
        self._views: dict[str, torch.Tensor] = {}
        self._masters: dict[str, torch.Tensor] = {}
        self._comm = None
        self._ep_state: dict = {}
        self._layer = 0
        self.load_meter = None                                   # ExpertLoadMeter once expert re-placement is switched on
        self.grad_sumsq: dict[str, torch.Tensor] = {}
        self.routing_plan = None                                 # counts / permutation of the current MoE layer call, when the routing kernels made them

    @classmethod
    def create(cls, *, world_size: int, rank: int, device, implementation: str = "b200", mcfg: ModelConfig | None = None) -> "Runtime":
        assert mcfg is not None, "Runtime.create needs the model configuration to plan the sharding"
        return cls(world_size, rank, device, implementation, mcfg)

    # ------------------------------------------------------------------ placement queries (init / checkpoints)
    def shard_info(self, path: str, spec: Any) -> ShardInfo:
        base = path.split("#")[0]
        if base in self.plan.expert:
            return ShardInfo(((0, self.rank, self.ep_size),))
        if base in self.plan.owner and self.plan.owner[base] != self.rank:
            return ShardInfo(absent=True)
        return ShardInfo()

    def shard_of(self, path: str, t: torch.Tensor):
        spec = self.plan.specs.get(path)
        if spec is None:
            return tuple(t.shape), ShardInfo()
        info = self.shard_info(path, spec)
        return tuple(spec.shape), (ShardInfo() if info.absent else info)

    def writes_leaf(self, path: str) -> bool:
        if path in self.plan.expert:
            return True
        if path in self.plan.owner:
            return self.plan.owner[path] == self.rank
        return self.rank == 0

    def checkpoint_leaves(self, name: str, tree: Any) -> dict[str, tuple[tuple[int, ...], torch.dtype, tuple[int, ...]]] | None:
        """Global shape, dtype and chunk grid of every leaf of a parameter-shaped checkpointable, including the leaves
        this rank does not hold. ``tree`` supplies the dtype (moments differ from parameters)."""
        present = tree_dict(tree)
        if not present or not all(p in self.plan.specs for p in present):
            return None
        dtype = next(iter(present.values())).dtype
        tags = {self.plan.specs[p].tag for p in present}
        out = {}
        for p, spec in self.plan.specs.items():
            if spec.tag not in tags and name != "params":
                continue
            parts = [1] * len(spec.shape)
            if p in self.plan.expert:
                parts[0] = self.ep_size
            out[p] = (tuple(spec.shape), present[p].dtype if p in present else dtype, tuple(parts))
        return out

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ registration of the parameter tree
    def register(self, params: Any) -> None:
        """Binds the runtime to a parameter tree: allocates the bf16 compute copies and gradient buffers of every
        sharded dense leaf (and of the shared expert), fills them from the owners and remembers which tensor is which leaf."""
        from lyra_b200.parallel.comm import Comm

        leaves = tree_dict(params)
        self._masters = leaves
        self._path_of = {id(t): p for p, t in leaves.items()}
        c = self.mcfg
        entries: list[tuple[str, tuple[int, ...], int]] = []   # (name, shape, owner)
        for path, owner in self.plan.owner.items():
            entries.append((path, tuple(self.plan.specs[path].shape), owner))
        self._shared: dict[str, tuple[str, int]] = {}
        if self.ep_size > 1 and c.n_shared_experts:
            for path in sorted(self.plan.expert):
                if path.endswith(("mlp_up", "mlp_down")):
                    for j in range(c.n_shared_experts):
                        e = c.n_routed_experts + j
                        name = f"{path}#shared{j}"
                        entries.append((name, tuple(self.plan.specs[path].shape[1:]), e // self.e_local))
                        self._shared[name] = (path, e)
        self._entries = entries
        from lyra_b200.ops import cuda_ops

        grad_dtype = cuda_ops.GRAD_DTYPE if self.device.type == "cuda" else torch.float32
        self._comm = Comm(self, entries, grad_dtype)
        for name, shape, owner in entries:
            w = self._comm.weight_view(name).view(shape)
            w.requires_grad_(True)
            try:
                w.grad_dtype = None
            except Exception:
                pass
            self._views[name] = w
        self._name_of_view = {id(w): name for name, w in self._views.items()}
        if self._comm.p2p:
            cuda_ops.AG_HOOK = self._ag_hook
        self.refresh_weights()

    def _ag_hook(self, w):
        name = self._name_of_view.get(id(w))
        return self._comm.ag_info(name) if name is not None else None

    def _master_of(self, name: str) -> torch.Tensor:
        if name in self._shared:
            path, e = self._shared[name]
            return self._masters[path][e - self.rank * self.e_local]
        return self._masters[name]

    @torch.no_grad()
    def refresh_weights(self) -> None:
        """Owners publish bf16 copies of their masters; every rank pulls the leaves it does not own."""
        for name, shape, owner in self._entries:
            if owner == self.rank:
                self._comm.weight_view(name).view(shape).copy_(self._master_of(name).detach())
        self._comm.gather_weights()

    def finish_weight_pulls(self) -> None:
        """Completes every compute copy now (pulls that would otherwise ride inside the first forward GEMM of each leaf);
        for inference, where not every leaf's first use is a fused-pull GEMM."""
        if self._comm is not None and getattr(self._comm, "p2p", False):
            self._comm.finish_pending()
            self._comm.barrier()

    # ------------------------------------------------------------------ hooks used by the model / stepper
    def begin_layer(self, idx: int) -> None:
        self._layer = idx

    def begin_microbatch(self, index: int, total: int) -> None:
        if index == 0:
            self._comm.zero_grads()
            for w in self._views.values():
                w.grad = self._comm.grad_view_of(w)

    def materialize(self, p):
        if p is None or not isinstance(p, torch.Tensor):
            return p
        path = self._path_of.get(id(p))
        if path is not None and path in self._views:
            return self._views[path]
        return p

    def shared_expert_weights(self, up_leaf: torch.Tensor, down_leaf: torch.Tensor, j: int = 0):
        # leaves that were replaced after registration (ModelWeights.quantize) are found by the layer being applied; the shared
        # expert then runs from the bf16 copies of the registered masters
        up_path = self._path_of.get(id(up_leaf), f"layers/{self._layer}/mlp/mlp_up")
        down_path = self._path_of.get(id(down_leaf), f"layers/{self._layer}/mlp/mlp_down")
        return self._views[f"{up_path}#shared{j}"], self._views[f"{down_path}#shared{j}"]

    def tp_all_reduce(self, t):
        return t

    def sum_scalars(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def sum_over_ranks(self, *ts: torch.Tensor):
        stacked = torch.stack([t.float() for t in ts])
        dist.all_reduce(stacked, group=self.group)
        return tuple(stacked.unbind(0))

    def max_over_ranks(self, t: torch.Tensor) -> torch.Tensor:
        t = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    @torch.no_grad()
    def reduce_grads(self, grads: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """Turns per-rank gradients into the gradients of the leaves this rank updates: owned dense leaves are
        pull-reduced from every rank's buffer, replicated leaves are summed over ranks, expert leaves are local
        except the shared expert, whose slot receives the sum of every rank's shared-expert gradient."""
        out: dict[str, torch.Tensor] = {}
        reduced = self._comm.reduce_grads()                      # name -> reduced gradient (owned entries only)
        small = {p: g for p, g in grads.items() if p in self.plan.replicated}
        self._comm.all_reduce_small(small)
        for p, g in grads.items():
            if p in self.plan.replicated:
                out[p] = g
            elif p in self.plan.expert:
                out[p] = g
        for p in self.plan.expert:
            if p not in out and p in self._masters and p.endswith(("mlp_up", "mlp_down")):
                # an expert leaf that saw no routed token still needs a (zero) gradient slot for the shared expert
                out[p] = torch.zeros_like(self._masters[p], dtype=next(iter(grads.values())).dtype if grads else torch.float32)
        self.grad_sumsq = {}                                     # leaves whose norms the pull-reduce already produced (the optimizer reads this)
        for name, g in reduced.items():
            if name in self._shared:
                path, e = self._shared[name]
                out[path][e - self.rank * self.e_local].copy_(g.view(out[path].shape[1:]))
            else:
                out[name] = g.view(self.plan.specs[name].shape)
                sq = getattr(self._comm, "grad_sumsq", {}).get(name)
                if sq is not None:
                    self.grad_sumsq[name] = sq
        return out

    def after_optimizer(self, params: dict[str, torch.Tensor]) -> None:
        self.refresh_weights()

    def counts_once(self, path: str) -> bool:
        """Whether this rank counts ``path`` in global norms (replicated leaves are counted by rank 0 only)."""
        return path not in self.plan.replicated or self.rank == 0

    # ------------------------------------------------------------------ expert parallel MoE
    def meter_expert_load(self, inference: bool = False) -> bool:
        """Starts counting the tokens every routed expert slot receives (input of ``rebalance_experts``): in training forwards,
        or with ``inference`` in every model call (a serving process). Returns whether there is anything to re-place (experts
        sharded over more than one rank)."""
        if self.ep_size <= 1:
            return False
        if self.load_meter is None:
            from lyra_b200.parallel.placement import ExpertLoadMeter

            moe_layers = [i for i, kind in enumerate(self.mcfg.mlp_map) if kind == "moe"]
            self.load_meter = ExpertLoadMeter(moe_layers, self.mcfg.n_routed_experts, self.device)
        self.load_meter.always = inference
        return True

    def rebalance_experts(self, params: dict[str, torch.Tensor], optimizer_state=None, *, min_gain: float = 0.05) -> dict:
        """Collective, between steps: moves experts (masters and moments; parameters alone when serving) so that the ranks draw
        equal numbers of tokens."""
        from lyra_b200.parallel.placement import rebalance_experts
        from lyra_b200.training.optimizer import OptimizerState

        return rebalance_experts(self, params, optimizer_state if optimizer_state is not None else OptimizerState(), min_gain=min_gain)

    def ep_moe(self, xn, scores, indices, w, c: ModelConfig):
        from lyra_b200.parallel.ep import ep_moe_forward

        return ep_moe_forward(self, xn, scores, indices, w, c)
