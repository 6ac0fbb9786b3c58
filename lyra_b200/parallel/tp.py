"""Megatron-style tensor parallelism for inference (the ``model`` axis of ``ShardingRules``).

Roles in the reference: q / k / v and the MLP up-projections are column-sharded on the model axis, the attention output and
MLP down-projections row-sharded, with a sum over the axis after the output projection, the MoE down-projection and the
dense down-projection; biases of row-sharded layers are divided by the axis size before the sum
(lyra/model.py:366,549,628, lyra/kernels/ep_moe.py:58). Here:

* attention: every rank holds ``Nq / tp`` query heads and ``Nkv / tp`` kv heads (columns of q / k / v, rows of ``out``, the
  matching entries of ``sinks`` / ``xsa_alpha`` and columns of ``sdpa_gate``); its KV cache holds its kv heads only;
* dense MLP and experts: the hidden dimension is split (last axis of ``mlp_up`` and of its bias, row axis of ``mlp_down``);
* everything else (norm scales, router, embeddings, output biases) is replicated; the residual stream is replicated, and the
  partial results are summed with one all-reduce per block (``tp_all_reduce``; the expert down-projection bias enters as
  ``bias / tp`` on every rank so that the sum restores it).

Training on the model axis (every rank of an axis sees the same rows; ``TensorParallel.mesh`` adds a data axis of replicas
around it, with gradients summed over the replicas; expert parallelism is the other runtime's business):

* the all-reduce after a row-sharded layer is the identity in backward, and ``tp_copy`` - the identity in forward, applied
  where a replicated activation (the normalised layer input, the routing scores) enters sharded layers - sums the partial
  gradients over the axis in backward, so replicated parameters upstream see whole gradients (Megatron's ``g`` / ``f`` pair);
* replicated parameters that sit inside a sharded region receive partial gradients and are summed in ``reduce_grads``: the
  per-head-dim q / k norm scales (every rank normalises its own heads) and the expert down-projection bias (``bias / tp``);
* parameters, gradients and moments of a sharded leaf stay sharded; Muon's per-matrix RMS and Newton-Schulz need whole
  matrices, so ``optimizer_step`` gathers the gradient and the update direction over the axis (``gather_leaf``) and keeps
  its own slice of the result (``slice_leaf``). Adam is element-wise and stays local;
* checkpoints hold global arrays: every rank writes its slice (``shard_of`` / ``checkpoint_leaves``), rank 0 the replicated
  leaves.

The step runs the PyTorch optimizer (``owns_optimizer``) and library collectives on any ``torch.distributed`` backend; the
fused peer-memory paths of ``parallel/runtime.py`` do not apply to this axis."""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from lyra_b200.config import ModelConfig
from lyra_b200.nn.params import ShardInfo, tree_dict

_COLUMNS = {"q", "k", "v", "sdpa_gate"}                 # [C, heads * ...]: shard dim 1
_ROWS = {"out"}                                         # [heads * hd, C]: shard dim 0
_VECTORS = {"q_bias", "k_bias", "v_bias", "sinks", "xsa_alpha"}   # [heads (* hd)]: shard dim 0


_PARTIAL_GRADS = {"qnorm_scale", "knorm_scale"}         # replicated, but each rank sees only its own heads


class _SumForward(torch.autograd.Function):
    """Sum over the axis in forward, identity in backward (after a row-sharded layer)."""

    @staticmethod
    def forward(ctx, t, group):
        t = t.contiguous().clone()
        dist.all_reduce(t, group=group)
        return t

    @staticmethod
    def backward(ctx, g):
        return g, None


class _SumBackward(torch.autograd.Function):
    """Identity in forward, sum over the axis in backward (in front of column-sharded layers)."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return t.view_as(t)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def _bucketed_all_reduce(tensors: list[torch.Tensor], group, bucket_bytes: int = 256 << 20) -> None:
    """Sums every tensor over ``group`` in place, a few hundred MB per collective: one launch latency per bucket instead of one
    per leaf, with a bounded staging buffer."""
    by_dtype: dict[torch.dtype, list[torch.Tensor]] = {}
    for t in tensors:
        by_dtype.setdefault(t.dtype, []).append(t)
    for dtype, ts in by_dtype.items():
        bucket, size = [], 0
        limit = max(1, bucket_bytes // torch.empty((), dtype=dtype).element_size())

        def flush():
            if not bucket:
                return
            if len(bucket) == 1 and bucket[0].is_contiguous():
                dist.all_reduce(bucket[0], group=group)
                return
            flat = torch.cat([t.reshape(-1) for t in bucket])
            dist.all_reduce(flat, group=group)
            offset = 0
            for t in bucket:
                t.copy_(flat[offset:offset + t.numel()].view_as(t))
                offset += t.numel()

        for t in ts:
            if size + t.numel() > limit and bucket:
                flush()
                bucket, size = [], 0
            bucket.append(t)
            size += t.numel()
        flush()


class TensorParallel:
    """Runtime object accepted by ``model_apply(..., rt=...)``, ``BatchedGenerator(..., rt=...)`` and ``Stepper(..., rt=...)``."""

    implementation = "nccl"
    ep_size = 1
    data_size, data_rank = 1, 0                          # every rank of the axis works on the same rows
    owns_optimizer = True                                # the step uses the PyTorch optimizer with the gather hooks below
    load_meter = None

    def __init__(self, mcfg: ModelConfig, rank: int, size: int, group=None):
        """One model axis of ``size`` ranks (``group``, or all ranks); ``rank`` is the index on it. See ``mesh`` for data x model."""
        if mcfg.n_attn_heads % size or mcfg.n_kv_heads % size:
            raise ValueError(f"{mcfg.n_attn_heads} query / {mcfg.n_kv_heads} kv heads do not split over {size} ranks")
        self.mcfg, self.rank, self.tp_rank, self.tp_size, self.group = mcfg, rank, rank, size, group
        self.world, self.world_group, self.data_group = size, group, None
        self.n_kv_local = mcfg.n_kv_heads // size

    @classmethod
    def mesh(cls, mcfg: ModelConfig, rank: int, world: int, model_axis: int) -> "TensorParallel":
        """``world = data x model`` ranks of the default process group, the model axis fastest (ranks ``d * model .. d * model +
        model - 1`` hold one replica; the reference's ``tensor_parallel(data_axis, model_axis)`` layout, lyra/nn/params.py:168-265).
        Rows are split over the data axis; gradients are summed over it after the partial gradients of the model axis."""
        if world % model_axis:
            raise ValueError(f"{world} ranks do not split into model axes of {model_axis}")
        data = world // model_axis
        self = cls(mcfg, rank % model_axis, model_axis)
        self.rank, self.world, self.world_group = rank, world, None
        self.data_size, self.data_rank = data, rank // model_axis
        # every rank creates every group, in the same order
        for d in range(data):
            g = dist.new_group(list(range(d * model_axis, (d + 1) * model_axis)))
            if d == self.data_rank:
                self.group = g
        for m in range(model_axis):
            g = dist.new_group(list(range(m, world, model_axis)))
            if m == self.tp_rank:
                self.data_group = g
        return self

    # ------------------------------------------------------------------ placement
    def shard_info(self, path: str, spec: Any) -> ShardInfo:
        name = path.split("/")[-1]
        nd = len(spec.shape)
        if self.tp_size == 1:
            return ShardInfo()
        if name in _COLUMNS:
            return ShardInfo(((1, self.tp_rank, self.tp_size),))
        if name in _ROWS or name in _VECTORS:
            return ShardInfo(((0, self.tp_rank, self.tp_size),))
        if name in ("mlp_up", "mlp_up_bias"):
            return ShardInfo(((nd - 1, self.tp_rank, self.tp_size),))
        if name == "mlp_down":
            return ShardInfo(((nd - 2, self.tp_rank, self.tp_size),))
        return ShardInfo()

    # ------------------------------------------------------------------ hooks of the model code
    def materialize(self, p):
        return p

    def begin_layer(self, idx: int) -> None:
        pass

    def tp_all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            if torch.is_grad_enabled() and t.requires_grad:
                return _SumForward.apply(t, self.group)
            t = t.contiguous()
            dist.all_reduce(t, group=self.group)
        return t

    def tp_copy(self, t: torch.Tensor) -> torch.Tensor:
        """Marks the point where a replicated activation enters sharded layers."""
        if self.tp_size > 1 and torch.is_grad_enabled() and t.requires_grad:
            return _SumBackward.apply(t, self.group)
        return t

    # ------------------------------------------------------------------ training hooks (the stepper's contract)
    def _specs(self) -> dict:
        if not hasattr(self, "_spec_cache"):
            from lyra_b200.model import ModelWeights

            self._spec_cache = tree_dict(ModelWeights.spec(self.mcfg))
        return self._spec_cache

    def _info(self, path: str) -> ShardInfo:
        spec = self._specs().get(path)
        return self.shard_info(path, spec) if spec is not None else ShardInfo()

    def register(self, params: Any) -> None:
        pass

    def meter_expert_load(self) -> bool:
        return False                                      # every rank holds a slice of every expert: nothing to re-place

    def begin_microbatch(self, index: int, total: int) -> None:
        pass

    def after_optimizer(self, params: dict[str, torch.Tensor]) -> None:
        pass

    def barrier(self) -> None:
        dist.barrier(group=self.world_group)

    def sum_scalars(self, t: torch.Tensor) -> torch.Tensor:
        if self.data_size > 1:                            # the ranks of a model axis see the same rows; the data axis splits them
            dist.all_reduce(t, group=self.data_group)
        return t

    def sum_over_ranks(self, *ts: torch.Tensor):
        stacked = torch.stack([t.float() for t in ts])
        dist.all_reduce(stacked, group=self.world_group)
        return tuple(stacked.unbind(0))

    def max_over_ranks(self, t: torch.Tensor) -> torch.Tensor:
        t = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.world_group)
        return t

    def counts_once(self, path: str) -> bool:
        """Whether this rank counts ``path`` in global norms: on the first replica, every rank its own slice of a sharded leaf
        and the first rank the replicated leaves."""
        return self.data_rank == 0 and (bool(self._info(path).slices) or self.tp_rank == 0)

    @torch.no_grad()
    def reduce_grads(self, grads: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        specs = self._specs()
        for path, g in grads.items():
            name = path.split("/")[-1]
            if name in _PARTIAL_GRADS or (name == "mlp_down_bias" and specs[path].kind.startswith("moe_")):
                dist.all_reduce(g, group=self.group)
        if self.data_size > 1:                            # the loss terms carry 1 / data_size: a sum over the replicas
            _bucketed_all_reduce(list(grads.values()), self.data_group)
        return grads

    def gather_leaf(self, path: str, t: torch.Tensor) -> torch.Tensor:
        info = self._info(path)
        if not info.slices:
            return t
        (dim, _, parts), = info.slices
        pieces = [torch.empty_like(t) for _ in range(parts)]
        dist.all_gather(pieces, t.contiguous(), group=self.group)
        return torch.cat(pieces, dim=dim)

    def slice_leaf(self, path: str, full: torch.Tensor) -> torch.Tensor:
        return self._info(path).narrow(full)

    # ------------------------------------------------------------------ checkpoints (global arrays, one slice per rank)
    def shard_of(self, path: str, t: torch.Tensor):
        spec = self._specs().get(path)
        if spec is None:
            return tuple(t.shape), ShardInfo()
        return tuple(spec.shape), self.shard_info(path, spec)

    def writes_leaf(self, path: str) -> bool:
        return self.data_rank == 0 and (bool(self._info(path).slices) or self.tp_rank == 0)

    def checkpoint_leaves(self, name: str, tree: Any):
        present = tree_dict(tree)
        specs = self._specs()
        if not present or not all(p in specs for p in present):
            return None
        out = {}
        for p, t in present.items():
            parts = [1] * len(specs[p].shape)
            for dim, _, n in self._info(p).slices:
                parts[dim] = n
            out[p] = (tuple(specs[p].shape), t.dtype, tuple(parts))
        return out


def shared_terminal(rt: TensorParallel, input_fn=input, output_fn=print) -> dict:
    """``input_fn`` / ``output_fn`` for an interactive loop that runs on every rank of the axis: rank 0 talks to the user,
    the others receive what it read (an ``EOFError`` included) and print nothing."""

    def read(prompt: str) -> str:
        box = [None]
        if rt.rank == 0:
            try:
                box[0] = input_fn(prompt)
            except EOFError:
                box[0] = EOFError
        dist.broadcast_object_list(box, src=dist.get_global_rank(rt.world_group, 0) if rt.world_group is not None else 0, group=rt.world_group)
        if box[0] is EOFError:
            raise EOFError
        return box[0]

    def write(*args, **kwargs) -> None:
        if rt.rank == 0:
            output_fn(*args, **kwargs)

    return {"input_fn": read, "output_fn": write}
