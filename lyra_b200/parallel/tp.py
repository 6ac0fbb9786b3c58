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

This runtime is forward-only: there is no gradient or optimizer sharding for the model axis (training runs shard by leaf
ownership and by expert, see ``parallel/runtime.py``). It works on any ``torch.distributed`` backend; every rank must be
given the same input rows."""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from lyra_b200.config import ModelConfig
from lyra_b200.nn.params import ShardInfo

_COLUMNS = {"q", "k", "v", "sdpa_gate"}                 # [C, heads * ...]: shard dim 1
_ROWS = {"out"}                                         # [heads * hd, C]: shard dim 0
_VECTORS = {"q_bias", "k_bias", "v_bias", "sinks", "xsa_alpha"}   # [heads (* hd)]: shard dim 0


class TensorParallel:
    """Runtime object accepted by ``model_apply(..., rt=...)`` and ``BatchedGenerator(..., rt=...)``."""

    implementation = "nccl"
    ep_size = 1

    def __init__(self, mcfg: ModelConfig, rank: int, size: int, group=None):
        if mcfg.n_attn_heads % size or mcfg.n_kv_heads % size:
            raise ValueError(f"{mcfg.n_attn_heads} query / {mcfg.n_kv_heads} kv heads do not split over {size} ranks")
        self.mcfg, self.rank, self.tp_size, self.group = mcfg, rank, size, group
        self.world = size
        self.n_kv_local = mcfg.n_kv_heads // size

    # ------------------------------------------------------------------ placement
    def shard_info(self, path: str, spec: Any) -> ShardInfo:
        name = path.split("/")[-1]
        nd = len(spec.shape)
        if self.tp_size == 1:
            return ShardInfo()
        if name in _COLUMNS:
            return ShardInfo(((1, self.rank, self.tp_size),))
        if name in _ROWS or name in _VECTORS:
            return ShardInfo(((0, self.rank, self.tp_size),))
        if name in ("mlp_up", "mlp_up_bias"):
            return ShardInfo(((nd - 1, self.rank, self.tp_size),))
        if name == "mlp_down":
            return ShardInfo(((nd - 2, self.rank, self.tp_size),))
        return ShardInfo()

    # ------------------------------------------------------------------ hooks of the model code
    def materialize(self, p):
        return p

    def begin_layer(self, idx: int) -> None:
        pass

    def tp_all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            t = t.contiguous()
            dist.all_reduce(t, group=self.group)
        return t
