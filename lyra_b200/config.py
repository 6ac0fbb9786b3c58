"""Model configuration and the sharding plan.

Field names and defaults follow the reference's ``ModelConfig`` (lyra/model.py:39-130) and
``ShardingRules`` factories (lyra/nn/params.py:168-265) so run configurations carry over. The
sharding plan is re-thought for one NVSwitch box: a single ``world`` axis plays data-parallel,
FSDP (row-sharded fp32 masters, optimizer state and bf16 shadows) and expert-parallel at once;
tensor parallelism stays expressible as a second axis.
"""

from __future__ import annotations

import enum
import math
from dataclasses import asdict, dataclass, field, replace
from typing import Literal

import torch

PADDED_VOCAB_SIZE = 204800

MLPKind = Literal["dense", "moe"]
Implementation = Literal["auto", "b200", "torch", "nccl"]


class Mode(enum.Enum):
    NOCACHE = "nocache"
    PREFILL = "prefill"
    DECODE = "decode"


# --------------------------------------------------------------------------- MLP layer maps
def full_moe(layers: int) -> tuple[MLPKind, ...]:
    return ("moe",) * layers


def interleaved_moe(layers: int, every: int = 4, first: int = 4) -> tuple[MLPKind, ...]:
    """1-based layer numbers ``first, first+every, ...`` are MoE (lyra/nn/params.py:128-129)."""
    return tuple("moe" if (i >= first and (i - first) % every == 0) else "dense" for i in range(1, layers + 1))


def moe_outer_dense(layers: int, start_dense: int = 0, end_dense: int = 0) -> tuple[MLPKind, ...]:
    return tuple("dense" if (i < start_dense or i >= layers - end_dense) else "moe" for i in range(layers))


# --------------------------------------------------------------------------- sharding plan
@dataclass(frozen=True)
class ShardingRules:
    """Sizes of the logical axes. ``data * fsdp * expert * model`` = number of ranks.

    On the B200 build the ``data``, ``fsdp`` and ``expert`` roles are carried by one flat group of
    ranks (``world_axis``): the batch is split over it, dense parameters are row-sharded over it and
    experts are distributed over it. ``model`` is the Megatron tensor-parallel axis.
    """

    data: int = 1
    fsdp: int = 1
    expert: int = 1
    model: int = 1

    @property
    def data_axis_size(self) -> int:
        return self.data * self.fsdp * self.expert

    @property
    def model_axis_size(self) -> int:
        return self.model

    @property
    def expert_axis_size(self) -> int:
        return self.expert

    @property
    def fsdp_axis_size(self) -> int:
        return self.fsdp

    @property
    def world_size(self) -> int:
        return self.data * self.fsdp * self.expert * self.model


def no_sharding() -> ShardingRules:
    return ShardingRules()


def data_parallel(data_axis: int = 1) -> ShardingRules:
    return ShardingRules(data=data_axis)


def tensor_parallel(data_axis: int = 1, model_axis: int = 1) -> ShardingRules:
    return ShardingRules(data=data_axis, model=model_axis)


def expert_parallel(fsdp: int = 1, expert: int = 1) -> ShardingRules:
    return ShardingRules(fsdp=fsdp, expert=expert)


# --------------------------------------------------------------------------- model config
@dataclass(frozen=True, kw_only=True)
class ModelConfig:
    # Core
    name: str
    seq_len: int = 4096
    n_embd: int = 2048
    n_layers: int = 16
    vocab_size: int = 201088
    tie_embeddings: bool = True
    padded_vocab_size: int = PADDED_VOCAB_SIZE
    seed: int = 42

    # Attention
    head_dim: int = 128
    n_attn_heads: int = 16
    n_kv_heads: int = 4
    sliding_window: int = 128
    use_qk_norm: bool = True
    use_qkv_bias: bool = False
    use_attn_out_bias: bool = False
    use_learned_xsa: bool = False
    use_sdpa_output_gate: bool = False

    # MLP
    mlp_map: tuple[MLPKind, ...]
    n_routed_experts: int = 15
    n_shared_experts: int = 1
    n_active_experts: int = 4
    expert_mlp_widening: float = 2.0
    dense_mlp_widening: float = 3.0
    swiglu_beta: float = 1.702
    swiglu_limit: float = 7.0
    load_balance_weight: float = 1e-2
    router_z_loss_weight: float = 1e-4
    use_mlp_bias: bool = False
    use_router_bias: bool = True

    # RoPE
    rope_base: float = 150000.0
    rope_scale: float = 1.0
    ntk_alpha: float = 1.0
    ntk_beta: float = 32.0

    # Dtypes & quantisation
    param_dtype: torch.dtype = torch.float32
    compute_dtype: torch.dtype = torch.bfloat16
    gemm_dtype: torch.dtype = torch.bfloat16
    quantize_attn: bool = False
    quantize_mlp: bool = False
    quantize_cache: bool = False
    quant_block: tuple[int, int] = (256, 256)

    # Sharding & parameters
    sharding: ShardingRules = field(default_factory=ShardingRules)
    router_logit_std: float = 0.50
    w_init: str = "lecun_normal"
    b_init: str = "zeros"
    norm_init: str = "ones"

    # Kernels & ops
    mode: Mode = Mode.NOCACHE
    use_presorted_emb_gather: bool = True
    implementation: Implementation = "auto"

    # Misc
    sample_topk: int = 4
    sample_temperature: float = 0.8
    norm_eps: float = 1e-5

    def __post_init__(self):
        assert len(self.mlp_map) == self.n_layers, "mlp_map needs one entry per layer"

    @property
    def n_experts(self) -> int:
        return self.n_routed_experts + self.n_shared_experts

    @property
    def n_active_routed_experts(self) -> int:
        return self.n_active_experts - self.n_shared_experts

    @property
    def n_moe_layers(self) -> int:
        return self.mlp_map.count("moe")

    @property
    def residual_scale(self) -> float:
        return 1.0 / math.sqrt(2.0 * self.n_layers)

    @property
    def dense_residual_scale(self) -> float:
        return self.residual_scale * (self.n_active_experts**-0.5 if "moe" in self.mlp_map else 1.0)

    @property
    def expert_hidden(self) -> int:
        return int(self.n_embd * self.expert_mlp_widening) // 2

    @property
    def dense_hidden(self) -> int:
        return int(self.n_embd * self.dense_mlp_widening) // 2

    def layer_window(self, idx: int) -> int:
        """Even layers (0-based) are sliding-window, odd layers global (lyra/model.py:337)."""
        return self.sliding_window if idx % 2 == 0 else 0

    def to_dict(self) -> dict:
        d = asdict(self)
        for k, v in list(d.items()):
            if isinstance(v, torch.dtype):
                d[k] = str(v).replace("torch.", "")
            elif isinstance(v, enum.Enum):
                d[k] = v.value
        return d


def flops_per_token(c: ModelConfig) -> float:
    """Analytical training FLOPs per token used for MFU (dev/docs/kernels.md:29-38 of the reference):
    ``6 x active matmul parameters + 12 x heads x head_dim x mean attended positions`` summed over layers;
    rematerialisation is not counted."""
    q_dim, kv_dim = c.n_attn_heads * c.head_dim, c.n_kv_heads * c.head_dim
    attn = c.n_embd * q_dim + 2 * c.n_embd * kv_dim + q_dim * c.n_embd
    if c.use_sdpa_output_gate:
        attn += c.n_embd * c.n_attn_heads
    total = 0.0
    for idx, kind in enumerate(c.mlp_map):
        params = attn
        if kind == "moe":
            params += c.n_embd * c.n_routed_experts + c.n_active_experts * 3 * c.n_embd * c.expert_hidden
        else:
            params += 3 * c.n_embd * c.dense_hidden
        total += 6 * params
        window = c.layer_window(idx)
        T = c.seq_len
        if window and window < T:
            # mean over rows of min(row + 1, window)
            mean_pos = (window * (window + 1) / 2 + (T - window) * window) / T
        else:
            mean_pos = (T + 1) / 2
        total += 12 * c.n_attn_heads * c.head_dim * mean_pos
    total += 6 * c.n_embd * c.vocab_size
    return total


__all__ = [
    "Implementation", "MLPKind", "Mode", "ModelConfig", "PADDED_VOCAB_SIZE", "ShardingRules", "data_parallel",
    "expert_parallel", "flops_per_token", "full_moe", "interleaved_moe", "moe_outer_dense", "no_sharding", "replace",
    "tensor_parallel",
]
