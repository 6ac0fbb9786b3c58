"""Model: parameter trees and the forward functions.

The family is the reference's (lyra/model.py): gated GQA with alternating local/global windows,
learned attention sinks, QK-norm, optional tanh XSA and SDPA output gate, clamped SwiGLU,
dense / mixture-of-experts interleave with routed + shared experts, fp32 masters with bf16 compute.
Leaf names and shapes equal the reference's so checkpoints describe the same tree; weights are
stored ``[in, out]``.

What differs is the execution: each block is a short chain of fused sm_100a kernels resolved through
``lyra_b200.ops.api`` (norm, GEMM with residual epilogue, QK-norm+RoPE, flash attention, gate+XSA,
router, grouped expert GEMMs with SwiGLU epilogue, combine), and sharded parameters are obtained
through a ``Runtime`` that gathers them layer by layer over NVLink instead of all at once.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace
from functools import lru_cache
from typing import Any

import numpy as np
import torch

from lyra_b200.config import Mode, ModelConfig
from lyra_b200.nn.params import ArraySpec, Tag, init_weights, map_with_path
from lyra_b200.nn.quant import QArray, dequantize, quantize, qupdate
from lyra_b200.ops import api as ops
from lyra_b200.ops import reference as ref_ops
from lyra_b200.training.probe import NO_PROBE, Probe
from lyra_b200.utils.nvtx import scope

Param = Any  # torch.Tensor | ArraySpec | QArray | None


# --------------------------------------------------------------------------- spec helpers
def _matrix(c: ModelConfig, shape, kind: str, init: str | None = None) -> ArraySpec:
    return ArraySpec(tuple(shape), c.param_dtype, kind, init or c.w_init, Tag.MATRIX)


def _bias(c: ModelConfig, shape, kind: str, enabled: bool) -> ArraySpec | None:
    return ArraySpec(tuple(shape), c.param_dtype, kind, c.b_init, Tag.BIAS) if enabled else None


def _scalar(shape, kind: str, init: str) -> ArraySpec:
    return ArraySpec(tuple(shape), torch.float32, kind, init, Tag.SCALAR)


def _quantize_block(value: torch.Tensor, c: ModelConfig) -> QArray:
    k, n = c.quant_block
    return quantize(value, c.gemm_dtype, (math.gcd(value.shape[-2], k), math.gcd(value.shape[-1], n)))


# --------------------------------------------------------------------------- RoPE
@lru_cache(maxsize=8)
def precompute_freq_cis(config: ModelConfig) -> tuple[np.ndarray, np.ndarray]:
    """cos/sin tables ``[seq_len * rope_scale, head_dim/2]`` in fp32, computed in fp64 on the host with
    YaRN / NTK-by-parts when ``rope_scale > 1`` (lyra/model.py:160-180)."""
    c = config
    positions = np.arange(int(c.seq_len * c.rope_scale), dtype=np.float64)
    inv_freq = 1.0 / (c.rope_base ** (np.arange(0, c.head_dim, 2, dtype=np.float64) / c.head_dim))
    concentration = 1.0
    if c.rope_scale > 1.0:
        concentration = 0.1 * math.log(c.rope_scale) + 1.0
        dim_half = c.head_dim / 2.0
        log_base = math.log(c.rope_base) ** -1.0
        low = dim_half * math.log(c.seq_len / (c.ntk_beta * 2.0 * math.pi)) * log_base
        high = dim_half * math.log(c.seq_len / (c.ntk_alpha * 2.0 * math.pi)) * log_base
        ramp = 1.0 - np.clip((np.arange(int(dim_half), dtype=np.float64) - low) / (high - low), 0.0, 1.0)
        inv_freq = (1.0 - ramp) * (inv_freq / c.rope_scale) + ramp * inv_freq
    angles = np.einsum("i,j->ij", positions, inv_freq)
    return (np.cos(angles) * concentration).astype(np.float32), (np.sin(angles) * concentration).astype(np.float32)


_ROPE_DEVICE_CACHE: dict = {}


def rope_tables(config: ModelConfig, device) -> tuple[torch.Tensor, torch.Tensor]:
    key = (config, str(device))
    if key not in _ROPE_DEVICE_CACHE:
        cos, sin = precompute_freq_cis(config)
        _ROPE_DEVICE_CACHE[key] = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
    return _ROPE_DEVICE_CACHE[key]


# --------------------------------------------------------------------------- KV cache
@dataclass
class LayerCache:
    k: Any  # [B, Nkv, S, D] tensor or QArray
    v: Any


def _kv_append_kernel(cache: LayerCache, k: torch.Tensor, v: torch.Tensor, pos_dev: torch.Tensor) -> bool:
    """One launch that writes the new position of both caches (and their scales) at the device-resident position; False when
    the tensors are not what the kernel takes (then the PyTorch path below runs)."""
    from lyra_b200.ops import native

    quantised = isinstance(cache.k, QArray)
    kc, vc = (cache.k.qval, cache.v.qval) if quantised else (cache.k, cache.v)
    B, Nkv, T, D = k.shape
    if not (k.is_cuda and T == 1 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and native.kernels_available()
            and hasattr(native.kernels(), "lyra_kv_append") and kc.is_contiguous() and vc.is_contiguous() and kc.shape[:2] == (B, Nkv) and kc.shape[3] == D
            and k.stride(3) == 1 and v.stride(3) == 1 and v.shape == k.shape and pos_dev.dtype == torch.int32):
        return False
    if quantised:
        if not (kc.dtype == torch.float8_e4m3fn and tuple(cache.k.block) == (1, D) and cache.k.scale.dtype == torch.float32
                and cache.k.scale.is_contiguous() and cache.v.scale.is_contiguous()):
            return False
        ks, vs = cache.k.scale, cache.v.scale
    else:
        if kc.dtype != torch.bfloat16:
            return False
        ks = vs = None
    native.check(native.kernels().lyra_kv_append(native.ptr(k), native.ptr(v), native.c_ll(k.stride(0)), native.c_ll(k.stride(1)), native.c_ll(v.stride(0)), native.c_ll(v.stride(1)), native.ptr(kc), native.ptr(vc),
                                                 native.ptr(ks), native.ptr(vs), native.c_int(B), native.c_int(Nkv), native.c_int(kc.shape[2]), native.c_int(D),
                                                 native.ptr(pos_dev), native.c_int(int(quantised)), native.stream_ptr()), "lyra_kv_append")
    native.count_launch()
    return True


def cache_update(cache: LayerCache, k: torch.Tensor, v: torch.Tensor, start_pos: int, pos_dev: torch.Tensor | None = None) -> LayerCache:
    """Writes ``k, v [B, Nkv, T, D]`` at ``start_pos`` (in place). fp8 caches quantise per (position, head).
    With ``pos_dev`` (int device scalar, T == 1) the position is read on the device, so the call can be replayed."""
    if pos_dev is not None:
        if _kv_append_kernel(cache, k, v, pos_dev):
            return cache
        at = pos_dev.reshape(1).long()
        if isinstance(cache.k, QArray):
            for dst, new in ((cache.k, k), (cache.v, v)):
                qn = quantize(new.contiguous(), dst.dtype, dst.block, dst.stype)
                dst.qval.view(torch.uint8).index_copy_(2, at, qn.qval.view(torch.uint8))   # index_copy_ has no fp8 kernel
                dst.scale.index_copy_(2, at, qn.scale)
            return cache
        cache.k.index_copy_(2, at, k.to(cache.k.dtype))
        cache.v.index_copy_(2, at, v.to(cache.v.dtype))
        return cache
    if isinstance(cache.k, QArray):
        start = (0, 0, int(start_pos), 0)
        return LayerCache(k=qupdate(cache.k, k, start), v=qupdate(cache.v, v, start))
    T = k.shape[2]
    cache.k[:, :, start_pos:start_pos + T] = k.to(cache.k.dtype)
    cache.v[:, :, start_pos:start_pos + T] = v.to(cache.v.dtype)
    return cache


@dataclass
class ModelCache:
    layers: tuple[LayerCache, ...]
    pos: int
    pos_dev: Any = None  # optional int32 device scalar mirroring ``pos``: single-token decode then reads the position on the device

    @staticmethod
    def create(config: ModelConfig, batch: int, capacity: int, device, n_kv_local: int | None = None) -> "ModelCache":
        n_kv = n_kv_local or config.n_kv_heads
        shape = (batch, n_kv, capacity, config.head_dim)
        mk = lambda: torch.zeros(shape, dtype=config.compute_dtype, device=device)
        cache = ModelCache(layers=tuple(LayerCache(k=mk(), v=mk()) for _ in range(config.n_layers)), pos=0)
        return ModelCache.quantize(cache, config)

    @staticmethod
    def quantize(cache: "ModelCache", config: ModelConfig) -> "ModelCache":
        """fp8 cache with one scale per (sequence, kv head, position): block ``(1, head_dim)`` (lyra/model.py:221-226)."""
        if not config.quantize_cache:
            return cache
        dt = config.gemm_dtype if config.gemm_dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else torch.float8_e4m3fn
        q = lambda a: a if isinstance(a, QArray) else quantize(a, dt, block=(1, config.head_dim))
        return ModelCache(layers=tuple(LayerCache(k=q(l.k), v=q(l.v)) for l in cache.layers), pos=cache.pos)


# --------------------------------------------------------------------------- attention
@dataclass
class AttentionWeights:
    q: Param
    k: Param
    v: Param
    out: Param
    q_bias: Param
    k_bias: Param
    v_bias: Param
    out_bias: Param
    sinks: Param
    norm_scale: Param
    qnorm_scale: Param
    knorm_scale: Param
    xsa_alpha: Param
    sdpa_gate: Param

    @classmethod
    def spec(cls, c: ModelConfig) -> "AttentionWeights":
        q_dim, kv_dim = c.n_attn_heads * c.head_dim, c.n_kv_heads * c.head_dim
        return cls(
            q=_matrix(c, (c.n_embd, q_dim), "attn_q"),
            q_bias=_bias(c, (q_dim,), "attn_qkv_bias", c.use_qkv_bias),
            k=_matrix(c, (c.n_embd, kv_dim), "attn_kv"),
            k_bias=_bias(c, (kv_dim,), "attn_qkv_bias", c.use_qkv_bias),
            v=_matrix(c, (c.n_embd, kv_dim), "attn_kv"),
            v_bias=_bias(c, (kv_dim,), "attn_qkv_bias", c.use_qkv_bias),
            sinks=_scalar((c.n_attn_heads,), "attn_sink", c.b_init),
            out=_matrix(c, (q_dim, c.n_embd), "attn_out"),
            out_bias=_bias(c, (c.n_embd,), "attn_out_bias", c.use_attn_out_bias),
            norm_scale=_scalar((c.n_embd,), "norm_scale", c.norm_init),
            qnorm_scale=_scalar((c.head_dim,), "norm_scale", c.norm_init) if c.use_qk_norm else None,
            knorm_scale=_scalar((c.head_dim,), "norm_scale", c.norm_init) if c.use_qk_norm else None,
            xsa_alpha=_scalar((c.n_attn_heads,), "attn_sink", c.b_init) if c.use_learned_xsa else None,
            # zero-init: 2 * sigmoid(0) = 1, the gate starts as the identity
            sdpa_gate=ArraySpec((c.n_embd, c.n_attn_heads), torch.float32, "attn_q", "zeros", Tag.DEFAULT)
            if c.use_sdpa_output_gate else None,
        )

    @staticmethod
    def quantize(w: "AttentionWeights", c: ModelConfig) -> "AttentionWeights":
        if not c.quantize_attn:
            return w
        q = lambda x: x if isinstance(x, QArray) else _quantize_block(x, c)
        return replace(w, q=q(w.q), k=q(w.k), v=q(w.v), out=q(w.out))


def _dq(w, dtype):
    return dequantize(w, dtype) if isinstance(w, QArray) else w


def attention_apply(x, w: AttentionWeights, idx: int, pos: int, freq_cis, cache: LayerCache | None, config: ModelConfig,
                    *, probe: Probe = NO_PROBE, rt=None, pos_dev=None):
    """Pre-norm attention block with residual (lyra/model.py:285-374). ``x [B, T, C]`` in the compute dtype."""
    c = config
    impl = c.implementation
    B, T, C = x.shape
    W = (lambda p, kind=None: rt.materialize(p) if rt is not None else p)
    with scope("attention"):
        h = ops.rms_norm(x, W(w.norm_scale), c.norm_eps, impl)
        probe.tensor("norm_out", h)
        if rt is not None and rt.tp_size > 1:
            h = rt.tp_copy(h)                                # q / k / v and the gate are column-sharded: their input gradients are partial
        with scope("qkv_projection"):
            wq, wk, wv = W(w.q), W(w.k), W(w.v)
            if (c.mode == Mode.DECODE and T == 1 and not probe.enabled and not torch.is_grad_enabled() and (rt is None or rt.tp_size == 1)
                    and ops.use_kernels(h, impl) and all(isinstance(t, torch.Tensor) and t.ndim == 2 for t in (wq, wk, wv))
                    and not ops._cuda().pull_pending(wq, wk, wv)):
                # a decode step: one product with the fused [C, q | k | v] matrix (two launches instead of six)
                fused, fused_bias = ops._cuda().fused_columns((wq, wk, wv), (W(w.q_bias), W(w.k_bias), W(w.v_bias)))
                qkv = ops.linear(h, fused, fused_bias, impl)
                q, k, v = (t.reshape(B, T, -1, c.head_dim) for t in qkv.split([wq.shape[1], wk.shape[1], wv.shape[1]], dim=-1))
                if w.sdpa_gate is not None or c.use_learned_xsa:
                    v = v.contiguous()                       # the gate / XSA kernel reads the values as a tensor of their own
            else:
                q = ops.linear(h, _dq(wq, h.dtype), W(w.q_bias), impl).reshape(B, T, -1, c.head_dim)
                k = ops.linear(h, _dq(wk, h.dtype), W(w.k_bias), impl).reshape(B, T, -1, c.head_dim)
                v = ops.linear(h, _dq(wv, h.dtype), W(w.v_bias), impl).reshape(B, T, -1, c.head_dim)
        if probe.enabled and w.qnorm_scale is not None:
            probe.tensor("q_pre_norm", q)
            probe.tensor("k_pre_norm", k)
        with scope("qknorm_rope"):
            cos, sin = freq_cis
            q, k = ops.qk_norm_rope(q, k, W(w.qnorm_scale), W(w.knorm_scale), cos, sin, c.norm_eps, impl)
        probe.tensor("q", q)
        probe.tensor("k", k)
        probe.tensor("v", v)

        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)  # heads first
        sinks = W(w.sinks)
        current_v = v
        updated_cache = None
        window = c.layer_window(idx)
        probe.tensor("sinks", sinks)
        with scope("attention_kernel"):
            if c.mode == Mode.NOCACHE:
                t = ops.attention(q, k, v, sinks, c.head_dim**-0.5, window, 0, impl)
            else:
                assert cache is not None
                updated_cache = cache_update(cache, k, v, pos, pos_dev)
                if c.mode == Mode.DECODE:
                    t = ops.decode_attention(q, updated_cache.k, updated_cache.v, sinks, c.head_dim**-0.5, window, pos, impl, pos_dev=pos_dev)
                else:
                    t = ops.attention(q, k, v, sinks, c.head_dim**-0.5, window, pos, impl) if pos == 0 else \
                        ops.decode_attention(q, updated_cache.k, updated_cache.v, sinks, c.head_dim**-0.5, window, pos, impl)
        probe.tensor("attn_out", t)

        if w.sdpa_gate is not None or c.use_learned_xsa:
            with scope("gate_xsa"):
                t = ops.gate_xsa(t, h, W(w.sdpa_gate), current_v, W(w.xsa_alpha) if c.use_learned_xsa else None, impl)
            if probe.enabled and w.sdpa_gate is not None:
                gate = 2.0 * torch.sigmoid(h.float() @ W(w.sdpa_gate).float())
                probe.scalars("sdpa_gate", {"mean": gate.mean(), "std": gate.std(unbiased=False)})
            if c.use_learned_xsa:
                probe.tensor("xsa_out", t)

        with scope("output_projection"):
            t = t.transpose(1, 2).reshape(B, T, -1)
            if probe.enabled or (rt is not None and rt.tp_size > 1):
                t = ops.linear(t, _dq(W(w.out), t.dtype), None, impl)
                if rt is not None:
                    t = rt.tp_all_reduce(t)
                if w.out_bias is not None:
                    t = t + W(w.out_bias).to(t.dtype)
                probe.tensor("out_proj", t)
                t = t * c.residual_scale
                probe.residual("residual", x, t)
                out = (x + t).to(x.dtype)
            else:
                # residual add and 1/sqrt(2L) scale ride in the GEMM epilogue
                out = ops.linear(t, _dq(W(w.out), t.dtype), W(w.out_bias), impl, residual=x, alpha=c.residual_scale)
    return out, updated_cache


# --------------------------------------------------------------------------- MoE
@dataclass
class MoEWeights:
    router: Param
    router_bias: Param
    mlp_up: Param
    mlp_up_bias: Param
    mlp_down: Param
    mlp_down_bias: Param
    norm_scale: Param

    @classmethod
    def spec(cls, c: ModelConfig) -> "MoEWeights":
        hidden = c.expert_hidden
        return cls(
            router=ArraySpec((c.n_embd, c.n_routed_experts), torch.float32, "router", "fan_in_trunc", Tag.DEFAULT,
                             init_scale=c.router_logit_std**2),
            router_bias=ArraySpec((c.n_routed_experts,), torch.float32, "router_bias", c.b_init, Tag.BIAS)
            if c.use_router_bias else None,
            mlp_up=_matrix(c, (c.n_experts, c.n_embd, 2, hidden), "moe_mlp_up"),
            mlp_up_bias=_bias(c, (c.n_experts, 2, hidden), "moe_mlp_up_bias", c.use_mlp_bias),
            mlp_down=_matrix(c, (c.n_experts, hidden, c.n_embd), "moe_mlp_down"),
            mlp_down_bias=_bias(c, (c.n_experts, c.n_embd), "moe_mlp_down_bias", c.use_mlp_bias),
            norm_scale=_scalar((c.n_embd,), "norm_scale", c.norm_init),
        )

    @staticmethod
    def quantize(w: "MoEWeights", c: ModelConfig) -> "MoEWeights":
        if not c.quantize_mlp:
            return w
        up, down = w.mlp_up, w.mlp_down
        if not isinstance(up, QArray):
            up = _quantize_block(up.reshape(*up.shape[:-2], -1), c)
        if not isinstance(down, QArray):
            down = _quantize_block(down, c)
        return replace(w, mlp_up=up, mlp_down=down)


def calculate_aux_loss(router_logits, expert_indices, config: ModelConfig, *, probe: Probe = NO_PROBE):
    """Switch load-balance term + router z-loss on the local tokens (lyra/model.py:418-448)."""
    F_, E = router_logits.shape
    K = expert_indices.shape[-1]
    logits = router_logits.float()
    counts = ref_ops.count_ids(expert_indices, E).float()
    assigned = torch.softmax(logits, dim=-1).sum(0) / F_
    assignments = (counts / (F_ * K)).detach()
    lb_term = E * (assigned * assignments).sum()
    z_term = torch.logsumexp(logits, dim=-1).square().mean()
    lb_loss, z_loss = config.load_balance_weight * lb_term, config.router_z_loss_weight * z_term
    aux = lb_loss + z_loss
    if probe.enabled:
        mean_count = counts.mean().clamp_min(1.0)
        probe.scalars("aux_loss", {
            "lb_term": lb_term, "lb_loss": lb_loss, "z_term": z_term, "z_loss": z_loss, "aux_loss": aux,
            "load_cv": counts.std(unbiased=False) / mean_count, "max_load_violation": counts.max() / mean_count - 1.0,
            "min_expert_count": counts.min(), "max_expert_count": counts.max(),
        })
    return aux.float()


ROUTING_TAPE: dict | None = None
"""Numerics tests that compare two implementations of the model set this to ``{"replay": False, "choices": []}`` for the first
run (the experts chosen by every MoE layer call are recorded) and flip ``replay`` for the second, which then takes the recorded
experts instead of its own top-k: near-tie choices that flip between two bf16 paths no longer blur the comparison."""


def route_tokens(t, w: MoEWeights, config: ModelConfig, *, probe: Probe = NO_PROBE, rt=None, plan_out: list | None = None):
    """fp32 router, top-k over routed experts, softmax over the selected logits, shared experts appended
    with score 1 (lyra/model.py:451-480). Returns ``(scores [F, K], indices [F, K], aux_loss)``. When the routing kernels
    ran, their ``RoutingPlan`` (counts, offsets and the expert-sorted order of the routed choices) is appended to ``plan_out``."""
    c = config
    W = (lambda p: rt.materialize(p) if rt is not None else p)
    k = c.n_active_routed_experts
    with scope("router"):
        kernels = ops.use_kernels(t, c.implementation)
        f32 = ops._cuda().fp32_param if kernels else (lambda p: p.float())       # cached conversion of a bf16 checkpoint's router
        logits = t.float() @ f32(W(w.router))
        if (ROUTING_TAPE is None and not probe.enabled and kernels and (rt is None or rt.tp_size == 1)):
            from lyra_b200.ops import routing

            if routing.supported(c.n_routed_experts, k):
                # one kernel chain: top-k, scores, both auxiliary terms, counts and the expert-sorted permutation
                scores, idx, aux, plan = routing.route(logits, f32(W(w.router_bias)) if w.router_bias is not None else None, k,
                                                       c.load_balance_weight, c.router_z_loss_weight)
                meter = getattr(rt, "load_meter", None)
                if meter is not None and (meter.always or torch.is_grad_enabled()):
                    meter.add_counts(rt._layer, plan.counts)
                if rt is not None:
                    rt.routing_plan = plan                   # picked up by the expert exchange of this layer call
                if plan_out is not None:
                    plan_out.append(plan)
                if c.n_shared_experts:
                    shared = torch.arange(c.n_routed_experts, c.n_experts, device=idx.device, dtype=idx.dtype)
                    idx = torch.cat([idx, shared[None].expand(t.shape[0], -1)], dim=-1)
                    scores = torch.cat([scores, scores.new_ones(t.shape[0], c.n_shared_experts)], dim=-1)
                return scores, idx, aux
        if w.router_bias is not None:
            logits = logits + W(w.router_bias).float()
    if rt is not None:
        rt.routing_plan = None
    if ROUTING_TAPE is not None and ROUTING_TAPE["replay"]:
        idx = ROUTING_TAPE["choices"].pop(0)
        vals = torch.gather(logits, -1, idx)
    else:
        vals, idx = torch.topk(logits, k, dim=-1)  # ties -> lower index first, like lax.top_k
        if ROUTING_TAPE is not None:
            ROUTING_TAPE["choices"].append(idx)
    scores = torch.softmax(vals, dim=-1)
    aux = calculate_aux_loss(logits, idx, c, probe=probe)
    meter = getattr(rt, "load_meter", None)
    if meter is not None and (meter.always or torch.is_grad_enabled()):   # training forwards (or every call of a serving process)
        meter.add(rt._layer, idx)
    if probe.enabled:
        probe.routing("routing", router_logits=logits, expert_scores=scores,
                      group_sizes=ref_ops.count_ids(idx, c.n_routed_experts),
                      n_experts=c.n_routed_experts, n_active=k)
    if c.n_shared_experts:
        shared = torch.arange(c.n_routed_experts, c.n_experts, device=idx.device, dtype=idx.dtype)
        idx = torch.cat([idx, shared[None].expand(t.shape[0], -1)], dim=-1)
        scores = torch.cat([scores, scores.new_ones(t.shape[0], c.n_shared_experts)], dim=-1)
    return scores, idx, aux


def bpermute(expert_ids: torch.Tensor, n_experts: int):
    """Stable counting-sort permutation (lyra/model.py:483-491): ``permutation[dst] = assignment`` and
    ``destinations[assignment] = dst`` with ``dst = group_offset[e] + rank within expert in token order``."""
    permutation = torch.argsort(expert_ids, stable=True)
    destinations = torch.empty_like(permutation)
    destinations[permutation] = torch.arange(expert_ids.numel(), device=expert_ids.device)
    return permutation, destinations


def moe_apply(x, w: MoEWeights, config: ModelConfig, *, probe: Probe = NO_PROBE, rt=None):
    """Pre-norm mixture-of-experts block with residual; returns ``(x + branch, aux_loss)`` (lyra/model.py:498-567).

    On one rank the shared expert is simply expert ``n_routed`` of the grouped GEMM. Under expert parallelism the
    routed experts go through the fused dispatch/combine path and the shared expert runs as an FSDP-sharded dense
    MLP on the local tokens (no per-call weight broadcast)."""
    c = config
    impl = c.implementation
    B, T, C = x.shape
    W = (lambda p: rt.materialize(p) if rt is not None else p)
    with scope("moe"):
        xn = ops.rms_norm(x, W(w.norm_scale), c.norm_eps, impl)
        probe.tensor("norm_out", xn)
        xn = xn.reshape(B * T, C)
        with scope("route_tokens"):
            plans: list = []
            scores, indices, aux = route_tokens(xn, w, c, probe=probe, rt=rt, plan_out=plans)
        tp = rt.tp_size if rt is not None else 1
        # tensor parallel: every rank holds a slice of each expert's hidden units; the partial outputs are summed below, so the
        # (replicated) down-projection bias enters as bias / tp on every rank (lyra/model.py:549)
        down_bias = w.mlp_down_bias / tp if (tp > 1 and w.mlp_down_bias is not None) else w.mlp_down_bias
        if tp > 1:                                           # the experts' hidden units are split: gradients of their inputs are partial
            xn, scores = rt.tp_copy(xn), rt.tp_copy(scores)
        if rt is not None and rt.ep_size > 1:
            t = rt.ep_moe(xn, scores, indices, w, c)
        elif c.mode == Mode.DECODE and ops.use_kernels(xn, impl) and not xn.requires_grad:
            t = ops._cuda().decode_moe(xn, scores, indices, w.mlp_up, w.mlp_up_bias, w.mlp_down, down_bias,
                                       c.swiglu_beta, c.swiglu_limit, plans[0] if plans and not c.n_shared_experts else None)
        else:
            up, down = w.mlp_up, w.mlp_down
            if isinstance(up, QArray):
                up = dequantize(up, xn.dtype).reshape(c.n_experts, C, 2, -1)
            if isinstance(down, QArray):
                down = dequantize(down, xn.dtype)
            with scope("experts"):
                t = ops.moe_experts(xn, scores, indices, up, w.mlp_up_bias, down, down_bias,
                                    c.swiglu_beta, c.swiglu_limit, impl)
        if tp > 1:
            t = rt.tp_all_reduce(t)
        t = t.reshape(B, T, C).to(x.dtype)
        probe.tensor("combined", t)
        t = t * c.residual_scale
        probe.residual("residual", x, t)
        return x + t, aux


# --------------------------------------------------------------------------- dense MLP
@dataclass
class DenseMLPWeights:
    mlp_up: Param
    mlp_up_bias: Param
    mlp_down: Param
    mlp_down_bias: Param
    norm_scale: Param

    @classmethod
    def spec(cls, c: ModelConfig) -> "DenseMLPWeights":
        hidden = c.dense_hidden
        return cls(
            mlp_up=_matrix(c, (c.n_embd, 2, hidden), "dense_mlp_up"),
            mlp_up_bias=_bias(c, (1, 2, hidden), "dense_mlp_up_bias", c.use_mlp_bias),
            mlp_down=_matrix(c, (hidden, c.n_embd), "dense_mlp_down"),
            mlp_down_bias=_bias(c, (1, c.n_embd), "dense_mlp_down_bias", c.use_mlp_bias),
            norm_scale=_scalar((c.n_embd,), "norm_scale", c.norm_init),
        )

    @staticmethod
    def quantize(w: "DenseMLPWeights", c: ModelConfig) -> "DenseMLPWeights":
        if not c.quantize_mlp:
            return w
        up, down = w.mlp_up, w.mlp_down
        if not isinstance(up, QArray) and up.numel() == 0:
            raise ValueError("this rank holds only a placeholder of a dense MLP leaf (another rank owns it): quantised serving under the "
                             "leaf-ownership runtime needs a model whose MLPs are all mixtures of experts, or tensor parallelism")
        if not isinstance(up, QArray):
            k, n = c.quant_block
            up = quantize(up, c.gemm_dtype, (math.gcd(up.shape[-3], k), 1, math.gcd(up.shape[-1], n)))
        if not isinstance(down, QArray):
            down = _quantize_block(down, c)
        return replace(w, mlp_up=up, mlp_down=down)


def dense_mlp_apply(x, w: DenseMLPWeights, config: ModelConfig, *, probe: Probe = NO_PROBE, rt=None):
    """norm -> up-projection + SwiGLU -> down-projection (+ residual, scaled) (lyra/model.py:609-636)."""
    c = config
    impl = c.implementation
    W = (lambda p: rt.materialize(p) if rt is not None else p)
    with scope("dense_mlp"):
        t = ops.rms_norm(x, W(w.norm_scale), c.norm_eps, impl)
        probe.tensor("norm_out", t)
        if rt is not None and rt.tp_size > 1:
            t = rt.tp_copy(t)
        up = _dq(W(w.mlp_up), t.dtype)
        if probe.detailed:
            C, _, H = up.shape
            pre = t @ up.reshape(C, 2 * H).to(t.dtype)
            probe.tensor("up_out", pre)
            probe.swiglu("swiglu", pre, limit=c.swiglu_limit)
        with scope("up_swiglu"):
            t = ops.linear_swiglu(t, up, W(w.mlp_up_bias), c.swiglu_beta, c.swiglu_limit, impl)
        probe.tensor("act_out", t)
        with scope("down_projection"):
            down = _dq(W(w.mlp_down), t.dtype)
            bias = W(w.mlp_down_bias)
            bias = bias.reshape(-1) if bias is not None else None
            if probe.enabled or (rt is not None and rt.tp_size > 1):
                t = ops.linear(t, down, None, impl)
                if rt is not None:
                    t = rt.tp_all_reduce(t)
                if bias is not None:
                    t = t + bias.to(t.dtype)
                probe.tensor("down_out", t)
                t = t * c.dense_residual_scale
                probe.residual("residual", x, t)
                return (x + t).to(x.dtype)
            return ops.linear(t, down, bias, impl, residual=x, alpha=c.dense_residual_scale)


def mlp_apply(x, w, config: ModelConfig, *, probe: Probe = NO_PROBE, rt=None):
    if isinstance(w, MoEWeights):
        return moe_apply(x, w, config, probe=probe, rt=rt)
    return dense_mlp_apply(x, w, config, probe=probe, rt=rt), x.new_zeros((), dtype=torch.float32)


# --------------------------------------------------------------------------- model
@dataclass
class TokenEmbeddings:
    emb: Param
    unemb: Param
    norm_scale: Param

    @classmethod
    def spec(cls, c: ModelConfig) -> "TokenEmbeddings":
        shape = (c.padded_vocab_size, c.n_embd)
        return cls(
            emb=ArraySpec(shape, c.param_dtype, "emb", "emb", Tag.EMBEDDING),
            unemb=None if c.tie_embeddings else ArraySpec(shape, c.param_dtype, "unemb", "emb", Tag.EMBEDDING),
            norm_scale=_scalar((c.n_embd,), "norm_scale", c.norm_init),
        )


def lm_head_weight(tok: TokenEmbeddings, config: ModelConfig):
    return tok.emb if config.tie_embeddings else tok.unemb


@dataclass
class LayerWeights:
    attn: AttentionWeights
    mlp: Any

    @classmethod
    def spec(cls, idx: int, c: ModelConfig) -> "LayerWeights":
        mlp = MoEWeights.spec(c) if c.mlp_map[idx] == "moe" else DenseMLPWeights.spec(c)
        return cls(attn=AttentionWeights.spec(c), mlp=mlp)


@dataclass
class ModelWeights:
    tok: TokenEmbeddings
    layers: list

    @classmethod
    def spec(cls, c: ModelConfig) -> "ModelWeights":
        return cls(tok=TokenEmbeddings.spec(c), layers=[LayerWeights.spec(i, c) for i in range(c.n_layers)])

    @classmethod
    def init(cls, seed: int, c: ModelConfig, device="cpu", shard_fn=None) -> "ModelWeights":
        """Random initialisation (lyra/model.py:96-99,133-151; variance 1/fan_in truncated normal for matrices,
        ``0.5/sqrt(C)`` router, 1/C embeddings, zeros for biases/sinks/xsa/gate, ones for norms). Each leaf has its
        own random stream keyed by its path, so the gate being present changes no other initial value."""
        return init_weights(cls.spec(c), seed, device, shard_fn)

    @classmethod
    def load(cls, source, c: ModelConfig, device="cpu", rt=None) -> "ModelWeights":
        from lyra_b200.nn.checkpoints import load_checkpointables, resolve_checkpoint

        return load_checkpointables(resolve_checkpoint(source), {"params": cls.spec(c)}, device=device, rt=rt)["params"]

    @staticmethod
    def quantize(w: "ModelWeights", c: ModelConfig) -> "ModelWeights":
        mlp = lambda m: MoEWeights.quantize(m, c) if isinstance(m, MoEWeights) else DenseMLPWeights.quantize(m, c)
        return ModelWeights(tok=w.tok, layers=[LayerWeights(attn=AttentionWeights.quantize(l.attn, c), mlp=mlp(l.mlp)) for l in w.layers])

    def to(self, device) -> "ModelWeights":
        return map_with_path(lambda _, t: t.to(device), self)


def model_apply(tokens, model: ModelWeights, cache: ModelCache | None, config: ModelConfig, *,
                return_hidden_states: bool = False, probe: Probe = NO_PROBE, rt=None):
    """Forward pass (lyra/model.py:734-793). Returns ``(logits | hidden, aux_loss, cache)``; with
    ``return_hidden_states`` the final-normed hidden states are returned and logits are never materialised."""
    c = config
    impl = c.implementation
    T = tokens.shape[1]
    W = (lambda p: rt.materialize(p) if rt is not None else p)
    with scope("model"):
        with scope("token_embedding"):
            h = ops.embedding(W(model.tok.emb), tokens, impl, c.use_presorted_emb_gather).to(c.compute_dtype)
        probe.tensor("embs", h)
        start_pos = cache.pos if cache is not None else 0
        cos, sin = rope_tables(c, h.device)
        pos_dev = cache.pos_dev if (cache is not None and c.mode == Mode.DECODE and T == 1) else None
        if pos_dev is not None:
            at = pos_dev.reshape(1).long()
            freq_cis = (cos.index_select(0, at)[None, :, None, :], sin.index_select(0, at)[None, :, None, :])
        else:
            freq_cis = (cos[start_pos:start_pos + T][None, :, None, :], sin[start_pos:start_pos + T][None, :, None, :])

        aux_loss = torch.zeros((), dtype=torch.float32, device=h.device)
        caches = []
        for idx, layer in enumerate(model.layers):
            lp = probe.scope(f"layer.{idx:02d}")
            with scope(f"layer_{idx:02d}"):
                if rt is not None:
                    rt.begin_layer(idx)
                lc = cache.layers[idx] if cache is not None else None
                h, lc = attention_apply(h, layer.attn, idx, start_pos, freq_cis, lc, c, probe=lp.scope("attn"), rt=rt, pos_dev=pos_dev)
                h, layer_aux = mlp_apply(h, layer.mlp, c, probe=lp.scope("mlp"), rt=rt)
            aux_loss = aux_loss + layer_aux
            caches.append(lc)
        if c.n_moe_layers:
            aux_loss = aux_loss / c.n_moe_layers
        updated = None if cache is None else ModelCache(layers=tuple(caches), pos=start_pos + T, pos_dev=cache.pos_dev)

        head = probe.scope("head")
        head.tensor("pre_norm", h)
        with scope("output_norm"):
            h = ops.rms_norm(h, W(model.tok.norm_scale), c.norm_eps, impl)
        head.tensor("norm_out", h)
        unemb = W(lm_head_weight(model.tok, c))
        if return_hidden_states:
            head.logit_subsample("logits_subsample", h, unemb, vocab_size=c.vocab_size)
            return h, aux_loss, updated
        logits = (h @ unemb.to(c.compute_dtype).t()).float()
        logits[..., c.vocab_size:] = float("-inf")
        head.logits("logits", logits)
        return logits, aux_loss, updated
