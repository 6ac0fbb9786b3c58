"""Step functions: gradient-accumulating train step, validation, numerics and sampling steps
(lyra/training/steps.py:32-191), written for explicit streams instead of a tracing compiler.

Per step: each microbatch is copied host->device from pinned memory on a copy stream while the previous one
computes; forward + backward accumulate gradients; the runtime reduces them across ranks (fused with the
optimizer on the product path); the optimizer updates this rank's shards in place. The loss is the global
token mean: ``ce_sum / (A*B*T global) + aux / (A * data ranks)`` summed over microbatches and ranks."""

from __future__ import annotations

import math
from typing import Any, Iterator

import numpy as np
import torch

from lyra_b200.config import ModelConfig
from lyra_b200.model import ModelWeights, lm_head_weight, model_apply
from lyra_b200.nn.params import tree_dict
from lyra_b200.ops import api as ops
from lyra_b200.training.metrics import PPL_CE_CLAMP
from lyra_b200.training.optimizer import optimizer_step
from lyra_b200.training.probe import Probe, mean_over_ranks
from lyra_b200.training.state import TrainState
from lyra_b200.utils.nvtx import scope
from lyra_b200.utils.phases import span


def loss_parts(params: ModelWeights, x: torch.Tensor, y: torch.Tensor, config: ModelConfig, rt=None):
    """``(ce_sum, aux_loss)`` of one microbatch; the head is the fused linear cross-entropy (no logits tensor)."""
    with scope("loss"):
        B, T = x.shape
        h, aux, _ = model_apply(x, params, None, config, return_hidden_states=True, rt=rt)
        unemb = lm_head_weight(params.tok, config)
        if rt is not None:
            unemb = rt.materialize(unemb)
        ce_sum, _ = ops.linear_cross_entropy(h.reshape(B * T, -1), unemb, y.reshape(B * T), config.vocab_size, "sum", config.implementation)
    return ce_sum, aux


class Stepper:
    """Owns the device-side state of training: parameters (this rank's shards), optimizer state, streams."""

    def __init__(self, state: TrainState, mcfg: ModelConfig, tcfg, *, device, rt=None):
        self.state, self.mcfg, self.tcfg, self.rt, self.device = state, mcfg, tcfg, rt, torch.device(device)
        self.params = {p: t for p, t in tree_dict(state.params).items() if t.numel() > 0}  # placeholders of leaves owned by other ranks are skipped
        for p in self.params.values():
            if p.is_floating_point():
                p.requires_grad_(True)
                try:  # gradients may be kept in bf16 when fp32 ones do not fit (torch >= 2.9 checks the dtype)
                    p.grad_dtype = None
                except Exception:
                    pass
        self.world = rt.data_size if rt is not None else 1
        if rt is not None:
            rt.register(state.params)
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ host -> device
    def to_device(self, a) -> torch.Tensor:
        t = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))
        if t.is_cuda:
            return t
        if self.device.type != "cuda":
            return t.long() if t.dtype != torch.int64 else t
        if not t.is_pinned():
            t = t.pin_memory()
        self.h2d_bytes += t.numel() * t.element_size()
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.copy_stream):
            d = t.to(self.device, non_blocking=True)
        main.wait_stream(self.copy_stream)
        # The block belongs to the copy stream's pool but only the main stream reads it (embedding backward and the
        # cross-entropy backward read it last, long after the host has dropped its reference). Without this the allocator
        # would hand the block to the next staged microbatch while those kernels are still queued.
        d.record_stream(main)
        return d

    def _scales(self, A: int, B: int, T: int) -> tuple[float, float]:
        return 1.0 / (A * B * self.world * T), 1.0 / (A * self.world)

    # ------------------------------------------------------------------ train
    def train_step(self, xs, ys, step: int) -> dict[str, torch.Tensor]:
        """``xs, ys [A, B_local, T]`` int32 (host, preferably pinned). ``step`` is the 0-based schedule index."""
        A, B, T = xs.shape
        ce_scale, aux_scale = self._scales(A, B, T)
        totals = torch.zeros(3, dtype=torch.float32, device=self.device)
        with scope("gradient_accumulation"), span("forward_backward"):
            staged = [(self.to_device(xs[0]), self.to_device(ys[0]))]
            for a in range(A):
                x, y = staged[a]
                if a + 1 < A:  # next microbatch's copy overlaps this one's compute
                    staged.append((self.to_device(xs[a + 1]), self.to_device(ys[a + 1])))
                with scope("microbatch_forward_backward"):
                    if self.rt is not None:
                        self.rt.begin_microbatch(a, A)
                    ce_sum, aux = loss_parts(self.state.params, x, y, self.mcfg, self.rt)
                    ce_term, aux_term = ce_sum.float() * ce_scale, aux * aux_scale
                    loss = ce_term + aux_term
                    loss.backward()
                    totals += torch.stack([loss.detach(), ce_term.detach(), aux_term.detach()])
                staged[a] = None
        grads = {p: (t.grad if t.grad is not None else torch.zeros_like(t)) for p, t in self.params.items() if t.requires_grad}
        if self.rt is not None:
            with span("gradient_reduce"):
                totals = self.rt.sum_scalars(totals)
                grads = self.rt.reduce_grads(grads)
        with scope("optimizer"), span("optimizer"):
            trainable = {p: t for p, t in self.params.items() if p in grads}
            t = self.tcfg
            fused = (self.device.type == "cuda" and self.mcfg.implementation in ("auto", "b200")
                     and (self.rt is None or not self.rt.owns_optimizer)
                     # the fused kernels hard-code fp32 masters, bf16 first moments and an fp32 second moment; other choices take the PyTorch step
                     and self.mcfg.param_dtype == torch.float32 and t.muon_moment_dtype == torch.bfloat16
                     and t.adam_mu_dtype == torch.bfloat16 and t.adam_nu_dtype == torch.float32)
            if fused:
                from lyra_b200.ops import cuda_ops
                from lyra_b200.training.optimizer_cuda import optimizer_step_cuda

                shadows = {p: sh for p, t in trainable.items() if (sh := cuda_ops.shadow_of(t)) is not None}
                metrics = optimizer_step_cuda(trainable, grads, self.state.optimizer, step, self.tcfg, shadows, rt=self.rt)
                cuda_ops.weights_changed()               # masters and bf16 copies were rewritten through raw pointers
            else:
                metrics = optimizer_step({p: t.detach() for p, t in trainable.items()}, grads, self.state.optimizer, step, self.tcfg, rt=self.rt)
                if self.device.type == "cuda":
                    from lyra_b200.ops import cuda_ops

                    cuda_ops.invalidate_shadows()
        for t in self.params.values():
            t.grad = None
        if self.rt is not None:
            with span("weight_refresh"):
                self.rt.after_optimizer(self.params)
        return {"loss": totals[0], "ce_loss": totals[1], "aux_loss": totals[2], **metrics}

    # ------------------------------------------------------------------ validation / numerics
    @torch.no_grad()
    def validation_step(self, xs, ys) -> dict[str, torch.Tensor]:
        A, B, T = xs.shape
        ce_scale, aux_scale = self._scales(A, B, T)
        totals = torch.zeros(3, dtype=torch.float32, device=self.device)
        for a in range(A):
            ce_sum, aux = loss_parts(self.state.params, self.to_device(xs[a]), self.to_device(ys[a]), self.mcfg, self.rt)
            ce_term, aux_term = ce_sum.float() * ce_scale, aux * aux_scale
            totals += torch.stack([ce_term + aux_term, ce_term, aux_term])
        if self.rt is not None:
            totals = self.rt.sum_scalars(totals)
        return {"eval_loss": totals[0], "eval_ce_loss": totals[1], "eval_aux_loss": totals[2]}

    @torch.no_grad()
    def numerics_step(self, xs, probe: Probe) -> dict[str, dict[str, torch.Tensor]]:
        probe.start()
        model_apply(self.to_device(xs[0]), self.state.params, None, self.mcfg, return_hidden_states=True, probe=probe, rt=self.rt)
        return mean_over_ranks(probe.collect())


def run_validation(stepper: Stepper, batches: Iterator, *, eval_batches: int, microbatches: int) -> dict[str, Any]:
    totals: dict[str, Any] = {}
    for _ in range(eval_batches):
        xs, ys = zip(*(next(batches) for _ in range(microbatches)))
        for name, value in stepper.validation_step(np.stack(xs), np.stack(ys)).items():
            totals[name] = totals.get(name, 0.0) + value
    metrics = {name: value / eval_batches for name, value in totals.items()}
    metrics["eval_perplexity"] = math.exp(min(float(metrics["eval_ce_loss"]), PPL_CE_CLAMP))
    return metrics
