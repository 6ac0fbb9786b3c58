"""Headline benchmark: lyra-medium pretraining step, tokens/s and MFU on N B200s of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 3 --warmup 3
    python bench.py --impl reference ...        # the unmodified reference, when it can be installed

Workload (weak scaling): every GPU runs `accumulation_steps` microbatches of 2 x 4096 synthetic tokens per optimizer
step (the reference's train-medium preset accumulates 8 microbatches; lyra/training/presets.py:31), iid-uniform
token ids over the 201,088-token vocabulary from a fixed seed, random-init fp32 master weights, bf16 compute, Muon +
Adam update inside the timed region. `value` is whole-job tokens/s, device-timed with CUDA events, max over ranks.
The `e2e` figure runs the same steps through the public `Stepper.train_step` API with inputs copied from pinned host
memory every microbatch and the loss read back to the host every step.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from dataclasses import replace
from pathlib import Path

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("LYRA_LOG_KERNELS", "0")
# kernels are loaded when the library is, not at their first launch: a first launch that has to load code can stall the host while
# this rank's peers already spin in (bounded) waits for it
os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BASELINE_TOKENS_PER_S = 34150.0  # reference's published headline: lyra-small on one TPU v6e (README.md:33); nothing is published for lyra-medium


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "torch", "nccl"])
    ap.add_argument("--variant", default="lyra-medium")
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--accumulation", type=int, default=None)
    ap.add_argument("--rebalance-experts", action=argparse.BooleanOptionalAction, default=True,
                    help="several GPUs: meter the experts' token counts during warm-up and re-place the experts on the ranks once before the "
                         "timed steps (what `scripts/train.py --rebalance-experts-every N` does periodically; a relabelling of the experts, "
                         "the model is unchanged). --no-rebalance-experts keeps the static placement")
    ap.add_argument("--memory-mode", default="auto", choices=["auto", "tight", "roomy"],
                    help="tight: bf16 gradients, no resident bf16 weight copies, SwiGLU pre-activations recomputed (what one GPU needs to hold all "
                         "17.7 B parameters); roomy: fp32 gradients, bf16 copies, pre-activations kept; auto: tight only when the state would not fit. "
                         "Running several GPUs in tight mode gives a like-for-like curve against the one-GPU point")
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncate the model (the result is then labelled invalid)")
    return ap.parse_args()


def reference_arm(args) -> None:
    """The reference needs Python >= 3.14, jax 0.11.2 (+cuda13), orbax, grain and array_record; none is installed and
    there is no package index, so it cannot be installed or run here."""
    reason = "reference needs Python>=3.14 and jax==0.11.2/orbax/grain/array_record, none installable offline (pip --no-index: no matching distribution)"
    try:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import jax  # noqa: F401
        import lyra  # noqa: F401

        reason = "reference imports, but no GPU-enabled jaxlib is present"
    except Exception:
        pass
    print(json.dumps({"impl": "reference", "unavailable": reason}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    from lyra_b200.config import flops_per_token
    from lyra_b200.model import ModelWeights
    from lyra_b200.ops import cuda_ops, native
    from lyra_b200.training.presets import TRAINING_PRESETS
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper
    from lyra_b200.variants import model_variant

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    # b200  : the product - own kernels for compute, own peer-memory kernels for every multi-GPU data path
    # nccl  : stand-in for a library-collective build, NOT the reference: the same compute kernels, but weights, gradients and
    #         expert tokens move through torch.distributed (NCCL) broadcast / reduce / all_to_all as in lyra/training/steps.py:75-91
    #         and lyra/kernels/ep_moe.py:130-149
    # torch : PyTorch library ops (cuBLAS, eager attention) for compute and NCCL for communication
    impl = {"b200": "auto", "torch": "torch", "nccl": "auto"}[args.impl]
    mcfg = replace(model_variant(args.variant), implementation=impl)
    valid = True
    if args.layers is not None:
        mcfg = replace(mcfg, n_layers=args.layers, mlp_map=mcfg.mlp_map[: args.layers])
        valid = False
    rt = None
    if world > 1:
        from lyra_b200.parallel.runtime import Runtime

        dist.init_process_group("nccl", device_id=device)
        rt = Runtime.create(world_size=world, rank=rank, device=device, implementation="nccl" if args.impl in ("nccl", "torch") else "b200", mcfg=mcfg)
    preset = TRAINING_PRESETS.get("train-" + args.variant.removeprefix("lyra-"))
    acc = args.accumulation or (preset.accumulation_steps if preset else 1)
    B, T = args.micro_batch, mcfg.seq_len
    tcfg = replace(preset, batch_size=B * world, accumulation_steps=acc) if preset else None
    if tcfg is None:
        from lyra_b200.training.train import TrainingConfig

        tcfg = TrainingConfig(batch_size=B * world, accumulation_steps=acc)

    # memory plan: on one GPU the 17.7B-parameter model leaves no room for bf16 weight copies or fp32 gradients
    from lyra_b200.nn.params import param_count

    n_params = param_count(ModelWeights.spec(mcfg))
    local_params = n_params / world if rt is not None else n_params
    tight = local_params * 14 > 150e9 if args.memory_mode == "auto" else args.memory_mode == "tight"
    cuda_ops.set_memory_mode(keep_shadows=not tight, grad_dtype=torch.bfloat16 if tight else torch.float32, save_preact=not tight)

    if args.impl == "torch":
        # eager attention keeps [heads, T, T] fp32 scores of every layer for backward: this does not fit for the 4096-token variants
        est = mcfg.n_layers * mcfg.n_attn_heads * B * T * T * 4 * 2 + local_params * 12
        if est > 170e9:
            if rank == 0:
                print(json.dumps({"impl": "torch", "unavailable": f"PyTorch eager path needs about {est / 1e9:.0f} GB per GPU for {args.variant} at "
                                  f"{B}x{T} tokens (attention scores of all layers are kept for backward)"}))
            if world > 1:
                dist.destroy_process_group()
            return
    shard_fn = rt.shard_info if rt is not None else None
    weights = ModelWeights.init(mcfg.seed, mcfg, device=device, shard_fn=shard_fn)
    state = init_train_state(weights, mcfg, tcfg)
    stepper = Stepper(state, mcfg, tcfg, device=device, rt=rt)

    rng = np.random.default_rng(1234 + rank)
    total_steps = args.warmup + 2 * args.steps
    host_x = [torch.from_numpy(rng.integers(0, mcfg.vocab_size, size=(acc, B, T), dtype=np.int64).astype(np.int32)).pin_memory()
              for _ in range(min(total_steps, 4))]
    host_y = [torch.roll(x, -1, dims=-1).contiguous().pin_memory() for x in host_x]
    dev_x = [x.to(device) for x in host_x]
    dev_y = [y.to(device) for y in host_y]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    placement = None
    metering = args.rebalance_experts and rt is not None and rt.meter_expert_load()
    step_idx = 0
    for _ in range(args.warmup):
        stepper.train_step(dev_x[step_idx % len(dev_x)], dev_y[step_idx % len(dev_y)], step_idx)
        step_idx += 1
    if metering:   # what the training loop does every --rebalance-experts-every steps
        placement = {k: round(float(v), 4) for k, v in rt.rebalance_experts(stepper.params, state.optimizer).items()}
        stepper.train_step(dev_x[step_idx % len(dev_x)], dev_y[step_idx % len(dev_y)], step_idx)   # one untimed step on the new placement
        step_idx += 1
    barrier()
    native.check_status()

    # ---- device-timed region: K steps, inputs resident on the device
    launches0 = native.launches()
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = stepper.train_step(dev_x[step_idx % len(dev_x)], dev_y[step_idx % len(dev_y)], step_idx)
            step_idx += 1
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    launches = native.launches() - launches0
    loss = float(out["loss"])

    # ---- end to end: pinned host inputs copied every microbatch, loss read back every step
    stepper.h2d_bytes = 0
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    d2h = 0
    for _ in range(args.steps):
        out = stepper.train_step(host_x[step_idx % len(host_x)], host_y[step_idx % len(host_y)], step_idx)
        loss_e2e = out["loss"].item()
        d2h += out["loss"].element_size()
        step_idx += 1
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1)
    native.check_status()

    # ---- one more untimed step with CUDA events around the phases of a step (device time, max over ranks)
    from lyra_b200.utils.phases import collect

    names = ["forward_backward", "ep_wait", "gradient_reduce", "optimizer", "weight_refresh", "step"]
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with collect() as spans:
        p0.record()
        stepper.train_step(dev_x[step_idx % len(dev_x)], dev_y[step_idx % len(dev_y)], step_idx)
        p1.record()
        sums = spans.totals_ms()
    sums["step"] = p0.elapsed_time(p1)
    step_idx += 1
    native.check_status()

    times = torch.tensor([ms, ms_e2e] + [sums.get(n, 0.0) for n in names], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(times[0]), float(times[1])
    phases = {n: round(float(v), 1) for n, v in zip(names, times[2:])}
    phases["note"] = ("ms of one extra step, CUDA events, max over ranks per phase; ep_wait (flag and arrival-counter wait kernels of the expert "
                      "exchange) lies inside forward_backward; tile waits inside the grouped GEMMs are not separable; step - (forward_backward + "
                      "gradient_reduce + optimizer + weight_refresh) is host gaps")

    tokens_per_step = acc * B * T * world
    value = tokens_per_step * args.steps / (ms / 1e3)
    value_e2e = tokens_per_step * args.steps / (ms_e2e / 1e3)
    fpt = flops_per_token(mcfg)
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peak = json.loads(peaks_file.read_text())["bf16_tflops_sustained"] if peaks_file.exists() else 1400.0
    if rank == 0:
        line = {
            "metric": "train tokens/s (lyra-medium)" if args.variant == "lyra-medium" else f"train tokens/s ({args.variant})",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 2), "higher_is_better": True, "scaling": "weak",
            # the reference publishes an end-to-end figure for lyra-small only (one TPU v6e); other variants have none
            "vs_baseline": round(value / BASELINE_TOKENS_PER_S, 3) if args.variant == "lyra-small" else None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": args.variant, "global_batch": B * world * acc, "seq_len": T, "per_gpu_microbatch": f"{B}x{T}",
                       "accumulation_steps": acc, "parallelism": ("single" if world == 1 else f"fsdp+ep{world}"),
                       "optimizer": "muon+adam in timed region", "l2": "per-step working set (weights, activations) far exceeds the 126 MB L2",
                       "memory_mode": "tight" if tight else "roomy",
                       "grad_dtype": str(cuda_ops.GRAD_DTYPE).replace("torch.", ""), "bf16_weight_copies": cuda_ops.KEEP_SHADOWS,
                       "params": n_params, "valid": valid, **({"expert_placement": placement} if placement is not None else {})},
            "mfu_of_measured_sustained_bf16": round(value * fpt / world / (peak * 1e12), 4),
            "flops_per_token": fpt, "loss": round(loss, 4),
            "clocks": clocks.summary(),
            "e2e": {"value": round(value_e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": stepper.h2d_bytes // max(args.steps, 1),
                    "d2h_bytes_per_step": d2h // max(args.steps, 1), "ms_per_step": round(ms_e2e / args.steps, 2), "loss": round(loss_e2e, 4)},
            "phases": phases,
            "gpu_launches": launches,
            "max_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1),
            "max_reserved_gb": round(torch.cuda.max_memory_reserved() / 1e9, 1),
            "allocator_retries": int(torch.cuda.memory_stats().get("num_alloc_retries", 0)),   # > 0: the step ran at the memory limit
            "baseline_note": "the reference's only published end-to-end figure is lyra-small, 34,150 tok/s on one TPU v6e (README.md:33); vs_baseline is that ratio for --variant lyra-small and null for variants without a published number",
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
