"""Batched prefill + decode throughput of a GPT-OSS-shaped model on one GPU (random bf16 weights, synthetic prompts).

    python bench/serve.py                                  # gpt-oss-20b, batch 64, 1024-token prompts, 128 new tokens
    python bench/serve.py --variant lyra-small --batch 8 --prompt 256 --new 64
    python bench/serve.py --layers 4 --new 8 --no-graph    # a small case (e.g. under a profiler)
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/serve.py --variant gpt-oss-120b
                                                           # experts sharded over the ranks, every rank serves its own batch
    ... bench/serve.py --variant gpt-oss-120b --tensor-parallel     # heads and hidden units split instead, one shared batch

Prints one JSON line: prefill tokens/s, decode tokens/s with the per-token launch sequence replayed from a CUDA graph and
launched eagerly, and the decode step time against the time to read the active weights and the KV cache once at the
measured HBM bandwidth. Device timings are CUDA events around the whole prefill / the whole decode loop after one
untimed round; the working set (weights + cache) is far larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os

import sys
from dataclasses import replace
from pathlib import Path

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # load kernels with the library, not at first launch (multi-rank waits)
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def hbm_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    return (json.loads(p.read_text())["hbm_gbs"], "measured") if p.exists() else (6650.0, "fallback")


def timed(fn) -> tuple[float, object]:
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    out = fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e), out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", default="gpt-oss-20b")
    ap.add_argument("--batch", type=int, default=64, help="prompts per rank (expert parallel: every rank serves its own batch)")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="prompts served by the whole job, split evenly over the ranks (overrides --batch; the gpt-oss-120b headline is 64 over 8 ranks)")
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to this many layers (0 = all)")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 expert weights and an e4m3 KV cache")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--profile-decode", action="store_true",
                    help="bracket the timed decode with cudaProfilerStart / Stop, so that a profiler started with "
                         "--profile-from-start off sees the decode steps only (not initialisation or prefill)")
    ap.add_argument("--rebalance", action="store_true",
                    help="expert parallel: one metered warm-up request, then the experts are re-placed on the ranks by its token counts")
    ap.add_argument("--tensor-parallel", action="store_true",
                    help="several ranks: split heads and hidden units over the ranks (one shared batch, library all-reduce per block) instead of expert parallelism")
    args = ap.parse_args()

    from lyra_b200.generate import BatchedGenerator
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.params import param_count, tree_leaves
    from lyra_b200.nn.quant import QArray
    from lyra_b200.ops import native
    from lyra_b200.variants import model_variant

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if args.global_batch:
        if args.global_batch % world and not args.tensor_parallel:
            raise SystemExit(f"--global-batch {args.global_batch} does not split over {world} ranks")
        args.batch = args.global_batch if args.tensor_parallel else args.global_batch // world
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    mcfg = replace(model_variant(args.variant), param_dtype=torch.bfloat16, sample_temperature=0.0)
    if args.layers:
        mcfg = replace(mcfg, n_layers=args.layers, mlp_map=mcfg.mlp_map[: args.layers])
    if args.fp8:
        mcfg = replace(mcfg, quantize_mlp=True, quantize_cache=True, gemm_dtype=torch.float8_e4m3fn, quant_block=(64, 64))
    rt = None
    tp = world > 1 and args.tensor_parallel
    if tp:          # tensor parallel: every rank holds a slice of every layer and all ranks serve the same batch
        import torch.distributed as dist

        from lyra_b200.parallel.tp import TensorParallel

        dist.init_process_group("nccl", device_id=dev)
        rt = TensorParallel(mcfg, rank, world)
        model = ModelWeights.init(0, mcfg, device=dev, shard_fn=rt.shard_info)
    elif world > 1:   # expert parallel: experts sharded over the ranks, attention replicated, one batch per rank
        import torch.distributed as dist

        from lyra_b200.parallel.runtime import Runtime

        dist.init_process_group("nccl", device_id=dev)
        rt = Runtime.create(world_size=world, rank=rank, device=dev, implementation="b200", mcfg=mcfg)
        model = ModelWeights.init(0, mcfg, device=dev, shard_fn=rt.shard_info)
        rt.register(model)
        rt.finish_weight_pulls()
    else:
        model = ModelWeights.init(0, mcfg, device=dev)
    if args.fp8:
        model = ModelWeights.quantize(model, mcfg)
    capacity = args.prompt + args.new
    prompts = torch.randint(0, mcfg.vocab_size, (args.batch, args.prompt), device=dev,
                            generator=torch.Generator(device=dev).manual_seed(1 if tp else 1 + rank))   # one shared batch under tensor parallelism
    served = 1 if tp else world                              # batches served by the job

    placement = None
    if args.rebalance and world > 1 and not tp:
        from lyra_b200.nn.params import tree_dict

        rt.meter_expert_load(inference=True)
        gen = BatchedGenerator(model, mcfg, batch=args.batch, capacity=capacity, device=dev, rt=rt, use_cuda_graph=False)
        gen.decode(gen.prefill(prompts), min(args.new, 8))
        placement = rt.rebalance_experts(tree_dict(model))
        rt.load_meter = None                               # the timed runs carry no metering
        del gen
        torch.cuda.empty_cache()

    results = {}
    for mode in (["eager"] if args.no_graph else ["graph", "eager"]):
        gen = BatchedGenerator(model, mcfg, batch=args.batch, capacity=capacity, device=dev, rt=rt, use_cuda_graph=(mode == "graph"))
        first = gen.prefill(prompts)                       # untimed round: one-time set-up, graph capture
        gen.decode(first, min(args.new, 4))
        t_pre, first = timed(lambda: gen.prefill(prompts))
        l0 = native.launches()
        if args.profile_decode:
            torch.cuda.profiler.start()
        t_dec, toks = timed(lambda: gen.decode(first, args.new))
        if args.profile_decode:
            torch.cuda.profiler.stop()
        native.check_status()
        if world > 1:   # the job's time is the slowest rank's
            t = torch.tensor([t_pre, t_dec], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_pre, t_dec = float(t[0]), float(t[1])
        results[mode] = {"prefill_ms": t_pre, "decode_ms": t_dec, "tokens": toks, "launches_per_token": (native.launches() - l0) / max(1, args.new - 1)}
        del gen
        torch.cuda.empty_cache()

    best = "eager" if args.no_graph else "graph"
    if not args.no_graph:
        same = bool(torch.equal(results["graph"]["tokens"], results["eager"]["tokens"]))
    steps = args.new - 1
    # bytes one decode step must read: every weight that takes part (all attention weights, the router, the experts that
    # received a token: at most min(E, batch * k) per layer) and the visible KV rows
    def nbytes(t):
        return (t.qval.numel() + t.scale.numel() * 4) if isinstance(t, QArray) else t.numel() * t.element_size()
    total_w = sum(nbytes(t) for t in tree_leaves(model))
    expert_w = sum(nbytes(t) for l in model.layers for t in (l.mlp.mlp_up, l.mlp.mlp_down) if hasattr(l.mlp, "router"))
    frac_active = min(1.0, args.batch * mcfg.n_active_experts / max(1, mcfg.n_experts))
    kv_el = 1 if args.fp8 else 2
    mean_pos = args.prompt + args.new / 2
    kv = sum(2 * args.batch * (mcfg.n_kv_heads // (world if tp else 1)) * min(mean_pos, mcfg.layer_window(i) or mean_pos) * mcfg.head_dim * kv_el for i in range(mcfg.n_layers))
    step_bytes = total_w - expert_w * (1 - frac_active) + kv
    bw, kind = hbm_gbs()
    step_ms = results[best]["decode_ms"] / steps
    line = {
        "bench": "batched serve", "n_gpus": world, "parallelism": (f"tp{world}" if tp else f"ep{world} + data-parallel attention") if world > 1 else "single", "model": mcfg.name, "layers": mcfg.n_layers, "params": param_count(ModelWeights.spec(mcfg)), "batch_per_rank": args.batch, "global_batch": served * args.batch,
        "prompt_len": args.prompt, "new_tokens": args.new, "dtype": "bf16" + (" + e4m3 experts and KV" if args.fp8 else ""), "data": "synthetic tokens, random-init weights",
        "prefill_tokens_per_s": round(served * args.batch * args.prompt / results[best]["prefill_ms"] * 1e3, 1),
        "decode_tokens_per_s": round(served * args.batch * steps / results[best]["decode_ms"] * 1e3, 1),
        "decode_ms_per_step": round(step_ms, 3),
        "decode_bytes_per_step_gb": round(step_bytes / 1e9, 3),
        f"decode_frac_of_{kind}_hbm": round(step_bytes / (step_ms * 1e-3) / 1e9 / bw, 3),
        "own_kernel_launches_per_token_eager": round(results["eager"]["launches_per_token"], 1) if "eager" in results else None,
    }
    if not args.no_graph:
        line["decode_tokens_per_s_eager"] = round(served * args.batch * steps / results["eager"]["decode_ms"] * 1e3, 1)
        line["graph_equals_eager"] = same
    if placement is not None:
        line["expert_placement"] = {k: round(float(v), 4) for k, v in placement.items()}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
