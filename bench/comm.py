"""Multi-GPU communication kernels against their rooflines (run with torchrun on >= 2 GPUs):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/comm.py

Each line: device time (CUDA events, max over ranks, median of 10 after 3 warm-ups, L2 flushed between runs) and the
achieved fraction of  max(FLOPs / measured bf16 peak, bytes over NVLink / 770 GB/s)  for the fused kernels: the all-gather
(peer pull) fused GEMM and the expert-parallel return fused into the grouped GEMM epilogue (peer stores).
"""

from __future__ import annotations

import json
import os

import statistics
import sys
from pathlib import Path

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # load kernels with the library, not at first launch (multi-rank waits)
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction on this pool


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text())["bf16_tflops"] if p.exists() else 1590.0


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from lyra_b200.ops import gemm as G, native
    from lyra_b200.parallel.comm import SymmetricSlab

    lib = native.kernels()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, setup=None, iters=10, warmup=3):
        ts = []
        for i in range(warmup + iters):
            if setup:
                setup()
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            if i >= warmup:
                ts.append(s.elapsed_time(e))
        t = torch.tensor([statistics.median(ts)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    peak = peaks()
    only_ep = len(sys.argv) > 1 and sys.argv[1] == "ep"      # `bench/comm.py ep`: just the MoE-layer and gradient-reduce rows
    if only_ep:
        bench_ep_layer(world, rank, dev, peak, timed)
        bench_reduce(world, rank, dev, timed)
        native.check_status()
        dist.destroy_process_group()
        return
    owner = (rank + 1) % world  # every rank pulls from its neighbour
    for (M, K, N) in [(8192, 4096, 4096), (8192, 4096, 12288), (8192, 6144, 4096), (2048, 4096, 4096)]:
        slab = SymmetricSlab(K * N * 2, dev, dist.group.WORLD.group_name)
        w = slab.view(0, K * N, torch.bfloat16).view(K, N)
        w.copy_((torch.randn(K, N, device=dev) / 64).bfloat16())
        local = torch.empty_like(w)
        x = torch.randn(M, K, device=dev).bfloat16()
        flags = torch.zeros((N + 255) // 256, dtype=torch.int32, device=dev)
        ep = [0]

        def fused():
            ep[0] += 1
            G.gemm_allgather(x, local, [slab.peer_ptrs[owner]], 1, K, flags, ep[0])

        def copy_then_gemm():
            native.check(lib.lyra_p2p_copy(native.ptr(local), native.c_void_p(slab.peer_ptrs[owner]), native.c_ll(K * N * 2), native.stream_ptr()), "copy")
            G.gemm(x, local, b_mn=True)

        t_gemm = timed(lambda: G.gemm(x, local, b_mn=True))
        t_copy = timed(lambda: native.check(lib.lyra_p2p_copy(native.ptr(local), native.c_void_p(slab.peer_ptrs[owner]), native.c_ll(K * N * 2), native.stream_ptr()), "copy"))
        t_seq = timed(copy_then_gemm)
        t_fused = timed(fused)
        flops, nbytes = 2.0 * M * N * K, K * N * 2.0
        roof_ms = max(flops / (peak * 1e12), nbytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"kernel": f"allgather-fused gemm M{M} K{K} N{N}", "world": world, "fused_ms": round(t_fused, 4),
                              "gemm_only_ms": round(t_gemm, 4), "peer_copy_ms": round(t_copy, 4), "copy_then_gemm_ms": round(t_seq, 4),
                              "peer_copy_gbs": round(nbytes / t_copy / 1e6, 1), "roofline_ms": round(roof_ms, 4),
                              "frac_of_roofline": round(roof_ms / t_fused, 3)}), flush=True)
        if (M, K, N) == (8192, 4096, 4096) and world > 2:
            # what the runtime does once per step and leaf: every rank pulls the same leaf from its one owner at the same moment
            def incast():
                ep[0] += 1
                G.gemm_allgather(x, local, [slab.peer_ptrs[0]], 0 if rank == 0 else 1, K, flags, ep[0])

            t_in = timed(incast)
            roof_in = max(flops / (peak * 1e12), (world - 1) * nbytes / (NVLINK_GBS * 1e9)) * 1e3   # the owner's egress carries world - 1 copies
            if rank == 0:
                print(json.dumps({"kernel": f"allgather-fused gemm M{M} K{K} N{N}, all ranks pull from one owner", "world": world,
                                  "fused_ms": round(t_in, 4), "roofline_ms": round(roof_in, 4), "frac_of_roofline": round(roof_in / t_in, 3)}), flush=True)
        del slab
    # ---- expert-parallel return leg fused into the grouped GEMM epilogue ------------------------------------------------
    # Every rank holds R expert-sorted rows [R, H] (El local experts, R / El rows each) that came from all ranks in equal
    # parts; the down-projection's result rows go back to slot `a` of their source rank's return buffer.
    import ctypes

    def arr(ptrs):
        return (ctypes.c_longlong * len(ptrs))(*ptrs)

    for (R, H, C, El) in [(32768, 2048, 4096, 4), (8192, 2048, 4096, 4), (32768, 2880, 2880, 16)]:
        E = El * world
        per_e = R // El
        act = (torch.randn(R, H, device=dev) / 8).bfloat16()
        w = (torch.randn(El, H, C, device=dev) / H ** 0.5).bfloat16()
        tile_group = (torch.arange(R // 128, device=dev) // (per_e // 128)).to(torch.int32)
        offsets = (torch.arange(El + 1, device=dev) * per_e).to(torch.int32)
        counts = torch.full((world, E), per_e // world, dtype=torch.int32, device=dev)
        # row r of expert j came from source rank (r_in_expert // (per_e / world)); slots are dense per source
        r_in = torch.arange(R, device=dev) % per_e
        src = (r_in // (per_e // world)).to(torch.int64)
        slot = (torch.arange(R, device=dev) // per_e) * (per_e // world) + r_in % (per_e // world) + rank * (R // world)
        meta = ((src << 24) | slot).to(torch.int32)
        ret = SymmetricSlab(R * C * 2, dev, dist.group.WORLD.group_name)
        row_dest = meta.clone()
        out_local = torch.empty(R, C, dtype=torch.bfloat16, device=dev)

        def fused():
            G.grouped_gemm(act, w, tile_group, row_dest=row_dest, peer_out=ret.peer_ptrs)

        def unfused():
            G.grouped_gemm(act, w, tile_group, out=out_local)
            native.check(lib.lyra_ep_return(native.ptr(out_local), native.ptr(meta), native.ptr(offsets), native.ptr(counts), world, rank, E, El,
                                            arr(ret.peer_ptrs), R, C, native.stream_ptr()), "ep_return")

        t_gemm = timed(lambda: G.grouped_gemm(act, w, tile_group, out=out_local))
        t_unfused = timed(unfused)
        t_fused = timed(fused)
        torch.cuda.synchronize()
        dist.barrier()
        # correctness of the fused path against the unfused one (same buffer, same slots)
        fused(); torch.cuda.synchronize(); dist.barrier()
        a = ret.view(0, R * C, torch.bfloat16).clone()
        dist.barrier()
        unfused(); torch.cuda.synchronize(); dist.barrier()
        same = bool(torch.equal(a, ret.view(0, R * C, torch.bfloat16)))
        flops = 2.0 * R * H * C
        nbytes = R * C * 2.0 * (world - 1) / world
        roof_ms = max(flops / (peak * 1e12), nbytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"kernel": f"EP return fused into grouped GEMM R{R} H{H} C{C} experts/rank {El}", "world": world,
                              "fused_ms": round(t_fused, 4), "gemm_only_ms": round(t_gemm, 4), "gemm_then_return_kernel_ms": round(t_unfused, 4),
                              "roofline_ms": round(roof_ms, 4), "frac_of_roofline": round(roof_ms / t_fused, 3), "equals_unfused": same}), flush=True)
        del ret
    bench_ep_layer(world, rank, dev, peak, timed)
    bench_reduce(world, rank, dev, timed)
    native.check_status()
    dist.destroy_process_group()


def bench_ep_layer(world, rank, dev, peak, timed):
    """One expert-parallel MoE layer forward (lyra-medium shapes: 2 x 4096 tokens per rank, 31 routed experts top-3 + shared
    expert, C = H = 4096): the tile-granular exchange (dispatch consumed inside the up-projection GEMM, return and score
    inside the down-projection epilogue, shared expert in the wait) against the barrier-ordered exchange and against NCCL
    all-to-all with the same expert kernels. Roofline = max(FLOPs / measured bf16 peak, bytes that must cross NVLink in one
    direction / 770 GB/s)."""
    from lyra_b200.config import ModelConfig
    from lyra_b200.model import ModelWeights
    from lyra_b200.ops import native
    from lyra_b200.parallel import ep
    from lyra_b200.parallel.runtime import Runtime

    if 32 % world:
        return
    c = ModelConfig(name="ep-bench", seq_len=4096, n_embd=4096, n_layers=1, head_dim=128, n_attn_heads=32, n_kv_heads=8, n_routed_experts=31,
                    n_shared_experts=1, n_active_experts=4, mlp_map=("moe",), vocab_size=4000, padded_vocab_size=4096, tie_embeddings=False)
    F_, C, H, Kr = 8192, c.n_embd, c.expert_hidden, c.n_active_routed_experts
    g = torch.Generator(device="cpu").manual_seed(50 + rank)
    xn = torch.randn(F_, C, generator=g).to(dev).bfloat16()
    vals, idx = torch.topk(torch.randn(F_, c.n_routed_experts, generator=g), Kr, dim=-1)
    scores = torch.cat([torch.softmax(vals, -1), torch.ones(F_, 1)], -1).to(dev)
    idx = torch.cat([idx, torch.full((F_, 1), c.n_routed_experts)], -1).to(dev)
    rows = F_ * Kr
    flops = (rows + F_) * (2.0 * C * 2 * H + 2.0 * H * C)
    link_bytes = 2.0 * rows * C * 2 * (world - 1) / world
    roof_ms = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
    results = {}
    for name, impl, tiles in (("nccl_all_to_all", "nccl", None), ("barrier_exchange", "b200", False), ("tile_exchange", "b200", True)):
        rt = Runtime.create(world_size=world, rank=rank, device=dev, implementation=impl, mcfg=c)
        w = ModelWeights.init(0, c, device=dev, shard_fn=rt.shard_info)
        rt.register(w)
        rt.finish_weight_pulls()
        if tiles is not None:
            ep.TILE_DISPATCH = tiles
        moe = w.layers[0].mlp

        def layer():
            with torch.no_grad():
                rt.begin_layer(0)
                rt.ep_moe(xn, scores, idx, moe, c)

        results[name] = timed(layer, iters=8, warmup=3)
        native.check_status()
        del rt, w, moe
        torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps({"kernel": f"EP MoE layer forward F{F_} K{Kr}+shared C{C} H{H} E32", "world": world,
                          **{k + "_ms": round(v, 4) for k, v in results.items()}, "roofline_ms": round(roof_ms, 4),
                          "frac_of_roofline_tile_exchange": round(roof_ms / results["tile_exchange"], 3),
                          "frac_of_roofline_barrier_exchange": round(roof_ms / results["barrier_exchange"], 3),
                          "frac_of_roofline_nccl": round(roof_ms / results["nccl_all_to_all"], 3)}), flush=True)


def bench_reduce(world, rank, dev, timed):
    """Gradient pull-reduce with the sum of squares fused in: every rank owns 1/world of a 1 GiB fp32 gradient slab and sums
    its part over all ranks' slabs. Bytes over NVLink per rank (ingress) = (world - 1) x its part."""
    import ctypes

    from lyra_b200.ops import native
    from lyra_b200.parallel.comm import SymmetricSlab

    lib = native.kernels()
    total = 1 << 28                                            # fp32 elements per rank's slab (1 GiB)
    part = total // world
    slab = SymmetricSlab(total * 4, dev, dist.group.WORLD.group_name)
    slab.view(0, total, torch.float32).normal_()
    out = torch.empty(part, dtype=torch.float32, device=dev)
    lib.lyra_reduce_pull_norm_blocks.restype = ctypes.c_int
    partial = torch.zeros(int(lib.lyra_reduce_pull_norm_blocks(ctypes.c_longlong(part))), 2, dtype=torch.float32, device=dev)
    peers = (ctypes.c_longlong * world)(*[p + rank * part * 4 for p in slab.peer_ptrs])

    def fused():
        native.check(lib.lyra_reduce_pull_norm(native.ptr(out), peers, world, ctypes.c_longlong(part), 0, 0, ctypes.c_longlong(0), 1, native.ptr(partial),
                                               native.stream_ptr()), "reduce_pull_norm")

    def unfused():
        native.check(lib.lyra_reduce_pull(native.ptr(out), peers, world, ctypes.c_longlong(part), 0, 0, native.stream_ptr()), "reduce_pull")
        torch.linalg.vector_norm(out, 2, dtype=torch.float32)

    t_fused, t_unfused = timed(fused), timed(unfused)
    link_bytes = (world - 1) * part * 4.0
    roof_ms = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    if rank == 0:
        print(json.dumps({"kernel": f"gradient pull-reduce + sum of squares, {part * 4 >> 20} MiB per owner", "world": world, "fused_ms": round(t_fused, 4),
                          "reduce_then_norm_ms": round(t_unfused, 4), "ingress_gbs": round(link_bytes / t_fused / 1e6, 1),
                          "roofline_ms": round(roof_ms, 4), "frac_of_roofline": round(roof_ms / t_fused, 3)}), flush=True)
    del slab


if __name__ == "__main__":
    main()
