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
    native.check_status()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
