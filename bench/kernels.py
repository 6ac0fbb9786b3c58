"""Per-kernel device timings against the measured roofline denominators.

    python bench/kernels.py gemm            # tcgen05 GEMM family vs torch.matmul (cuBLAS)
    python bench/kernels.py all

Timing: CUDA events on the launching stream, 3 warm-up runs, an L2 flush (a 256 MB write) between
timed runs, median of the timed runs. Peaks come from MEASURED_PEAKS.json at the repository root when it
exists (fractions are "of measured"), else 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""

from __future__ import annotations

import json
import statistics
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


_flush = None


def time_ms(fn, iters: int = 10, warmup: int = 3) -> float:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def report(name: str, ms: float, flops: float = 0.0, bytes_: float = 0.0, ref_ms: float | None = None) -> dict:
    pk = peaks()
    row = {"kernel": name, "ms": round(ms, 4)}
    if flops:
        row["tflops"] = round(flops / ms / 1e9, 1)
        row[f"frac_of_{pk['kind']}_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
    if bytes_:
        row["gbs"] = round(bytes_ / ms / 1e6, 1)
        row[f"frac_of_{pk['kind']}_hbm"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)
    if ref_ms is not None:
        row["library_ms"] = round(ref_ms, 4)
    print(json.dumps(row), flush=True)
    return row


def bench_gemm():
    from lyra_b200.ops import gemm as G

    for (M, N, K) in [(8192, 4096, 4096), (8192, 12288, 4096), (8192, 4096, 6144), (16384, 4096, 2048), (4096, 4096, 4096)]:
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = torch.randn(K, N, device="cuda").bfloat16()
        dy = torch.randn(M, N, device="cuda").bfloat16()
        fl = 2.0 * M * N * K
        report(f"gemm fwd x@W M{M} N{N} K{K}", time_ms(lambda: G.gemm(x, w, b_mn=True)), fl, ref_ms=time_ms(lambda: x @ w))
        report(f"gemm dgrad dy@W^T M{M} N{N} K{K}", time_ms(lambda: G.gemm(dy, w)), fl, ref_ms=time_ms(lambda: dy @ w.t()))
        report(f"gemm wgrad x^T@dy M{M} N{N} K{K}", time_ms(lambda: G.gemm(x, dy, a_mn=True, b_mn=True, out_dtype=torch.float32)), fl,
               ref_ms=time_ms(lambda: x.t() @ dy))
    # MoE shapes of the reference's kernel table (M=65536 routed rows, 16 experts, K=2048, N=4096)
    M, E, K, H = 65536, 16, 2048, 2048
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(E, K, 2 * H, device="cuda") / 32).bfloat16()
    tg = torch.arange(M // 128, device="cuda", dtype=torch.int32) // (M // 128 // E)
    report("moe up+swiglu M65536 G16 K2048 N4096", time_ms(lambda: G.grouped_gemm(x, w, tg, swiglu=True)), 2.0 * M * K * 2 * H)
    h = torch.randn(M, H, device="cuda").bfloat16()
    wd = (torch.randn(E, H, K, device="cuda") / 32).bfloat16()
    report("moe down M65536 G16 K2048 N2048", time_ms(lambda: G.grouped_gemm(h, wd, tg)), 2.0 * M * H * K)


BENCHES = {"gemm": bench_gemm}



def bench_attention():
    from lyra_b200.ops import attention as A

    for (B, Nq, Nkv, T, D, name) in [(4, 16, 4, 4096, 128, "small"), (2, 32, 8, 4096, 128, "medium")]:
        q = torch.randn(B, T, Nq, D, device="cuda").bfloat16().transpose(1, 2)
        k = torch.randn(B, T, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
        v = torch.randn(B, T, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
        do = torch.randn(B, T, Nq, D, device="cuda").bfloat16().transpose(1, 2)
        sinks = torch.zeros(Nq, device="cuda")
        for window in (0, 128):
            mean_pos = (T + 1) / 2 if not window else (window * (window + 1) / 2 + (T - window) * window) / T
            fl = 4.0 * B * Nq * T * mean_pos * D
            out, lse = A.flash_fwd(q, k, v, sinks, D ** -0.5, window)
            report(f"flash fwd {name} B{B} T{T} {Nq}q/{Nkv}kv hd{D} window{window}", time_ms(lambda: A.flash_fwd(q, k, v, sinks, D ** -0.5, window)), fl)
            report(f"flash bwd {name} B{B} T{T} {Nq}q/{Nkv}kv hd{D} window{window}",
                   time_ms(lambda: A.flash_bwd(q, k, v, out, do, lse, sinks, D ** -0.5, window)), 2.5 * fl)


BENCHES["attention"] = bench_attention


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    for name, fn in BENCHES.items():
        if which in ("all", name):
            fn()
