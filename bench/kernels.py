"""Per-kernel device timings against the measured roofline denominators.

    python bench/kernels.py gemm            # tcgen05 GEMM family vs torch.matmul (cuBLAS)
    python bench/kernels.py attention | ce | elementwise | decode | decode_gemm | all
    python bench/kernels.py one <case>      # three launches of one small case, for a profiler capture (cases: see ONE)

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


def time_graph_ms(fn, iters: int = 10) -> float:
    """Device time of ``fn`` replayed from a CUDA graph (the way the decode loop runs it): no host launch gaps between its kernels."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    times = []
    for _ in range(iters + 2):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times[2:])


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


def bench_ce():
    """Fused linear + cross-entropy (logits never stored) against torch's matmul + cross_entropy."""
    from lyra_b200.ops import cuda_ops

    for (M, C, V) in [(8192, 2048, 200064), (8192, 4096, 200064)]:
        x = (torch.randn(M, C, device="cuda") / 4).bfloat16().requires_grad_()
        w = (torch.randn(V, C, device="cuda") / 64).requires_grad_()   # [padded vocabulary, C], as the model stores it
        y = torch.randint(0, V - 64, (M,), device="cuda")
        fl = 2.0 * M * C * V

        def fwd():
            with torch.no_grad():
                return cuda_ops.linear_cross_entropy(x, w, y, V - 64)[0]

        def fwd_bwd():
            x.grad = None
            w.grad = None
            cuda_ops.linear_cross_entropy(x, w, y, V - 64)[0].backward()

        report(f"linear-CE fwd M{M} C{C} V{V}", time_ms(fwd, iters=5), fl)
        report(f"linear-CE fwd+bwd M{M} C{C} V{V}", time_ms(fwd_bwd, iters=5), 4.0 * fl)   # fwd + recompute + dX + dW
        del x, w


BENCHES["ce"] = bench_ce


def bench_elementwise():
    """Bandwidth-bound kernels: bytes are the algorithmic minimum (each tensor read or written once)."""
    from lyra_b200.ops import elementwise as E

    M, C = 32768, 4096
    x = torch.randn(M, C, device="cuda").bfloat16()
    scale = torch.ones(C, device="cuda")
    dy = torch.randn(M, C, device="cuda").bfloat16()
    report(f"rmsnorm fwd M{M} C{C}", time_ms(lambda: E.RMSNorm.apply(x, scale, 1e-6)), bytes_=2.0 * M * C * 2)
    xr = x.clone().requires_grad_()
    sr = scale.clone().requires_grad_()
    out = E.RMSNorm.apply(xr, sr, 1e-6)
    report(f"rmsnorm bwd M{M} C{C}", time_ms(lambda: torch.autograd.grad(out, (xr, sr), dy, retain_graph=True)), bytes_=3.0 * M * C * 2)
    H = 8192
    pre = torch.randn(M // 2, 2 * H, device="cuda").bfloat16()
    dact = torch.randn(M // 2, H, device="cuda").bfloat16()
    report(f"swiglu fwd M{M // 2} H{H}", time_ms(lambda: E.swiglu_fwd(pre, 1.702, 7.0)), bytes_=3.0 * (M // 2) * H * 2)
    report(f"swiglu bwd M{M // 2} H{H}", time_ms(lambda: E.swiglu_bwd(pre, dact, 1.702, 7.0)), bytes_=5.0 * (M // 2) * H * 2)


BENCHES["elementwise"] = bench_elementwise


def bench_decode():
    """Single-token attention over a KV cache: bytes = visible K and V rows read once."""
    from lyra_b200.nn.quant import quantize
    from lyra_b200.ops import decode

    for (B, Nq, Nkv, S, D, name) in [(64, 64, 8, 2048, 64, "gpt-oss heads"), (8, 32, 8, 16384, 128, "lyra-medium heads"), (1, 32, 8, 32768, 128, "single sequence")]:
        q = torch.randn(B, Nq, 1, D, device="cuda").bfloat16()
        k = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
        v = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
        sinks = torch.zeros(Nq, device="cuda")
        pos = S - 1
        for window in (0, 128):
            n_keys = min(window, pos + 1) if window else pos + 1
            report(f"decode attention bf16 cache {name} B{B} {Nq}q/{Nkv}kv hd{D} S{S} window{window}",
                   time_ms(lambda: decode.decode_attention(q, k, v, sinks, D ** -0.5, window, pos)), bytes_=2.0 * B * Nkv * n_keys * D * 2)
        k8 = quantize(k, torch.float8_e4m3fn, block=(1, D))
        v8 = quantize(v, torch.float8_e4m3fn, block=(1, D))
        report(f"decode attention fp8 cache {name} B{B} {Nq}q/{Nkv}kv hd{D} S{S} window0",
               time_ms(lambda: decode.decode_attention(q, k8, v8, sinks, D ** -0.5, 0, pos)), bytes_=2.0 * B * Nkv * (pos + 1) * (D + 4))
        del k, v, k8, v8


BENCHES["decode"] = bench_decode


def bench_decode_gemm():
    """Small-M expert products of one decode step: bytes = weights of the experts that have rows, read once."""
    import os

    from lyra_b200.nn.quant import quantize
    from lyra_b200.ops import decode

    for (G, K, N, rows_per, name) in [(32, 2880, 5760, 8, "gpt-oss up"), (32, 2880, 2880, 8, "gpt-oss down"), (16, 4096, 4096, 4, "lyra-medium expert"),
                                      (1, 4096, 6144, 64, "dense qkv, 64 rows")]:
        R = G * rows_per
        x = torch.randn(R, K, device="cuda").bfloat16()
        w = (torch.randn(G, K, N, device="cuda") / K ** 0.5).bfloat16()
        offsets = (torch.arange(G + 1, device="cuda", dtype=torch.int32) * rows_per) if G > 1 else None
        for panel in (64, 128, 192):
            if N % panel:
                continue
            os.environ["LYRA_DECODE_PANEL"] = str(panel)
            report(f"decode gemm bf16 {name} G{G} K{K} N{N} rows/group {rows_per} panel{panel}",
                   time_ms(lambda: decode.decode_gemm(x, w, offsets=offsets)), bytes_=2.0 * G * K * N)
            if panel == 128:
                report(f"decode gemm bf16 {name} G{G} K{K} N{N} rows/group {rows_per} panel{panel} (CUDA graph replay)",
                       time_graph_ms(lambda: decode.decode_gemm(x, w, offsets=offsets, max_group_rows=rows_per)), bytes_=2.0 * G * K * N)
        os.environ.pop("LYRA_DECODE_PANEL", None)
        w8 = quantize(w, torch.float8_e4m3fn, block=(64, 64))
        for tc in (False, True):     # mma.sync kernel that dequantises in flight / tcgen05 e4m3 x e4m3 kernel (activation quantisation included)
            decode.F8_TENSOR_CORES = tc
            report(f"decode gemm e4m3 {'tcgen05' if tc else 'dequantise + mma.sync'} {name} G{G} K{K} N{N} rows/group {rows_per}",
                   time_ms(lambda: decode.decode_gemm(x, w8, offsets=offsets, max_group_rows=rows_per)), bytes_=1.0 * G * K * N)
            report(f"decode gemm e4m3 {'tcgen05' if tc else 'dequantise + mma.sync'} {name} G{G} K{K} N{N} rows/group {rows_per} (CUDA graph replay)",
                   time_graph_ms(lambda: decode.decode_gemm(x, w8, offsets=offsets, max_group_rows=rows_per)), bytes_=1.0 * G * K * N)
        del w, w8
    # one decode step of a 128-expert layer on one rank: 8 tokens x top-4 land on about 28 experts, one or two rows each
    G, K, N = 128, 2880, 5760
    torch.manual_seed(0)
    ids, _ = torch.sort(torch.randint(0, G, (32,), device="cuda"))
    counts = torch.bincount(ids, minlength=G)
    offsets = torch.zeros(G + 1, dtype=torch.int32, device="cuda")
    offsets[1:] = torch.cumsum(counts, 0)
    active, most = int((counts > 0).sum()), int(counts.max())
    x = torch.randn(32, K, device="cuda").bfloat16()
    w8 = quantize((torch.randn(G, K, N, device="cuda") / K ** 0.5).bfloat16(), torch.float8_e4m3fn, block=(64, 64))
    decode.F8_TENSOR_CORES = True
    report(f"decode gemm e4m3 tcgen05 gpt-oss-120b up G{G} K{K} N{N} 32 rows on {active} experts (CUDA graph replay)",
           time_graph_ms(lambda: decode.decode_gemm(x, w8, offsets=offsets, max_group_rows=most)), bytes_=1.0 * active * K * N)


BENCHES["decode_gemm"] = bench_decode_gemm


def _one_gemm():
    from lyra_b200.ops import gemm as G
    x = torch.randn(8192, 4096, device="cuda").bfloat16()
    w = torch.randn(4096, 8192, device="cuda").bfloat16()
    return lambda: G.gemm(x, w, b_mn=True)


def _one_attention(backward: bool, window: int = 0):
    from lyra_b200.ops import attention as A
    B, Nq, Nkv, T, D = 2, 32, 8, 4096, 128
    q, k, v, do = (torch.randn(B, T, n, D, device="cuda").bfloat16().transpose(1, 2) for n in (Nq, Nkv, Nkv, Nq))
    sinks = torch.zeros(Nq, device="cuda")
    out, lse = A.flash_fwd(q, k, v, sinks, D ** -0.5, window)
    if backward:
        return lambda: A.flash_bwd(q, k, v, out, do, lse, sinks, D ** -0.5, window)
    return lambda: A.flash_fwd(q, k, v, sinks, D ** -0.5, window)


def _one_ce():
    from lyra_b200.ops import cuda_ops
    M, C, V = 4096, 2048, 200064
    x = (torch.randn(M, C, device="cuda") / 4).bfloat16().requires_grad_()
    w = (torch.randn(V, C, device="cuda") / 64).requires_grad_()
    y = torch.randint(0, V - 64, (M,), device="cuda")
    return lambda: cuda_ops.linear_cross_entropy(x, w, y, V - 64)[0].backward()


def _one_rmsnorm():
    from lyra_b200.ops import elementwise as E
    x = torch.randn(32768, 4096, device="cuda").bfloat16()
    scale = torch.ones(4096, device="cuda")
    return lambda: E.RMSNorm.apply(x, scale, 1e-6)


def _one_moe():
    from lyra_b200.ops import gemm as G
    M, Eg, K, H = 32768, 16, 2048, 2048
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(Eg, K, 2 * H, device="cuda") / 32).bfloat16()
    tg = torch.arange(M // 128, device="cuda", dtype=torch.int32) // (M // 128 // Eg)
    return lambda: G.grouped_gemm(x, w, tg, swiglu=True)


def _one_decode():
    from lyra_b200.ops import decode
    B, Nq, Nkv, S, D = 16, 32, 8, 8192, 128
    q = torch.randn(B, Nq, 1, D, device="cuda").bfloat16()
    k = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
    v = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
    sinks = torch.zeros(Nq, device="cuda")
    return lambda: decode.decode_attention(q, k, v, sinks, D ** -0.5, 0, S - 1)


def _one_decode_gemm():
    from lyra_b200.ops import decode
    G_, K, N, rows = 32, 2880, 5760, 8
    x = torch.randn(G_ * rows, K, device="cuda").bfloat16()
    w = (torch.randn(G_, K, N, device="cuda") / K ** 0.5).bfloat16()
    offsets = torch.arange(G_ + 1, device="cuda", dtype=torch.int32) * rows
    return lambda: decode.decode_gemm(x, w, offsets=offsets)


def _one_decode_gemm_f8():
    from lyra_b200.nn.quant import quantize
    from lyra_b200.ops import decode
    G_, K, N, rows = 32, 2880, 5760, 8
    x = torch.randn(G_ * rows, K, device="cuda").bfloat16()
    w8 = quantize((torch.randn(G_, K, N, device="cuda") / K ** 0.5).bfloat16(), torch.float8_e4m3fn, block=(64, 64))
    offsets = torch.arange(G_ + 1, device="cuda", dtype=torch.int32) * rows
    return lambda: decode.decode_gemm(x, w8, offsets=offsets, max_group_rows=rows)


ONE = {"decode_gemm": _one_decode_gemm, "decode_gemm_f8": _one_decode_gemm_f8, "gemm": _one_gemm, "flash_fwd": lambda: _one_attention(False), "flash_bwd": lambda: _one_attention(True),
       "flash_fwd_window": lambda: _one_attention(False, 128), "ce": _one_ce, "rmsnorm": _one_rmsnorm, "moe_up": _one_moe, "decode": lambda: _one_decode()}


def run_one(case: str) -> None:
    """Three launches of one case (inputs larger than L2 in total, well under 1 GB resident), then a synchronize."""
    fn = ONE[case]()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    from lyra_b200.ops import native
    native.check_status()
    print(json.dumps({"case": case, "ok": True}))


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which == "one":
        run_one(sys.argv[2])
        sys.exit(0)
    for name, fn in BENCHES.items():
        if which in ("all", name):
            fn()
