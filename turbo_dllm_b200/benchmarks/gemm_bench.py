"""Times the tcgen05 GEMM against the measured bf16 matmul peak.

    python -m turbo_dllm_b200.benchmarks.gemm_bench --shapes 8192x8192x8192 --iters 10

Prints one JSON line per shape: TFLOP/s of this kernel, of torch.matmul (cuBLAS) on the same
inputs, and the fraction of the measured peak when MEASURED_PEAKS.json is present.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def flush_l2(buf):
    buf.zero_()


def time_fn(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush_l2(flush)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


def layer_shapes(rows: int, hidden: int, qkv: int, ffn: int) -> list[tuple[str, str]]:
    """(MxNxK, layout) of every GEMM one decoder layer runs: forward, input gradient, weight gradient."""
    out = []
    for n_out, k_in in ((qkv, hidden), (hidden, hidden), (2 * ffn, hidden), (hidden, ffn)):
        out.append((f"{rows}x{n_out}x{k_in}", "kk"))      # y = x W^T
        out.append((f"{rows}x{k_in}x{n_out}", "kn"))      # dx = dy W
        out.append((f"{n_out}x{k_in}x{rows}", "nn"))      # dW = dy^T x
    return out


def main(argv=None):
    from turbo_dllm_b200.ops.gemm import gemm

    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192x8192x8192,16384x12288x4096,16384x4096x12288")
    ap.add_argument("--layouts", default="kk,kn,nn")
    ap.add_argument("--layer", default=None,
                    help="rows,hidden,qkv_dim,ffn: time every GEMM of one decoder layer instead of --shapes")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    peak = None
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    pk = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if args.layer:
        work = layer_shapes(*(int(v) for v in args.layer.split(",")))
    else:
        work = [(shp, lay) for shp in args.shapes.split(",") for lay in args.layouts.split(",")]
    for shp, lay in work:
        M, N, K = (int(v) for v in shp.split("x"))
        if True:
            a_mn, b_mn = lay[0] == "n", lay[1] == "n"
            a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
            b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            med, best = time_fn(lambda: gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out),
                                args.iters, args.warmup, flush)
            A = a.t() if a_mn else a
            B = b if b_mn else b.t()
            medc, bestc = time_fn(lambda: torch.matmul(A, B, out=out), args.iters, args.warmup, flush)
            fl = 2.0 * M * N * K
            rec = {"shape": shp, "layout": lay, "ms": round(med, 4), "tflops": round(fl / med / 1e9, 1),
                   "tflops_best": round(fl / best / 1e9, 1), "cublas_ms": round(medc, 4),
                   "cublas_tflops": round(fl / medc / 1e9, 1)}
            if peak:
                rec["frac_of_measured_peak"] = round(fl / med / 1e9 / peak, 3)
            print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
