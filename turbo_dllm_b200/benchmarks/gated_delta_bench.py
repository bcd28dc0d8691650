"""Times the chunked gated delta rule on one GPU: the state-scan kernels against the PyTorch loop.

    python -m turbo_dllm_b200.benchmarks.gated_delta_bench --seq 8192 --heads 32 --chunk 32

Prints one JSON line per mode (`native` = `csrc/gated_delta_scan.cu`, `torch` = batched-product loop):
forward and forward+backward device time (CUDA events around the call, median after warm-up) of
`ops.gated_delta.gated_delta_chunked` with states returned, plus the time of the scan kernels' share
estimated from the algorithmic work: per chunk and head 3 products of C x Dk x Dv and one of C x C x Dv
forward, about 2.3 times that backward. `--blocks` times the noisy-block pattern instead: many one-chunk
sequences that each start from their own state.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main(argv=None):
    from turbo_dllm_b200.ops.gated_delta import gated_delta_chunked, gdn_gate, l2_normalize

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--dk", type=int, default=128)
    ap.add_argument("--dv", type=int, default=128)
    ap.add_argument("--chunk", type=int, default=32)
    ap.add_argument("--blocks", type=int, default=0, help="time this many one-chunk sequences with initial states")
    ap.add_argument("--modes", nargs="+", default=["native", "torch"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    B, T = (a.blocks, a.chunk) if a.blocks else (a.batch, a.seq)
    g = torch.Generator(device=dev).manual_seed(0)
    r = lambda *s: torch.randn(*s, device=dev, generator=g)
    q, k = l2_normalize(r(B, T, a.heads, a.dk)), l2_normalize(r(B, T, a.heads, a.dk))
    v = r(B, T, a.heads, a.dv).requires_grad_(True)
    gate = gdn_gate(r(B, T, a.heads), torch.zeros(a.heads, device=dev), torch.zeros(a.heads, device=dev))
    beta = torch.sigmoid(r(B, T, a.heads))
    s0 = (r(B, a.heads, a.dk, a.dv) * 0.1).requires_grad_(True) if a.blocks else None
    go = r(B, T, a.heads, a.dv)
    chunks = B * a.heads * (T // a.chunk)
    flop_fwd = chunks * 2.0 * (3 * a.chunk * a.dk * a.dv + a.chunk * a.chunk * a.dv)
    for mode in a.modes:
        os.environ["TDLLM_GDN_SCAN"] = mode

        def fwd():
            with torch.no_grad():
                return gated_delta_chunked(q, k, v, gate, beta, initial_state=s0, chunk=a.chunk, return_states=True)

        def fwd_bwd():
            o, _, st = gated_delta_chunked(q, k, v, gate, beta, initial_state=s0, chunk=a.chunk, return_states=True)
            ((o * go).sum() + st.sum() * 1e-3).backward()
            v.grad = None
            if s0 is not None:
                s0.grad = None

        ms_f = _time(fwd, a.iters, a.warmup)
        ms_fb = _time(fwd_bwd, a.iters, a.warmup)
        print(json.dumps({"mode": mode, "shape": {"batch": B, "tokens": T, "heads": a.heads, "dk": a.dk, "dv": a.dv,
                                                    "chunk": a.chunk}, "forward_ms": round(ms_f, 3),
                          "forward_backward_ms": round(ms_fb, 3), "scan_gflop_forward": round(flop_fwd / 1e9, 2)}),
              flush=True)


if __name__ == "__main__":
    main()
