"""Times the block-diffusion attention kernels (forward, backward) on one GPU.

    python -m turbo_dllm_b200.benchmarks.attention_bench --seq 32768 --block 32 --heads 32 --kv-heads 8

FLOPs are counted on the exactly visible query-key pairs (4·pairs·D per head forward,
10·pairs·D backward), the convention of the reference's exact attention-pair counters
(dllm_parallel/core/profiling/perf.py:872-878). Prints one JSON line.

`--baseline flex|sdpa` times the same mask, shapes and call through a stock PyTorch path on the same device, so
that the kernels have an anchor: `flex` is torch FlexAttention with a block mask built from the same codes
(it compiles its kernels with Triton; when that is not possible on the box the run falls back to `sdpa` and says
so), `sdpa` is scaled_dot_product_attention with the dense boolean mask (rows² bytes: keep --seq at 8192 or so).
The baseline is timed here only; nothing in the package calls it.
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def main(argv=None):
    from turbo_dllm_b200.ops.attention import (attention_backward_native, attention_forward_native,
                                               single_sequence_layout)

    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--block", type=int, default=32)
    ap.add_argument("--views", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--fwd-only", action="store_true")
    ap.add_argument("--bwd-modes", default="fused,split", help="backward variants to time (TDLLM_ATTN_BWD values)")
    ap.add_argument("--baseline", default="none", choices=("none", "sdpa", "flex"),
                    help="also time the same mask through stock PyTorch attention")
    args = ap.parse_args(argv)
    D = 128
    dev = "cuda"
    layout = single_sequence_layout(args.seq, args.block, dev, args.views)
    n = (args.views + 1) * args.seq
    B = args.seq // args.block
    pairs = args.views * (args.block ** 2) * B * (B + 1) // 2 + (args.block ** 2) * B * (B + 1) // 2
    qkv = (torch.randn(n, (args.heads + 2 * args.kv_heads) * D, device=dev) * 0.5).bfloat16()
    q = qkv[:, : args.heads * D].view(n, args.heads, D)
    k = qkv[:, args.heads * D:(args.heads + args.kv_heads) * D].view(n, args.kv_heads, D)
    v = qkv[:, (args.heads + args.kv_heads) * D:].view(n, args.kv_heads, D)
    scale = 1 / math.sqrt(D)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    layout.tile_lists()

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2]

    out, lse = attention_forward_native(q, k, v, layout, scale)
    fwd_ms = timeit(lambda: attention_forward_native(q, k, v, layout, scale))
    rec = {"seq": args.seq, "block": args.block, "views": args.views, "heads": args.heads,
           "kv_heads": args.kv_heads, "pairs": pairs,
           "visited_tile_pairs": layout.tile_lists()["visited_tiles"],
           "fwd_ms": round(fwd_ms, 3),
           "fwd_tflops_exact_pairs": round(4.0 * pairs * D * args.heads / fwd_ms / 1e9, 1),
           "fwd_tflops_visited_tiles": round(4.0 * layout.tile_lists()["visited_tiles"] * 128 * 128 * D
                                             * args.heads / fwd_ms / 1e9, 1)}
    if not args.fwd_only:
        dout = torch.randn_like(out)
        dqkv = torch.empty_like(qkv)
        import os

        for mode in args.bwd_modes.split(","):
            os.environ["TDLLM_ATTN_BWD"] = mode
            bwd_ms = timeit(lambda: attention_backward_native(q, k, v, out, dout, lse, layout, scale, dqkv))
            rec[f"bwd_{mode}_ms"] = round(bwd_ms, 3)
            rec[f"bwd_{mode}_tflops_exact_pairs"] = round(10.0 * pairs * D * args.heads / bwd_ms / 1e9, 1)
    if args.baseline != "none":
        rec.update(_baseline(args.baseline, layout, q, k, v, scale, timeit, pairs, D, args.heads))
        if "baseline_fwd_ms" in rec:
            rec["fwd_speedup_vs_baseline"] = round(rec["baseline_fwd_ms"] / fwd_ms, 2)
            best = min((rec[f"bwd_{m}_ms"] for m in args.bwd_modes.split(",") if f"bwd_{m}_ms" in rec), default=None)
            if best and "baseline_bwd_ms" in rec:
                rec["bwd_speedup_vs_baseline"] = round(rec["baseline_bwd_ms"] / best, 2)
    print(json.dumps(rec), flush=True)


def _baseline(kind, layout, q, k, v, scale, timeit, pairs, D, heads):
    """Forward and backward of stock PyTorch attention under the same mask. q [n, Hq, D], k/v [n, Hkv, D]."""
    import torch.nn.functional as F

    n = q.shape[0]
    qb = q.permute(1, 0, 2)[None].contiguous().requires_grad_()      # [1, H, n, D]
    kb = k.permute(1, 0, 2)[None].contiguous().requires_grad_()
    vb = v.permute(1, 0, 2)[None].contiguous().requires_grad_()
    note = {}
    fn = None
    if kind == "flex":
        try:
            from torch.nn.attention.flex_attention import create_block_mask, flex_attention

            lo, hi, grp, code = (t.long() for t in (layout.q_lo, layout.q_hi, layout.q_grp, layout.k_code))

            def visible(b, h, qi, ki):
                c = code[ki]
                return torch.where(c >= 0, (c >= lo[qi]) & (c < hi[qi]), c == grp[qi])

            bm = create_block_mask(visible, None, None, n, n, device=q.device)
            compiled = torch.compile(flex_attention)
            fn = lambda: compiled(qb, kb, vb, block_mask=bm, scale=scale, enable_gqa=True)
            fn()
            torch.cuda.synchronize()
        except Exception as e:      # no Triton tool chain for this device, or the compile failed
            note["baseline_flex_unavailable"] = f"{type(e).__name__}: {str(e)[:160]}"
            fn, kind = None, "sdpa"
    if fn is None:
        dense = layout.dense_mask()[None, None]
        fn = lambda: F.scaled_dot_product_attention(qb, kb, vb, attn_mask=dense, scale=scale, enable_gqa=True)
    out = fn()
    dout = torch.randn_like(out)
    fwd = timeit(lambda: fn())

    def fwd_bwd():
        o = fn()
        o.backward(dout)
        qb.grad = kb.grad = vb.grad = None

    both = timeit(fwd_bwd)
    bwd = max(both - fwd, 1e-6)
    return {**note, "baseline": kind, "baseline_fwd_ms": round(fwd, 3), "baseline_bwd_ms": round(bwd, 3),
            "baseline_fwd_tflops_exact_pairs": round(4.0 * pairs * D * heads / fwd / 1e9, 1),
            "baseline_bwd_tflops_exact_pairs": round(10.0 * pairs * D * heads / bwd / 1e9, 1)}


if __name__ == "__main__":
    main()
