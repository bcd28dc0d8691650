"""Issue cost of one tcgen05.mma (128 x N x 16, bf16) for the single issuing thread.

    python -m turbo_dllm_b200.benchmarks.mma_issue_bench

One JSON line per (N, operand form): cycles per MMA spent by the issuing thread, cycles per MMA
until completion, and the ideal tensor-pipe cycles (128·N·16 MACs at 4096 MACs per cycle per SM).
When the issue cost is above the ideal, a kernel built from MMAs of that size is issue-bound.
"""
from __future__ import annotations

import argparse
import ctypes
import json

import torch


def main(argv=None):
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops._util import ptr, stream

    native.register_signatures({
        "tdllm_mma_issue_probe": (native.c_int, [native.c_int] * 6 + [native.c_void_p, native.c_void_p]),
    })
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=4096)
    ap.add_argument("--ctas", type=int, default=1)
    args = ap.parse_args(argv)
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    for n in (32, 64, 128, 256):
        for a_tmem, accs, uniform in ((0, 1, 0), (1, 1, 0), (0, 1, 1), (1, 1, 1), (0, 2, 1), (0, 4, 1)):
            if accs * n > 256:
                continue
            for _ in range(2):
                native.check(native.lib().tdllm_mma_issue_probe(n, args.iters, a_tmem, accs, uniform, args.ctas,
                                                                ptr(out), stream()), "mma_issue_probe")
                torch.cuda.synchronize()
            native.raise_on_device_error()
            issue, done = (int(v) for v in out.tolist())
            print(json.dumps({"n": n, "a_operand": "tmem" if a_tmem else "smem", "accumulators": accs,
                              "issue": "elected lane, warp-uniform loop" if uniform else "lane 0, divergent loop",
                              "iters": args.iters,
                              "ctas": args.ctas, "issue_cycles_per_mma": round(issue / args.iters, 2),
                              "complete_cycles_per_mma": round(done / args.iters, 2),
                              "ideal_tensor_cycles_per_mma": 128 * n * 16 / 4096}), flush=True)


if __name__ == "__main__":
    main()
