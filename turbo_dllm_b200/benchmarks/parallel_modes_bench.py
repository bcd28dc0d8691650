"""Compares the three ways of spreading one long sequence over W ranks, with identical settings:

* `pure_cp`   : context parallelism W: clean K/V sharded and the tokens INSIDE every noisy block divided over the
                ranks (two-ended), all K/V rows exchanged (`pure_cp_replicated`: the variant that keeps every
                noisy block whole on every rank, W-fold redundant noisy work, for comparison),
* `pure_bp`   : block parallelism W with a replicated clean prefix (no K/V exchange, redundant clean work),
* `csbp`      : context-sharded block parallelism, CP = BP = W (the fused layout).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m turbo_dllm_b200.benchmarks.parallel_modes_bench --config turbo_dllm_b200/recipes/examples/csbp8-qwen3-1p7b-128k.yaml

The config's topology section is overridden per mode; everything else (model, sequence length, objective,
optimizer) stays the same. Rank 0 prints one JSON line per mode: ms/step (MAX over ranks; CUDA events on
GPUs, wall clock on CPU), input tokens/s of the whole job, peak device memory, and the loss of the last step,
which must agree between modes up to rounding because all three compute the same function.

Reference counterpart: benchmarks/profile_parallel_modes.sh:4-24 (pure CP / replicated-prefix BP / fused CP+BP
with identical settings).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

MODES = {
    "pure_cp": lambda w: {"context_parallel_size": w, "block_parallel_size": 1, "replicate_clean_prefix": False},
    "pure_cp_replicated": lambda w: {"context_parallel_size": w, "block_parallel_size": 1,
                                     "replicate_clean_prefix": False},
    "pure_bp": lambda w: {"context_parallel_size": 1, "block_parallel_size": w, "replicate_clean_prefix": True},
    "csbp": lambda w: {"context_parallel_size": w, "block_parallel_size": w, "replicate_clean_prefix": False},
}


def run_mode(spec, mode: str, *, device, steps: int, warmup: int, transport: str | None = None) -> dict:
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    world = dist.get_world_size()
    kernel = {"pure_cp_token_split": mode != "pure_cp_replicated"}
    if transport:
        kernel["cp_bp_clean_kv_transport"] = transport
    s = spec.with_overrides({"topology": MODES[mode](world), "kernel": kernel}).validate(world_size=world)
    rt = build_parallel_runtime(s, device=device)
    session = TrainingSession(s, device=device, runtime=rt)
    cuda = torch.device(device).type == "cuda"
    for _ in range(warmup):
        session.step()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
    dist.barrier()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    t0 = time.perf_counter()
    last = None
    for _ in range(steps):
        last = session.step()
    if cuda:
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / steps
    stats = torch.tensor([ms, torch.cuda.max_memory_allocated() / 2 ** 20 if cuda else 0.0], dtype=torch.float64,
                         device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    loss = last.loss_sum.double().clone()
    dist.all_reduce(loss)
    tokens = s.model.seq_len * s.training.batch_size * rt.data_parallel_size
    out = {"mode": mode, "world": world, "transport": s.kernel.cp_bp_clean_kv_transport, "topology": MODES[mode](world), "ms_per_step": round(float(stats[0]), 3),
           "input_tokens_per_s": round(tokens / float(stats[0]) * 1e3, 1), "peak_mib": round(float(stats[1]), 1),
           "loss": float(loss) / last.denominator, "seq_len": s.model.seq_len, "steps": steps, "warmup": warmup}
    session.close()
    del session
    if cuda:
        torch.cuda.empty_cache()
    return out


def main(argv=None) -> int:
    from turbo_dllm_b200.config.run_spec import load_run_spec

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--modes", nargs="+", default=["pure_cp", "pure_bp", "csbp"], choices=list(MODES))
    ap.add_argument("--transport", default=None, choices=("collective", "fused"),
                    help="clean K/V transport of the context-parallel modes (default: the config's)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=None)
    a = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", rank))
    cuda = torch.cuda.is_available()
    device = f"cuda:{local}" if cuda else "cpu"
    if cuda:
        torch.cuda.set_device(local)
    own = not dist.is_initialized()
    if own:
        dist.init_process_group("nccl" if cuda else "gloo")
    spec = load_run_spec(a.config)
    if a.seq_len:
        spec = spec.with_overrides({"model": {"seq_len": a.seq_len}})
    for mode in a.modes:
        rec = run_mode(spec, mode, device=device, steps=a.steps, warmup=a.warmup, transport=a.transport)
        if rank == 0:
            print(json.dumps(rec), flush=True)
    if own:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
