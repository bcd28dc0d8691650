"""Times one layer's context-sharded attention (forward, forward + backward) per transport, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m turbo_dllm_b200.benchmarks.csbp_attention_bench --seq 131072 --block 64 --heads 16 --kv-heads 8

Context- and block-parallel degree = number of ranks. Every rank holds the packed q|k|v rows of its noisy
blocks and of its clean shard (random values) and runs the attention of `parallel/context_attention.py` with
each transport: `collective` (NCCL all-gather, attention kernel, NCCL reduce-scatter), `peer_pull` (the same
with stand-alone peer-memory copy kernels) and `fused` (the transfer inside the attention kernels). Device
time is taken with CUDA events after warm-up, with a barrier before every timed call, and reduced with MAX over
ranks. Rank 0 prints one JSON line per transport with

* FLOPs on the exactly visible query-key pairs of the slowest rank (4·pairs·D per head forward, 10·pairs·D
  backward);
* the bytes that must cross NVLink per GPU: forward, every remote clean K|V row once (bf16, inbound); backward,
  the fp32 dK|dV partial sums of the remote rows this rank's queries see (outbound);
* `--emulate-peers W` runs rank 0 of a W-rank group in ONE process on one GPU: the peers' staged rows, ready flags
  and gradient accumulators are buffers of the same GPU, so the fused kernels execute exactly the code of a
  W-rank run (pull warps, arrival counters, peer adds) with HBM in place of NVLink. This is the form a profiler
  can capture (a profiler must not wrap a multi-rank command).
* roofline = the slower of FLOPs ÷ the measured bf16 GEMM burst rate and NVLink bytes ÷ 770 GB/s (measured
  peer-copy bandwidth per direction), and the achieved fraction.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

PEER_GBS = 770.0
PEAK_TFLOPS = 1604.6     # measured cuBLAS bf16 burst rate of this pool's B200s


class _LocalBuffers:
    """Stand-in for a symmetric buffer when every "rank" lives on this GPU: one tensor per emulated rank."""

    def __init__(self, nbytes: int, world: int, dev, fill: int | None = None, shared: bool = False):
        import ctypes

        n = (nbytes + 3) // 4
        first = torch.zeros(n, dtype=torch.int32, device=dev)
        self.tensors = [first if (shared or r == 0) else torch.zeros(n, dtype=torch.int32, device=dev)
                        for r in range(world)]
        if fill is not None:
            for t in self.tensors:
                t.fill_(fill)
        self.ptrs = [t.data_ptr() for t in self.tensors]
        self.local = self.ptrs[0]
        self.ptr_array = (ctypes.c_void_p * world)(*self.ptrs)
        self.rank, self.world = 0, world

    def as_tensor(self, dtype, numel=None, offset_bytes: int = 0):
        t = self.tensors[0].view(torch.uint8)[offset_bytes:].view(dtype)
        return t if numel is None else t[:numel]

    def close(self):
        self.tensors = []


def emulate(args):
    """Rank 0 of an `args.emulate_peers`-rank context group in one process (see the module docstring)."""
    import ctypes

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.parallel import context_attention as ca
    from turbo_dllm_b200.parallel.layout import build_packed_layout, clean_positions_for_rank
    from turbo_dllm_b200.parallel.schedule import build_block_schedule
    from dataclasses import replace

    W, D = args.emulate_peers, 128
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = replace(PRESETS["synthetic:qwen3-1.7b"], num_attention_heads=args.heads, num_key_value_heads=args.kv_heads)
    sched = build_block_schedule(args.seq // args.block, W)
    kpos = [clean_positions_for_rank(args.seq, W, r, "dual_chunk", args.block, dev) for r in range(W)]
    kseq = [torch.zeros_like(p) for p in kpos]
    counts = [int(p.numel()) for p in kpos]
    layout = build_packed_layout(seq_len=args.seq, block_size=args.block, batch=1, views=args.views,
                                 owned_blocks=list(sched.blocks_by_worker[0]), clean_pos=kpos[0], device=dev)
    kv_cols = 2 * args.kv_heads * D
    ex = object.__new__(ca.FusedKVExchange)
    ex.native, ex.device, ex.group, ex.world, ex.rank = native, dev, None, W, 0
    ex.counts, ex.kv_cols = counts, kv_cols
    ex.n_rem = sum(counts[1:])
    ex.nlt, ex.nrt = (layout.rows + 127) // 128, (ex.n_rem + 127) // 128
    ex.acc_rows = (layout.n_noisy + max(counts) + 127) // 128 * 128
    ex.staging = [_LocalBuffers(max(counts) * kv_cols * 2, W, dev) for _ in range(2)]
    for b in ex.staging:
        for t in b.tensors[1:]:
            t.view(torch.bfloat16).normal_(0, 0.5)
    half = ex.acc_rows * (kv_cols // 2) * 4
    ex.acc_bytes = 2 * half
    ex.acc = [_LocalBuffers(ex.acc_bytes, W, dev) for _ in range(2)]
    ex.acc_dk = [(ctypes.c_void_p * W)(*b.ptrs) for b in ex.acc]
    ex.acc_dv = [(ctypes.c_void_p * W)(*[p + half for p in b.ptrs]) for b in ex.acc]
    big = 1 << 30
    ex.ready = _LocalBuffers(256, W, dev, fill=big, shared=True)

    class _Barrier:
        buf = _LocalBuffers(256, W, dev, fill=big, shared=True)
        epoch = 0

        def reserve(self, n):
            self.epoch += n
            return self.epoch - n + 1

    ex.barrier = _Barrier()
    ex.counts_arr = (ctypes.c_longlong * W)(*counts)
    ex.row0_arr = (ctypes.c_longlong * W)(*([layout.n_noisy] * W))
    ex.tile_ready = torch.zeros(max(ex.nrt, 1) + 1, dtype=torch.int32, device=dev)
    ex.counter = ex.tile_ready[-1:]
    ex.fwd_calls = ex.bwd_calls = 0
    cpa = object.__new__(ca.ContextParallelAttention)
    cpa.cfg, cpa.layout, cpa.cp, cpa.cp_rank, cpa.transport, cpa.exchange = cfg, layout, W, 0, "fused", ex
    cpa.mask = ca.fused_key_layout(layout, kpos, kseq, W, 0)
    cpa.mask.tile_lists()
    rows = layout.rows
    qkv = (torch.randn(rows, (args.heads + 2 * args.kv_heads) * D, device=dev) * 0.5).bfloat16().requires_grad_(True)
    dout = torch.randn(rows, args.heads * D, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

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

    def fwd():
        with torch.no_grad():
            return cpa(qkv, 0)

    def fwd_bwd():
        qkv.grad = None
        cpa(qkv, 0).backward(dout)

    fwd_ms = timeit(fwd)
    both_ms = timeit(fwd_bwd)
    native.raise_on_device_error()
    m = layout.mask
    pairs = float((m.q_hi.long() - m.q_lo.long()).sum()) + float(layout.n_noisy * args.block)
    print(json.dumps({"mode": f"rank 0 of {W} emulated on one GPU", "seq": args.seq, "block": args.block,
                      "heads": args.heads, "kv_heads": args.kv_heads, "rows": rows, "remote_rows": ex.n_rem,
                      "fwd_ms": round(fwd_ms, 3), "fwd_bwd_ms": round(both_ms, 3),
                      "fwd_tflops": round(4.0 * pairs * D * args.heads / fwd_ms / 1e9, 1),
                      "bwd_tflops": round(10.0 * pairs * D * args.heads / (both_ms - fwd_ms) / 1e9, 1),
                      "pulled_bytes": ex.n_rem * kv_cols * 2}), flush=True)


def main(argv=None):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.models.config import model_config_from_run_spec
    from turbo_dllm_b200.parallel.context_attention import ContextParallelAttention
    from turbo_dllm_b200.parallel.layout import build_packed_layout, clean_positions_for_rank, runtime_clean_layout
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime

    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--views", type=int, default=1)
    ap.add_argument("--transports", default="collective,peer_pull,fused")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--emulate-peers", type=int, default=0,
                    help="run rank 0 of a group of this size in one process on one GPU (profiler-friendly)")
    args = ap.parse_args(argv)
    if args.emulate_peers:
        return emulate(args)

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    D = 128
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    records = []
    for transport in args.transports.split(","):
        spec = RunSpec.from_mapping({
            "model": {"id": "synthetic:qwen3-1.7b", "seq_len": args.seq, "dtype": "bf16",
                      "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads},
            "objective": {"name": "fast_dllm_v2" if args.views == 2 else "standard_block_diffusion",
                          "block_size": args.block},
            "training": {"batch_size": 1, "steps": 1},
            "topology": {"context_parallel_size": world, "block_parallel_size": world},
            "kernel": {"cp_bp_clean_kv_transport": transport}}).validate(world_size=world)
        rt = build_parallel_runtime(spec, device=dev, rank=rank, world_size=world)
        cfg = model_config_from_run_spec(spec)
        lay = runtime_clean_layout(spec.kernel.cp_bp_clean_kv_layout, world)
        clean = clean_positions_for_rank(args.seq, world, rt.context_parallel_rank, lay, args.block, dev)
        layout = build_packed_layout(seq_len=args.seq, block_size=args.block, batch=1, views=args.views,
                                     owned_blocks=rt.owned_blocks, clean_pos=clean, device=dev)
        cpa = ContextParallelAttention(cfg, layout, rt, spec)
        cpa.mask.tile_lists()
        rows = layout.rows
        qkv = (torch.randn(rows, (args.heads + 2 * args.kv_heads) * D, device=dev) * 0.5).bfloat16().requires_grad_(True)
        dout = torch.randn(rows, args.heads * D, device=dev).bfloat16()

        def fwd():
            with torch.no_grad():
                return cpa(qkv, 0)

        def fwd_bwd():
            qkv.grad = None
            cpa(qkv, 0).backward(dout)

        fwd_ms = timeit(fwd)
        both_ms = timeit(fwd_bwd)
        native.raise_on_device_error()
        # exactly visible pairs of this rank's queries: clean keys in [lo, hi) plus the noisy rows' own block
        m = layout.mask
        pairs = float((m.q_hi.long() - m.q_lo.long()).sum()) + float(layout.n_noisy * args.block)
        t = torch.tensor([pairs], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pairs = float(t)
        n_rem = args.seq - int(clean.numel())
        kv_row_bytes = 2 * args.kv_heads * D * 2
        bytes_in = n_rem * kv_row_bytes
        bytes_out = n_rem * kv_row_bytes * 2            # fp32 partial sums, each remote row at least once
        f_fwd, f_bwd = 4.0 * pairs * D * args.heads, 10.0 * pairs * D * args.heads
        roof_fwd = max(f_fwd / (PEAK_TFLOPS * 1e12), bytes_in / (PEER_GBS * 1e9)) * 1e3
        roof_bwd = max(f_bwd / (PEAK_TFLOPS * 1e12), bytes_out / (PEER_GBS * 1e9)) * 1e3
        bwd_ms = both_ms - fwd_ms
        records.append({
            "transport": transport, "world": world, "seq": args.seq, "block": args.block, "heads": args.heads,
            "kv_heads": args.kv_heads, "rows_per_rank": rows, "remote_rows": n_rem,
            "fwd_ms": round(fwd_ms, 3), "fwd_bwd_ms": round(both_ms, 3), "bwd_ms": round(bwd_ms, 3),
            "fwd_tflops_per_gpu": round(f_fwd / fwd_ms / 1e9, 1), "bwd_tflops_per_gpu": round(f_bwd / bwd_ms / 1e9, 1),
            "nvlink_bytes_in_fwd": bytes_in, "nvlink_bytes_out_bwd_min": bytes_out,
            "fwd_roofline_ms": round(roof_fwd, 3), "fwd_fraction_of_roofline": round(roof_fwd / fwd_ms, 3),
            "bwd_roofline_ms": round(roof_bwd, 3), "bwd_fraction_of_roofline": round(roof_bwd / bwd_ms, 3),
            "fwd_bound": "compute" if f_fwd / (PEAK_TFLOPS * 1e12) > bytes_in / (PEER_GBS * 1e9) else "nvlink"})
        if getattr(cpa, "exchange", None) is not None:
            torch.cuda.synchronize()
            dist.barrier()
            cpa.exchange.close()
        rt.destroy()
        del cpa, qkv, dout
        torch.cuda.empty_cache()
    if rank == 0:
        for r in records:
            print(json.dumps(r), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
