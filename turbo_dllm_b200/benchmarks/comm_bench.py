"""Times the peer-memory kernels against their NVLink roofline, one process per GPU.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m turbo_dllm_b200.benchmarks.comm_bench --params 2000000000 --kv-rows 16384

Rank 0 prints one JSON line per kernel. Device time is taken with CUDA events around the launch,
after warm-up, and reduced with MAX over ranks. Roofline: the bytes that must cross NVLink per GPU
and direction, divided by the measured peer-copy bandwidth of this pool (770 GB/s per direction).

* fused ZeRO step (`csrc/comm.cu::tdllm_zero_fused_step`): every rank pulls its shard of the bf16
  gradients from the W-1 peers ((W-1)/W · 2P bytes in) and pushes its updated bf16 parameter shard
  to them ((W-1)/W · 2P bytes out); the AdamW update of the shard (16 bytes per owned parameter of
  HBM traffic) runs between the two.
* clean K|V gather (`tdllm_kv_gather`): every rank pulls the other ranks' rows once.
* its NCCL twins (`reduce_scatter` + `all_gather`, `all_gather`) on the same sizes.
* sequence-parallel forms: all-gather -> GEMM with the pull inside the kernel (`tdllm_gemm_allgather_bf16`) and
  GEMM -> reduce-scatter from the epilogue (`tdllm_gemm_reduce_scatter_bf16`) against NCCL + GEMM; expert
  dispatch + combine over peer memory (`csrc/moe_dispatch.cu`) against the all-to-all twin.
* row-parallel GEMM with the all-reduce in its epilogue (`tdllm_gemm_allreduce_bf16`) against the same GEMM
  followed by an NCCL all-reduce; its roofline is the slower of FLOPs ÷ measured GEMM peak and pushed bytes ÷ 770 GB/s.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

PEER_GBS = 770.0


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None):
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.models.dense import FlatParams
    from turbo_dllm_b200.optim.flat_adamw import FlatAdamW
    from turbo_dllm_b200.parallel.context_attention import PeerKVExchange
    from turbo_dllm_b200.parallel.fused_zero import FusedZeroSync

    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, default=2_000_000_000, help="bf16 parameters in the flat buffer")
    ap.add_argument("--kv-rows", type=int, default=16384, help="clean rows owned by every rank")
    ap.add_argument("--kv-row-elems", type=int, default=2048, help="K|V elements per row (2 * kv heads * head dim)")
    ap.add_argument("--tp-rows", type=int, default=32768, help="rows of the row-parallel products")
    ap.add_argument("--tp-hidden", type=int, default=4096)
    ap.add_argument("--tp-k", type=int, nargs="+", default=[4096, 12288], help="full K of the products (split over ranks)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    group = dist.group.WORLD
    out = []

    # ---- fused ZeRO step vs reduce_scatter + AdamW + all_gather
    n = (args.params // (world * 1024)) * world * 1024
    flat = FlatParams([("w", (n,), True)], torch.bfloat16, dev)
    flat.data.normal_(0, 0.02)
    sync = FusedZeroSync.create(flat, group)
    opt = FlatAdamW(flat, lr=1e-4, group=group, fused_sync=sync)
    flat.grad.normal_(0, 1e-3)

    def fused():
        opt.step(lr=1e-4, weight_decay=0.0, max_grad_norm=1.0)

    ms = _time(fused, args.iters, args.warmup)
    cross = (world - 1) / world * 2 * n      # bytes per direction per GPU, each phase
    out.append({"kernel": "zero_fused_step (pull-reduce + clip + AdamW + push)", "world": world, "params": n,
                "ms": round(ms, 3), "nvlink_bytes_in": cross, "nvlink_bytes_out": cross,
                "roofline_ms": round(2 * cross / (PEER_GBS * 1e9) * 1e3, 3),
                "fraction_of_roofline": round(2 * cross / (PEER_GBS * 1e9) * 1e3 / ms, 3),
                "note": "roofline = gradient pull then parameter push, each (W-1)/W*2P bytes at 770 GB/s per direction"})
    native.raise_on_device_error()
    sync_opt = opt
    # NCCL twin on separate buffers of the same size
    g = torch.randn(n, device=dev, dtype=torch.bfloat16) * 1e-3
    shard = torch.empty(n // world, device=dev, dtype=torch.bfloat16)
    full = torch.empty(n, device=dev, dtype=torch.bfloat16)

    def nccl():
        dist.reduce_scatter_tensor(shard, g, group=group)
        dist.all_gather_into_tensor(full, shard, group=group)

    ms2 = _time(nccl, args.iters, args.warmup)
    out.append({"kernel": "nccl reduce_scatter + all_gather (no optimizer math)", "world": world, "params": n,
                "ms": round(ms2, 3), "fraction_of_roofline": round(2 * cross / (PEER_GBS * 1e9) * 1e3 / ms2, 3)})
    del g, shard, full
    sync.close()
    del sync_opt, opt, flat
    torch.cuda.empty_cache()

    # ---- clean K|V gather vs all_gather
    counts = [args.kv_rows] * world
    ex = PeerKVExchange(group, dev, counts, args.kv_row_elems)
    x = torch.randn(args.kv_rows, args.kv_row_elems, device=dev).bfloat16()
    ms3 = _time(lambda: ex.gather(x), args.iters, args.warmup)
    pulled = (world - 1) * args.kv_rows * args.kv_row_elems * 2
    out.append({"kernel": "kv_gather (peer pull into local memory, includes the staging copy)", "world": world,
                "rows_per_rank": args.kv_rows, "ms": round(ms3, 3), "nvlink_bytes_in": pulled,
                "roofline_ms": round(pulled / (PEER_GBS * 1e9) * 1e3, 3),
                "fraction_of_roofline": round(pulled / (PEER_GBS * 1e9) * 1e3 / ms3, 3)})
    native.raise_on_device_error()
    full = torch.empty(world * args.kv_rows, args.kv_row_elems, device=dev, dtype=torch.bfloat16)
    ms4 = _time(lambda: dist.all_gather_into_tensor(full, x, group=group), args.iters, args.warmup)
    out.append({"kernel": "nccl all_gather of the same rows", "world": world, "ms": round(ms4, 3),
                "fraction_of_roofline": round(pulled / (PEER_GBS * 1e9) * 1e3 / ms4, 3)})
    ex.close()
    del full, x
    torch.cuda.empty_cache()

    # ---- row-parallel GEMM with the all-reduce in its epilogue vs GEMM + NCCL all-reduce
    from turbo_dllm_b200.ops.gemm import gemm
    from turbo_dllm_b200.parallel.fused_allreduce import FusedAllReduceGemm

    peaks_tflops = 1604.6   # measured cuBLAS bf16 burst rate of this pool
    M, N = args.tp_rows, args.tp_hidden
    ws = FusedAllReduceGemm(group, dev, M, N)
    for k_full in args.tp_k:
        K = k_full // world
        a = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        res = torch.randn(M, N, device=dev).bfloat16()
        o1 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms_f = _time(lambda: ws.matmul(a, w, residual=res, out=o1), args.iters, args.warmup)
        native.raise_on_device_error()

        def twin():
            o = gemm(a, w, residual=res if rank == 0 else None)
            dist.all_reduce(o, group=group)
            return o

        ms_n = _time(twin, args.iters, args.warmup)
        flops = 2.0 * M * N * K
        link = (world - 1) * M * N * 2
        roof = max(flops / (peaks_tflops * 1e12), link / (PEER_GBS * 1e9)) * 1e3
        out.append({"kernel": "gemm_allreduce (tcgen05 tiles + peer stores in one kernel)", "world": world,
                    "shape": f"{M}x{N}x{K} per rank", "ms": round(ms_f, 3), "gemm_plus_nccl_allreduce_ms": round(ms_n, 3),
                    "tflops_per_gpu": round(flops / ms_f / 1e9, 1), "nvlink_bytes_out": link,
                    "roofline_ms": round(roof, 3), "fraction_of_roofline": round(roof / ms_f, 3),
                    "bound": "compute" if flops / (peaks_tflops * 1e12) > link / (PEER_GBS * 1e9) else "nvlink"})
    ws.close()
    torch.cuda.empty_cache()

    # ---- sequence-parallel forms: all-gather -> GEMM (remote rows pulled inside the GEMM kernel) and
    #      GEMM -> reduce-scatter (partial tiles pushed to their owner from the epilogue) against NCCL + GEMM
    from turbo_dllm_b200.parallel.fused_sequence_parallel import FusedSequenceParallel

    H = args.tp_hidden
    Mr = (args.tp_rows // (256 * world)) * 256 * world
    sp = FusedSequenceParallel(group, dev, Mr, H)
    for k_full in args.tp_k:
        Nl = k_full // world                       # column-parallel width per rank (QKV or gate/up shard)
        x_loc = (torch.randn(Mr // world, H, device=dev) * 0.5).bfloat16()
        w_col = (torch.randn(Nl, H, device=dev) * 0.05).bfloat16()
        ms_ag = _time(lambda: sp.gather_matmul(x_loc, w_col), args.iters, args.warmup)
        native.raise_on_device_error()
        full = torch.empty(Mr, H, device=dev, dtype=torch.bfloat16)

        def ag_twin():
            dist.all_gather_into_tensor(full, x_loc, group=group)
            return gemm(full, w_col)

        ms_ag_n = _time(ag_twin, args.iters, args.warmup)
        flops = 2.0 * Mr * Nl * H
        link = (world - 1) * (Mr // world) * H * 2
        roof = max(flops / (peaks_tflops * 1e12), link / (PEER_GBS * 1e9)) * 1e3
        out.append({"kernel": "allgather_gemm (peer pull by extra warps of the tcgen05 GEMM)", "world": world,
                    "shape": f"{Mr}x{Nl}x{H} per rank", "ms": round(ms_ag, 3), "nccl_allgather_plus_gemm_ms": round(ms_ag_n, 3),
                    "tflops_per_gpu": round(flops / ms_ag / 1e9, 1), "nvlink_bytes_in": link, "roofline_ms": round(roof, 3),
                    "fraction_of_roofline": round(roof / ms_ag, 3),
                    "bound": "compute" if flops / (peaks_tflops * 1e12) > link / (PEER_GBS * 1e9) else "nvlink"})
        a_row = (torch.randn(Mr, Nl, device=dev) * 0.5).bfloat16()           # row-parallel input [rows, K/W]
        w_row = (torch.randn(H, Nl, device=dev) * 0.05).bfloat16()
        res = torch.randn(Mr // world, H, device=dev).bfloat16()
        ms_rs = _time(lambda: sp.matmul_scatter(a_row, w_row, residual=res), args.iters, args.warmup)
        native.raise_on_device_error()
        shard = torch.empty(Mr // world, H, device=dev, dtype=torch.bfloat16)

        def rs_twin():
            dist.reduce_scatter_tensor(shard, gemm(a_row, w_row), group=group)
            return shard.add_(res)

        ms_rs_n = _time(rs_twin, args.iters, args.warmup)
        flops = 2.0 * Mr * H * Nl
        link = (world - 1) * (Mr // world) * H * 2
        roof = max(flops / (peaks_tflops * 1e12), link / (PEER_GBS * 1e9)) * 1e3
        out.append({"kernel": "gemm_reduce_scatter (tcgen05 tiles pushed to their owner from the epilogue)",
                    "world": world, "shape": f"{Mr}x{H}x{Nl} per rank", "ms": round(ms_rs, 3),
                    "gemm_plus_nccl_reduce_scatter_ms": round(ms_rs_n, 3), "tflops_per_gpu": round(flops / ms_rs / 1e9, 1),
                    "nvlink_bytes_out": link, "roofline_ms": round(roof, 3), "fraction_of_roofline": round(roof / ms_rs, 3),
                    "bound": "compute" if flops / (peaks_tflops * 1e12) > link / (PEER_GBS * 1e9) else "nvlink"})
        del x_loc, w_col, full, a_row, w_row, res, shard
    sp.close()
    torch.cuda.empty_cache()

    # ---- expert dispatch + combine over peer memory against the all-to-all twin (same routing, no expert math)
    from turbo_dllm_b200.models.moe import _AllToAllRows
    from turbo_dllm_b200.parallel.expert_exchange import PeerExpertExchange, peer_combine, peer_dispatch

    rows, Hm, E, topk = 16384, 2048, 8 * world, 4
    torch.manual_seed(1234 + rank)
    xm = (torch.randn(rows, Hm, device=dev) * 0.5).bfloat16()
    idx = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(64)]).repeat(rows // 64, 1)
    wts = torch.full((rows, topk), 1.0 / topk, device=dev)
    exm = PeerExpertExchange(group, dev, rows=rows, top_k=topk, hidden=Hm, num_experts=E)
    flat32 = idx.reshape(-1).to(torch.int32).contiguous()

    def ep_peer():
        with torch.no_grad():
            st: dict = {}
            x_pad = peer_dispatch(xm, flat32, exm, st)
            return peer_combine(x_pad, wts, exm, st)

    ms_ep = _time(ep_peer, args.iters, args.warmup)
    native.raise_on_device_error()
    el = E // world

    def ep_twin():
        with torch.no_grad():
            flat_e = idx.reshape(-1)
            order = torch.argsort(flat_e, stable=True)
            token_of = torch.div(order, topk, rounding_mode="floor")
            x_perm = xm.index_select(0, token_of)
            counts_g = torch.bincount(flat_e, minlength=E)
            allc = torch.empty(world, E, dtype=counts_g.dtype, device=dev)
            dist.all_gather_into_tensor(allc.view(-1), counts_g, group=group)
            mine = allc[:, rank * el:(rank + 1) * el]
            sizes = torch.cat([counts_g.view(world, el).sum(1), mine.sum(1)]).tolist()
            recv = _AllToAllRows.apply(x_perm, sizes[:world], sizes[world:], group)
            back = _AllToAllRows.apply(recv, sizes[world:], sizes[:world], group)
            outm = torch.zeros_like(xm)
            outm.index_add_(0, token_of, back * wts.reshape(-1).index_select(0, order).to(back.dtype)[:, None])
            return outm

    ms_ep_n = _time(ep_twin, args.iters, args.warmup)
    link = rows * topk * Hm * 2 * (world - 1) / world          # per direction, dispatch; the same again for combine
    out.append({"kernel": "expert dispatch + combine (peer stores into owner slabs, pull-combine)", "world": world,
                "rows": rows, "top_k": topk, "hidden": Hm, "experts": E, "ms": round(ms_ep, 3),
                "all_to_all_twin_ms": round(ms_ep_n, 3), "nvlink_bytes_each_way": link,
                "roofline_ms": round(2 * link / (PEER_GBS * 1e9) * 1e3, 3),
                "fraction_of_roofline": round(2 * link / (PEER_GBS * 1e9) * 1e3 / ms_ep, 3),
                "note": "roofline = dispatched rows out, then combined rows back, each at 770 GB/s per direction"})
    exm.close()
    if rank == 0:
        for rec in out:
            print(json.dumps(rec), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
