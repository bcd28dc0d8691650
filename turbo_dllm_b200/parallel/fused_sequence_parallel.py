"""Sequence-parallel projections as single kernels over peer memory.

`gather_matmul`  : y = all_gather_rows(x_local) · Wᵀ. This rank's rows are copied into its slot of a symmetric
                   [rows, K] buffer and announced to the peers; the GEMM kernel's extra warps pull the peers' slots
                   into the same buffer while the tiles of local rows already run (csrc/gemm_sm100.cu, all-gather
                   form). The gathered rows come back as a view of that buffer (the weight-gradient product of the
                   backward pass reads them).
`matmul_scatter` : y_local = rows of this rank of Σ_ranks x_r · W_rᵀ (+ residual_local): the GEMM's epilogue pushes
                   every tile to its owner and only owners store (reduce-scatter form of the all-reduce epilogue).

Buffers. Gather buffers rotate (six by default): a rank can be at most one call ahead of its slowest peer, so two
would be enough against overwriting rows a peer still pulls; the others keep the gathered inputs of one decoder
layer alive until its backward pass has used them (with activation checkpointing a layer is recomputed and
back-propagated before the next one is touched; without it callers clone what they save). Reduce-scatter
workspaces alternate between two, as for the all-reduce GEMM.

Counterpart: Transformer Engine userbuffers (`ub_overlap_ag`, `ub_overlap_rs`) as configured in
dllm_parallel/core/parallel/transformer_engine.py:84-139.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..kernels import native
from ..ops._util import ptr, stream
from ..profiling.operator_trace import communication_scope
from .symm import SymmetricBuffer, peer_access_available

_V, _I, _LL = native.c_void_p, native.c_int, native.c_ll
native.register_signatures({
    "tdllm_symm_signal": (_I, [_V, _I, _I, _I, _V]),
    "tdllm_gemm_reduce_scatter_bf16": (_I, [_V] * 3 + [_I] * 3 + [_LL] * 3 + [_I] * 2 + [_V, _LL] + [_I] * 3
                                       + [_LL, _V, _V, _I, _V]),
    "tdllm_gemm_allgather_bf16": (_I, [_V] * 3 + [_I] * 3 + [_LL] * 2 + [_I] * 5 + [_V, _V, _V, _I, _I, _V]),
    "tdllm_gemm_flag_count": (_I, [_I, _I]),
})

MAX_RANKS = 8
EPI_STORE, EPI_SWIGLU = 0, 1


class FusedSequenceParallel:
    def __init__(self, group, device: torch.device, rows: int, cols: int, gather_buffers: int = 6):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= MAX_RANKS:
            raise RuntimeError(f"fused sequence parallelism supports 2..{MAX_RANKS} ranks, got {self.world}")
        if rows % (256 * self.world) or cols % 64:
            raise RuntimeError("fused sequence parallelism needs row shards of whole 256-row tiles and a width that "
                               "is a multiple of 64")
        if not peer_access_available(group):
            raise RuntimeError("GPUs of this group cannot address one another (no peer access)")
        self.rows, self.cols, self.n = int(rows), int(cols), int(rows) // self.world
        self.gbufs = [SymmetricBuffer(rows * cols * 2, group, device) for _ in range(max(2, gather_buffers))]
        self.gi = 0
        self.ready = SymmetricBuffer(256, group, device)
        self.tile_ready = torch.zeros(rows // 128 + 1, dtype=torch.int32, device=device)
        self.counter = self.tile_ready[-1:]
        self.gather_calls = 0
        nflags = native.lib().tdllm_gemm_flag_count(rows, cols)
        self.ws = [SymmetricBuffer(self.world * self.n * cols * 2, group, device) for _ in range(2)]
        self.flags = [SymmetricBuffer(self.world * nflags * 4, group, device) for _ in range(2)]
        for f in self.flags:
            f.as_tensor(torch.int32).zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self.epoch = [0, 0]
        self.flip = 0

    def gather_matmul(self, x_local: torch.Tensor, w: torch.Tensor, b_mn_major: bool = False,
                      swiglu: bool = False):
        """x_local [rows/world, K] (this rank's rows), w [N, K] (or [K, N] with `b_mn_major`) ->
        (y [rows, N] or [rows, N/2] with `swiglu`, gathered x [rows, K] as a view of the rotating buffer)."""
        n, K = x_local.shape
        N = w.shape[1] if b_mn_major else w.shape[0]
        if n != self.n or K != self.cols or (w.shape[0] if b_mn_major else w.shape[1]) != K:
            raise ValueError(f"gather_matmul: [{n},{K}] x {tuple(w.shape)} outside this workspace "
                             f"({self.n} rows per rank, width {self.cols})")
        if x_local.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.stride(1) != 1:
            raise ValueError("gather_matmul takes row-major bf16 operands")
        buf = self.gbufs[self.gi]
        self.gi = (self.gi + 1) % len(self.gbufs)
        full = buf.as_tensor(torch.bfloat16, self.rows * K).view(self.rows, K)
        full[self.rank * n:(self.rank + 1) * n].copy_(x_local)
        self.gather_calls += 1
        c = self.gather_calls
        lib = native.lib()
        native.check(lib.tdllm_symm_signal(self.ready.ptr_array, self.rank, self.world, c, stream()), "symm_signal")
        out = torch.empty(self.rows, N // 2 if swiglu else N, dtype=torch.bfloat16, device=x_local.device)
        with communication_scope("tensor", "forward", "allgather_gemm", (self.world - 1) * n * K * 2,
                                 self.rows * K * 2):
            native.check(lib.tdllm_gemm_allgather_bf16(
                buf.ptr_array, ptr(w), ptr(out), self.rows, N, K, w.stride(0), out.stride(0), int(b_mn_major),
                EPI_SWIGLU if swiglu else EPI_STORE, self.world, self.rank, c, self.ready.ptr_array,
                ptr(self.counter), ptr(self.tile_ready), c, 0, stream()), "gemm_allgather")
        return out, full

    def matmul_scatter(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
                       b_mn_major: bool = False) -> torch.Tensor:
        """x [rows, K_local] · w[N, K_local]ᵀ (or · w[K_local, N]) summed over the group, rows of this rank only
        (+ residual [rows/world, N]) -> [rows/world, N] bf16."""
        M, K = x.shape
        N = w.shape[1] if b_mn_major else w.shape[0]
        if M != self.rows or N != self.cols or (w.shape[0] if b_mn_major else w.shape[1]) != K:
            raise ValueError(f"matmul_scatter: [{M},{K}] x {tuple(w.shape)} outside this workspace "
                             f"({self.rows} rows, width {self.cols})")
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1:
            raise ValueError("matmul_scatter takes row-major bf16 operands")
        out = torch.empty(self.n, N, dtype=torch.bfloat16, device=x.device)
        b = self.flip
        self.flip ^= 1
        self.epoch[b] += 1
        with communication_scope("tensor", "forward", "gemm_reduce_scatter", (self.world - 1) * self.n * N * 2):
            native.check(native.lib().tdllm_gemm_reduce_scatter_bf16(
                ptr(x), ptr(w), ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0), 0, int(b_mn_major),
                ptr(residual) if residual is not None else None, residual.stride(0) if residual is not None else 0,
                self.world, self.rank, self.epoch[b], self.n, self.ws[b].ptr_array, self.flags[b].ptr_array, 0,
                stream()), "gemm_reduce_scatter")
        return out

    def close(self) -> None:
        for b in (*self.gbufs, self.ready, *self.ws, *self.flags):
            b.close()
