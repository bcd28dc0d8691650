"""Row-parallel GEMM with the all-reduce done inside the GEMM kernel over peer memory.

`D = Σ_ranks A_r · W_rᵀ (+ residual)`: every rank runs the same persistent tcgen05 GEMM on its K-slice;
the epilogue writes each 32×256 bf16 partial slice into the workspace of every rank with plain peer
stores, publishes a flag per (source rank, tile, warp slice), and one tile later sums the partials that
have arrived locally into the destination (csrc/gemm_sm100.cu, EPI_ALLREDUCE). Transfers of one tile
overlap the tensor-core work of the next; there is no collective call and no second kernel.

Two workspaces alternate between consecutive calls: a rank can only finish call c after every peer has
pushed its call-c partials, i.e. after every peer has left call c-1, so the buffers of call c+1 (those of
call c-1) are no longer read by anyone. Flags carry a growing epoch and are never reset.

Counterpart in the reference: Transformer Engine's userbuffers overlap of the row-parallel projections
(dllm_parallel/core/parallel/transformer_engine.py:84-139) and the reduce-from-tensor-parallel mapping
(dllm_parallel/core/parallel/mappings.py:75-185).
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..kernels import native
from ..ops._util import ptr, stream
from .symm import SymmetricBuffer, peer_access_available

native.register_signatures({
    "tdllm_gemm_allreduce_bf16": (native.c_int, [native.c_void_p] * 3 + [native.c_int] * 3 + [native.c_ll] * 3
                                  + [native.c_int] * 2 + [native.c_void_p, native.c_ll] + [native.c_int] * 3
                                  + [native.c_ll, native.c_void_p, native.c_void_p, native.c_int, native.c_void_p]),
    "tdllm_gemm_flag_count": (native.c_int, [native.c_int, native.c_int]),
    "tdllm_ce_exchange": (native.c_int, [native.c_void_p, native.c_int, native.c_int, native.c_void_p,
                                         native.c_void_p, native.c_int, native.c_int, native.c_int, native.c_ll,
                                         native.c_void_p, native.c_void_p, native.c_void_p]),
    "tdllm_ce_exchange_blocks": (native.c_int, [native.c_ll]),
})

MAX_RANKS = 8


class FusedAllReduceGemm:
    """Workspaces for products with at most `max_rows` rows and exactly `n_cols` output columns."""

    def __init__(self, group, device: torch.device, max_rows: int, n_cols: int):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= MAX_RANKS:
            raise RuntimeError(f"fused all-reduce GEMM supports 2..{MAX_RANKS} ranks, got {self.world}")
        if n_cols % 8:
            raise RuntimeError("fused all-reduce GEMM needs an output width that is a multiple of 8")
        if not peer_access_available(group):
            raise RuntimeError("GPUs of this group cannot address one another (no peer access)")
        self.max_rows, self.n_cols = int(max_rows), int(n_cols)
        nflags = native.lib().tdllm_gemm_flag_count(self.max_rows, self.n_cols)
        self.ws = [SymmetricBuffer(self.world * self.max_rows * self.n_cols * 2, group, device) for _ in range(2)]
        self.flags = [SymmetricBuffer(self.world * nflags * 4, group, device) for _ in range(2)]
        for f in self.flags:
            f.as_tensor(torch.int32).zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)   # nobody publishes an epoch into flags that are still being zeroed
        self.epoch = [0, 0]
        self.flip = 0

    def matmul(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None, b_mn_major: bool = False) -> torch.Tensor:
        """x [M, K_local] · w[N, K_local]ᵀ (or · w[K_local, N] with `b_mn_major`) summed over the group
        (+ residual [M, N]) -> [M, N] bf16."""
        M, K = x.shape
        N = w.shape[1] if b_mn_major else w.shape[0]
        if N != self.n_cols or M > self.max_rows or (w.shape[0] if b_mn_major else w.shape[1]) != K:
            raise ValueError(f"shape [{M},{K}]x[{N},{w.shape[1]}] outside this workspace ({self.max_rows} rows, "
                             f"{self.n_cols} columns)")
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1:
            raise ValueError("fused all-reduce GEMM takes row-major bf16 operands")
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        b = self.flip
        self.flip ^= 1
        self.epoch[b] += 1
        rc = native.lib().tdllm_gemm_allreduce_bf16(
            ptr(x), ptr(w), ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0), 0, int(b_mn_major),
            ptr(residual) if residual is not None else None, residual.stride(0) if residual is not None else 0,
            self.world, self.rank, self.epoch[b], self.max_rows, self.ws[b].ptr_array, self.flags[b].ptr_array,
            0, stream())
        native.check(rc, "gemm_allreduce")
        return out

    def close(self) -> None:
        for b in (*self.ws, *self.flags):
            b.close()


def maybe_create(group, device, max_rows: int, n_cols: int) -> FusedAllReduceGemm | None:
    """The workspace, or None (with the reason kept on the function) when the group cannot use it."""
    try:
        return FusedAllReduceGemm(group, device, max_rows, n_cols)
    except (RuntimeError, native.NativeKernelError) as e:
        maybe_create.last_reason = str(e)
        return None


maybe_create.last_reason = ""


class CrossEntropyExchange:
    """Cross-rank finish of vocab-parallel cross-entropy over peer memory: every rank contributes the
    (log-sum-exp, target logit) of its vocabulary shard per row and receives the global pair
    (csrc/comm.cu::ce_exchange_kernel). Replaces an all-gather and an all-reduce of per-row scalars.
    Two workspaces alternate and flags carry a growing epoch, as for the all-reduce GEMM.

    Counterpart: the in-kernel max / sum / target exchange of the reference's vocab-parallel fused
    linear-CE (dllm_parallel/core/csrc/fused_linear_ce/fused_linear_ce_cuda.cu:618-1268,
    dllm_parallel/core/parallel/cross_entropy.py:198-276)."""

    def __init__(self, group, device: torch.device, max_rows: int):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= 16:
            raise RuntimeError(f"cross-entropy exchange supports 2..16 ranks, got {self.world}")
        if not peer_access_available(group):
            raise RuntimeError("GPUs of this group cannot address one another (no peer access)")
        self.max_rows = int(max_rows)
        blocks = native.lib().tdllm_ce_exchange_blocks(self.max_rows)
        self.ws = [SymmetricBuffer(self.world * self.max_rows * 8, group, device) for _ in range(2)]
        self.flags = [SymmetricBuffer(self.world * blocks * 4, group, device) for _ in range(2)]
        for f in self.flags:
            f.as_tensor(torch.int32).zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self.epoch = [0, 0]
        self.flip = 0

    def finish(self, stats: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """stats [rows, n_tiles, 3] fp32 of this rank's shard -> (lse [rows], target logit [rows]), global."""
        rows, nt, _ = stats.shape
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed this workspace ({self.max_rows})")
        lse = torch.empty(rows, dtype=torch.float32, device=stats.device)
        tgt = torch.empty(rows, dtype=torch.float32, device=stats.device)
        b = self.flip
        self.flip ^= 1
        self.epoch[b] += 1
        rc = native.lib().tdllm_ce_exchange(ptr(stats), rows, nt, self.ws[b].ptr_array, self.flags[b].ptr_array,
                                            self.rank, self.world, self.epoch[b], self.max_rows, ptr(lse), ptr(tgt),
                                            stream())
        native.check(rc, "ce_exchange")
        return lse, tgt

    def close(self) -> None:
        for b in (*self.ws, *self.flags):
            b.close()
