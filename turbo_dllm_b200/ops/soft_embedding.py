"""Soft embeddings `softmax(h Wᵀ) W` without ever holding a [rows, vocab] tensor.

Used for self-conditioning: a detached first denoising pass predicts a distribution per noisy row, and
the expected embedding under that distribution is fed to the second pass. Rows are processed in chunks;
inside a chunk the vocabulary is walked in chunks with a running maximum, denominator and numerator
(online softmax), so the live memory is rows_chunk × vocab_chunk. With a vocabulary-sharded W every
rank reduces its shard the same way and the three running quantities are combined over the
tensor-parallel group. Forward only (the result is detached).

On bf16 CUDA tensors the two products of every chunk run on the tcgen05 GEMM; elsewhere in fp32.

Counterpart: dllm_parallel/core/kernels/streaming_soft_embedding.py:60-218.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..profiling import collectives as coll

from ._util import use_native
from .gemm import gemm


def _chunk_logits(rows: torch.Tensor, w_chunk: torch.Tensor, softcap: float | None) -> torch.Tensor:
    if use_native(rows, w_chunk):
        z = gemm(rows, w_chunk, out_dtype=torch.float32)
    else:
        z = rows.float() @ w_chunk.float().t()
    if softcap:
        z = softcap * torch.tanh(z / softcap)
    return z


def _online_shard(rows: torch.Tensor, weight: torch.Tensor, vocab_chunk: int, softcap: float | None):
    """(max [r], denominator [r], numerator [r, H]) of softmax(rows Wᵀ) W over this weight (shard)."""
    r, H = rows.shape
    dev = rows.device
    m = torch.full((r,), float("-inf"), dtype=torch.float32, device=dev)
    den = torch.zeros(r, dtype=torch.float32, device=dev)
    num = torch.zeros(r, H, dtype=torch.float32, device=dev)
    for v0 in range(0, weight.shape[0], vocab_chunk):
        wc = weight[v0:v0 + vocab_chunk]
        z = _chunk_logits(rows, wc, softcap)
        m_new = torch.maximum(m, z.max(dim=1).values)
        alpha = torch.exp(m - m_new)
        p = torch.exp(z - m_new[:, None])
        den = den * alpha + p.sum(1)
        if use_native(rows, wc):
            contrib = gemm(p.to(rows.dtype), wc, b_mn_major=True, out_dtype=torch.float32)
        else:
            contrib = p @ wc.float()
        num = num * alpha[:, None] + contrib
        m = m_new
    return m, den, num


@torch.no_grad()
def streaming_soft_embedding(hidden: torch.Tensor, weight: torch.Tensor, *, row_chunk_size: int = 256,
                             vocab_chunk_size: int = 32768, logit_softcap: float | None = None,
                             embedding_scale: float = 1.0, tp_group=None) -> torch.Tensor:
    """hidden [..., H], weight [V or V/tp, H] -> softmax(hidden Wᵀ) W · embedding_scale, same shape and
    dtype as `hidden`, detached. `tp_group`: the group over which `weight` is sharded by rows."""
    if row_chunk_size <= 0 or vocab_chunk_size <= 0:
        raise ValueError("chunk sizes must be positive")
    H = hidden.shape[-1]
    if weight.shape[1] != H:
        raise ValueError(f"weight has {weight.shape[1]} columns, hidden has {H}")
    flat = hidden.reshape(-1, H)
    out = torch.empty_like(flat)
    sharded = tp_group is not None and dist.is_initialized() and dist.get_world_size(tp_group) > 1
    for r0 in range(0, flat.shape[0], row_chunk_size):
        rows = flat[r0:r0 + row_chunk_size].contiguous()
        m, den, num = _online_shard(rows, weight, vocab_chunk_size, logit_softcap)
        if sharded:
            m_all = m.clone()
            coll.all_reduce(m_all, "tensor", op=dist.ReduceOp.MAX, group=tp_group)
            scale = torch.exp(m - m_all)
            den, num = den * scale, num * scale[:, None]
            coll.all_reduce(den, "tensor", group=tp_group)
            coll.all_reduce(num, "tensor", group=tp_group)
        out[r0:r0 + row_chunk_size] = (num / den[:, None] * embedding_scale).to(out.dtype)
    return out.view_as(hidden).detach()
