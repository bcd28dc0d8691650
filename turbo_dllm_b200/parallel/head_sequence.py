"""Head <-> sequence all-to-all for layers that need whole sequences (linear attention).

Before: every rank holds its own rows (a shard of the sequence) with the features of all heads.
`sequence_to_head_parallel` sends, to every rank r of the group, this rank's rows restricted to the
features of r's heads; afterwards every rank holds the rows of ALL ranks (in rank order) for its own
heads. `head_to_sequence_parallel` is the way back: rank r returns, to every rank s, the rows that
came from s; s concatenates what it gets along the feature axis in rank order. Each direction is one
`all_to_all_single` with per-rank row counts, and each is the other's backward pass.

Reference counterpart: dllm_parallel/core/models/backbones/qwen3_8/context_parallel.py:16-57
(`sequence_to_head_parallel_many`), :60-86 (`head_to_sequence_parallel`), :89-143.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..profiling import collectives as coll


def _exchange(x: torch.Tensor, send_rows: list[int], recv_rows: list[int], group) -> torch.Tensor:
    out = x.new_empty(sum(recv_rows), x.shape[1])
    coll.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_rows, input_split_sizes=send_rows,
                           domain="context_parallel", group=group)
    return out


class _RowsToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, stacked, row_counts, index, group):
        """stacked: [P * rows_mine, F], block r = this rank's rows with rank r's features."""
        ctx.row_counts, ctx.index, ctx.group = row_counts, index, group
        mine = row_counts[index]
        return _exchange(stacked, [mine] * len(row_counts), list(row_counts), group)

    @staticmethod
    def backward(ctx, g):
        mine = ctx.row_counts[ctx.index]
        return _exchange(g, list(ctx.row_counts), [mine] * len(ctx.row_counts), ctx.group), None, None, None


class _HeadsToRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gathered, row_counts, index, group):
        """gathered: [sum(row_counts), F] rows of all ranks for this rank's heads."""
        ctx.row_counts, ctx.index, ctx.group = row_counts, index, group
        mine = row_counts[index]
        return _exchange(gathered, list(row_counts), [mine] * len(row_counts), group)

    @staticmethod
    def backward(ctx, g):
        mine = ctx.row_counts[ctx.index]
        return _exchange(g, [mine] * len(ctx.row_counts), list(ctx.row_counts), ctx.group), None, None, None


def sequence_to_head_parallel(parts: list[torch.Tensor], row_counts: list[int], group) -> torch.Tensor:
    """parts[r]: this rank's rows [rows_mine, F] restricted to rank r's heads (same F for every r).
    Returns [sum(row_counts), F]: the rows of rank 0, then rank 1, ... for this rank's heads."""
    index = dist.get_rank(group)
    if len(parts) != len(row_counts) or any(p.shape != parts[0].shape for p in parts):
        raise ValueError("one equally shaped part per rank of the group is required")
    if parts[0].shape[0] != row_counts[index]:
        raise ValueError(f"this rank holds {parts[0].shape[0]} rows, the plan says {row_counts[index]}")
    return _RowsToHeads.apply(torch.cat(parts, dim=0), tuple(row_counts), index, group)


def head_to_sequence_parallel(gathered: torch.Tensor, row_counts: list[int], index: int, group) -> torch.Tensor:
    """gathered: [sum(row_counts), F] for this rank's heads -> this rank's rows with all heads
    [rows_mine, P * F] (features in rank order)."""
    if gathered.shape[0] != sum(row_counts):
        raise ValueError(f"expected {sum(row_counts)} gathered rows, got {gathered.shape[0]}")
    back = _HeadsToRows.apply(gathered, tuple(row_counts), index, group)
    mine, parts = row_counts[index], len(row_counts)
    return back.view(parts, mine, gathered.shape[1]).permute(1, 0, 2).reshape(mine, parts * gathered.shape[1])
