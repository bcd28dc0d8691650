"""Which clean tokens and noisy blocks a rank owns, and the packed-row layout of a rank.

Clean ownership: `contiguous` gives each context-parallel rank one balanced shard;
`dual_chunk` (zigzag) cuts the clean sequence into 2·CP balanced chunks and gives rank r the
chunks r and 2·CP-1-r, which balances block-causal work. A rank's packed rows are
`[noisy rows of its owned blocks (ascending) ; its clean shards]`.

Follows dllm_parallel/core/attention/cp_backend.py:75-122 (balanced bounds, clean shards),
dllm_parallel/core/attention/layout.py:288-299 (runtime layout choice) and the packed layout of
dllm_parallel/core/models/backbones/nemotron/model.py:3385-3520.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops.attention import MaskLayout, block_diffusion_layout


def balanced_bounds(n: int, parts: int, i: int) -> tuple[int, int]:
    base, rem = divmod(n, parts)
    start = i * base + min(i, rem)
    return start, start + base + (1 if i < rem else 0)


@dataclass(frozen=True)
class CleanShard:
    start: int
    stop: int
    chunk_index: int

    @property
    def length(self) -> int:
        return self.stop - self.start


def runtime_clean_layout(policy_layout: str, block_parallel_size: int) -> str:
    """zigzag policy means dual-chunk ownership whenever blocks are also distributed."""
    return "dual_chunk" if (policy_layout == "zigzag" and block_parallel_size > 1) else "contiguous"


def clean_shards_for_rank(seq_len: int, cp_size: int, cp_rank: int, layout: str = "dual_chunk",
                          align: int = 1) -> list[CleanShard]:
    """`align` rounds chunk boundaries to multiples (e.g. the diffusion block size)."""
    units = seq_len // align
    if seq_len % align:
        raise ValueError("seq_len must be a multiple of the alignment")
    if cp_size == 1:
        return [CleanShard(0, seq_len, 0)]
    if layout == "contiguous":
        a, b = balanced_bounds(units, cp_size, cp_rank)
        return [CleanShard(a * align, b * align, cp_rank)]
    if layout != "dual_chunk":
        raise ValueError(f"unknown clean layout {layout!r}")
    out = []
    for c in (cp_rank, 2 * cp_size - 1 - cp_rank):
        a, b = balanced_bounds(units, 2 * cp_size, c)
        if b > a:
            out.append(CleanShard(a * align, b * align, c))
    return out


def clean_positions_for_rank(seq_len, cp_size, cp_rank, layout="dual_chunk", align=1, device="cpu"):
    parts = [torch.arange(s.start, s.stop, device=device)
             for s in clean_shards_for_rank(seq_len, cp_size, cp_rank, layout, align)]
    return torch.cat(parts) if parts else torch.zeros(0, dtype=torch.long, device=device)


def pure_context_offsets(block_size: int, cp_size: int, cp_rank: int) -> list[int]:
    """Token offsets inside every diffusion block that context-parallel rank `cp_rank` computes when context
    parallelism runs without block parallelism: block_size / cp_size offsets per rank, taken from both ends of
    the block (rank r: the r-th slice from the front and the r-th from the back) when that share is even, one
    contiguous slice otherwise. Every offset belongs to exactly one rank.
    Semantics of dllm_parallel/core/attention/layout.py:54-132."""
    if block_size % cp_size:
        raise ValueError(f"block_size {block_size} must divide by context_parallel_size {cp_size}")
    per = block_size // cp_size
    if per % 2:
        return list(range(cp_rank * per, (cp_rank + 1) * per))
    h = per // 2
    return list(range(cp_rank * h, (cp_rank + 1) * h)) + list(range(block_size - (cp_rank + 1) * h,
                                                                    block_size - cp_rank * h))


@dataclass
class PackedLayout:
    """Row bookkeeping of one rank for one micro-batch shape (static across steps)."""

    noisy_pos: torch.Tensor      # [n_noisy] position of each noisy row inside its sequence
    noisy_seq: torch.Tensor      # [n_noisy] sequence index within the micro-batch
    noisy_view: torch.Tensor     # [n_noisy] noisy view (Fast-dLLM v2 has two)
    noisy_group: torch.Tensor    # [n_noisy] unique id of the noisy block
    clean_pos: torch.Tensor      # [n_clean]
    clean_seq: torch.Tensor      # [n_clean]
    positions: torch.Tensor      # [rows] RoPE positions of [noisy ; clean]
    mask: MaskLayout             # attention mask over the rank's own rows (keys = own rows)
    block_size: int
    clean_causal: bool = False   # clean rows attend causally (token by token) instead of block-causally
    noisy_offsets: tuple | None = None   # offsets inside a block this rank computes (pure context parallelism)
    window: int | None = None            # window of the sliding-window layers
    window_mask: MaskLayout | None = None   # the mask of those layers over the rank's own rows
    noisy_offset: torch.Tensor | None = None   # response-suffix packing: offset of each noisy row in the decoder tensors

    @property
    def n_noisy(self) -> int:
        return int(self.noisy_pos.shape[0])

    @property
    def n_clean(self) -> int:
        return int(self.clean_pos.shape[0])

    @property
    def rows(self) -> int:
        return self.n_noisy + self.n_clean


def noisy_rows(*, seq_len: int, block_size: int, batch: int, views: int = 1, owned_blocks=None,
               noisy_offsets=None, device="cpu"):
    """(position, sequence, view, block id) of the noisy rows of a rank, in packed order: sequence-major, then
    view, then block, then offset. The block id is the same on every rank that holds rows of the block."""
    nblocks = seq_len // block_size
    owned = list(range(nblocks)) if owned_blocks is None else sorted(owned_blocks)
    blk = torch.tensor(owned, dtype=torch.long, device=device)
    in_blk = (torch.arange(block_size, device=device) if noisy_offsets is None
              else torch.tensor(sorted(noisy_offsets), dtype=torch.long, device=device))
    pos1 = (blk[:, None] * block_size + in_blk[None, :]).reshape(-1)
    n1 = pos1.numel()
    seq_ids = torch.arange(batch, device=device)
    view_ids = torch.arange(views, device=device)
    noisy_pos = pos1.repeat(batch * views)
    noisy_seq = seq_ids.repeat_interleave(views * n1)
    noisy_view = view_ids.repeat_interleave(n1).repeat(batch)
    noisy_group = (noisy_seq * views + noisy_view) * nblocks + noisy_pos // block_size
    return noisy_pos, noisy_seq, noisy_view, noisy_group


def build_response_layout(*, seq_len: int, block_size: int, batch: int, response_start: int, valid_length: int,
                          decoder_length: int, window: int | None = None, device="cpu",
                          clean_causal: bool = False, owned_blocks=None) -> PackedLayout:
    """Rows of a batch whose noisy (decoder) rows cover only the response [response_start, valid_length): for every
    sequence `decoder_length` rows (whole blocks counted from the response start; rows past the response are
    padding at the last valid position), then all clean positions. A decoder block sees the clean tokens before
    its own first position. `owned_blocks`: the decoder blocks (counted from the response start) whose rows this
    rank holds under block parallelism; all of them by default.
    Layout of dllm_parallel/core/objectives/diffusiongemma.py:226-250."""
    off1 = torch.arange(decoder_length, device=device)
    nblk = decoder_length // block_size
    if owned_blocks is not None:
        keep = torch.zeros(nblk, dtype=torch.bool, device=device)
        keep[torch.as_tensor(sorted(owned_blocks), device=device)] = True
        off1 = off1[keep[off1 // block_size]]
    seq_ids = torch.arange(batch, device=device)
    noisy_off = off1.repeat(batch)
    noisy_seq = seq_ids.repeat_interleave(off1.numel())
    noisy_pos = (noisy_off + response_start).clamp(max=valid_length - 1)
    noisy_view = torch.zeros_like(noisy_seq)
    blk = noisy_off // block_size
    noisy_group = noisy_seq * nblk + blk
    noisy_stop = (response_start + blk * block_size).clamp(max=valid_length)
    cpos1 = torch.arange(seq_len, device=device)
    clean_pos = cpos1.repeat(batch)
    clean_seq = seq_ids.repeat_interleave(seq_len)
    kw = dict(noisy_seq=noisy_seq, clean_seq=clean_seq, clean_causal=clean_causal, noisy_stop=noisy_stop)
    mask = block_diffusion_layout(noisy_pos, noisy_group, clean_pos, block_size, **kw)
    wmask = block_diffusion_layout(noisy_pos, noisy_group, clean_pos, block_size, window=window, **kw) if window else None
    return PackedLayout(noisy_pos, noisy_seq, noisy_view, noisy_group, clean_pos, clean_seq,
                        torch.cat([noisy_pos, clean_pos]), mask, block_size, clean_causal, None, window or None, wmask,
                        noisy_off)


def build_packed_layout(*, seq_len: int, block_size: int, batch: int, views: int = 1,
                        owned_blocks=None, clean_pos: torch.Tensor | None = None,
                        window: int | None = None, device="cpu", clean_causal: bool = False,
                        noisy_offsets=None) -> PackedLayout:
    """Rows of one rank: for every sequence and view the noisy rows of `owned_blocks` (all offsets of a block,
    or only `noisy_offsets`: pure context parallelism splits the tokens inside every block), then for
    every sequence the clean rows `clean_pos` (default: all positions). `window`: also build the mask of the
    sliding-window layers (`window_mask`); `mask` always is the full-prefix one."""
    noisy_pos, noisy_seq, noisy_view, noisy_group = noisy_rows(
        seq_len=seq_len, block_size=block_size, batch=batch, views=views, owned_blocks=owned_blocks,
        noisy_offsets=noisy_offsets, device=device)
    seq_ids = torch.arange(batch, device=device)
    cpos1 = torch.arange(seq_len, device=device) if clean_pos is None else clean_pos.to(device)
    clean_pos_all = cpos1.repeat(batch)
    clean_seq = seq_ids.repeat_interleave(cpos1.numel())
    mask = block_diffusion_layout(noisy_pos, noisy_group, clean_pos_all, block_size, noisy_seq=noisy_seq,
                                  clean_seq=clean_seq, clean_causal=clean_causal)
    wmask = None
    if window:
        wmask = block_diffusion_layout(noisy_pos, noisy_group, clean_pos_all, block_size, noisy_seq=noisy_seq,
                                       clean_seq=clean_seq, window=window, clean_causal=clean_causal)
    return PackedLayout(noisy_pos, noisy_seq, noisy_view, noisy_group, clean_pos_all, clean_seq,
                        torch.cat([noisy_pos, clean_pos_all]), mask, block_size, clean_causal,
                        None if noisy_offsets is None else tuple(sorted(noisy_offsets)), window or None, wmask)
