"""Grouped (per-expert) linear layers as single launches of the tcgen05 GEMM.

Rows are sorted by expert and copied into a padded layout in which every expert's segment starts on a
256-row boundary (one CTA pair never spans two experts). Three products then run as one kernel each:

    forward          y[r]  = x[r] · W[e(r)]ᵀ          B slice chosen per row tile
    input gradient   dx[r] = dy[r] · W[e(r)]           B slice chosen per row tile (MN-major B)
    weight gradient  dW[e] = dy_eᵀ · x_e               per-expert range of K blocks, outputs stacked

All tables are built on the device from the per-expert counts; the padded capacity is the static bound
rows + 256·experts, so nothing here waits for the GPU. Padding rows are zero and produce zeros.

Counterpart of the reference's grouped expert GEMMs (`F.grouped_mm` in
dllm_parallel/core/models/backbones/diffusion_gemma/expert_parallel.py:283-321).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import native
from ._util import grad_sink, ptr, stream, use_native

native.register_signatures({
    "tdllm_gemm_grouped_bf16": (native.c_int, [native.c_void_p] * 3 + [native.c_int] * 3 + [native.c_ll] * 3
                                + [native.c_int] * 4 + [native.c_void_p, native.c_ll, native.c_ll, native.c_ll,
                                                        native.c_ll, native.c_void_p, native.c_void_p, native.c_int,
                                                        native.c_void_p]),
})

PAD = 256
EPI_STORE, EPI_SWIGLU = 0, 1


@dataclass
class GroupedRows:
    """Padded row layout of one routed batch (all tensors on the device)."""
    num_groups: int
    capacity: int               # rows of the padded buffers (multiple of 256)
    dest: torch.Tensor          # [rows] position of every sorted row in the padded layout
    mt_group: torch.Tensor      # [capacity / 128] expert of every 128-row tile
    row_begin: torch.Tensor     # [E] first padded row of every expert
    row_blocks_end: torch.Tensor  # [E] end of the expert's rows in 64-row blocks (rounded up)
    valid_tiles: torch.Tensor | None = None   # [capacity / 128] bool: tiles inside some expert's padded segment
    # (None = all). Tiles outside run no tensor-core work: a slab of static capacity is mostly such tiles.

    def k_range(self, k_blocks: int):
        """Per-tile K-block ranges for the forward / input-gradient products (None = every tile runs all of K)."""
        if self.valid_tiles is None:
            return None, None
        kend = (self.valid_tiles.to(torch.int32) * int(k_blocks)).contiguous()
        return torch.zeros_like(kend), kend


def build_grouped_rows(counts: torch.Tensor, sorted_rows: int) -> GroupedRows:
    """counts: [E] rows per expert (device, any integer dtype); rows are already sorted by expert."""
    E = counts.numel()
    dev = counts.device
    counts = counts.long()
    padded = (counts + PAD - 1) // PAD * PAD
    ends = padded.cumsum(0)
    begin = ends - padded
    capacity = (sorted_rows + E * PAD + PAD - 1) // PAD * PAD
    off = counts.cumsum(0) - counts
    e_sorted = torch.repeat_interleave(torch.arange(E, device=dev), counts, output_size=sorted_rows)
    dest = begin[e_sorted] + torch.arange(sorted_rows, device=dev) - off[e_sorted]
    tile_start = torch.arange(capacity // 128, device=dev) * 128
    mt_group = torch.searchsorted(ends, tile_start, right=True).clamp_(max=E - 1).to(torch.int32)
    blocks_end = (begin + (counts + 63) // 64 * 64) // 64
    return GroupedRows(E, capacity, dest, mt_group.contiguous(), begin, blocks_end)


def grouped_supported(x: torch.Tensor, w_all: torch.Tensor) -> bool:
    """The grouped kernels need N and K on tile boundaries (experts must not share a B tile / K block)."""
    E, N, K = w_all.shape
    return (use_native(x, w_all) and N % 256 == 0 and K % 64 == 0 and w_all.is_contiguous()
            and x.dtype == torch.bfloat16)


def _launch(a, b2d, d, M, N, K, a_mn, b_mn, accumulate, mode, mt_group, b_group_rows, b_rows_total,
            a_group_rows, a_m_total, kbegin, kend):
    rc = native.lib().tdllm_gemm_grouped_bf16(
        ptr(a), ptr(b2d), ptr(d), M, N, K, a.stride(0), b2d.stride(0), d.stride(0), int(a_mn), int(b_mn),
        int(accumulate), mode, ptr(mt_group) if mt_group is not None else None, b_group_rows, b_rows_total,
        a_group_rows, a_m_total, ptr(kbegin) if kbegin is not None else None,
        ptr(kend) if kend is not None else None, 0, stream())
    native.check(rc, "gemm_grouped")


class _GroupedLinear(torch.autograd.Function):
    """y = x_pad · W[e]ᵀ per row tile; dW lands in the stacked gradient slice of the flat buffer."""

    @staticmethod
    def forward(ctx, x_pad, w_all, g: GroupedRows):
        E, N, K = w_all.shape
        y = torch.empty(g.capacity, N, dtype=x_pad.dtype, device=x_pad.device)
        kb, ke = g.k_range(K // 64)
        _launch(x_pad, w_all.view(E * N, K), y, g.capacity, N, K, 0, 0, 0, EPI_STORE, g.mt_group, N, E * N,
                0, 0, kb, ke)
        ctx.save_for_backward(x_pad, w_all)
        ctx.g, ctx.wref = g, w_all
        return y

    @staticmethod
    def backward(ctx, dy):
        x_pad, w_all = ctx.saved_tensors
        g: GroupedRows = ctx.g
        E, N, K = w_all.shape
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x_pad)
            kb, ke = g.k_range(N // 64)
            _launch(dy, w_all.view(E * N, K), dx, g.capacity, K, N, 0, 1, 0, EPI_STORE, g.mt_group, N, E * N,
                    0, 0, kb, ke)
        # dW[e] = dy_eᵀ x_e: output rows e*N.., A = dy read MN-major with its M coordinate taken modulo N
        tiles = torch.arange(E * N // 128, device=dy.device)
        grp = (tiles * 128 // N).to(torch.int32)
        kbeg = (g.row_begin // 64)[grp.long()].to(torch.int32).contiguous()
        kend = g.row_blocks_end[grp.long()].to(torch.int32).contiguous()
        sink, _ = grad_sink(ctx.wref)
        dw = None
        if sink is not None:
            written = ctx.wref.expert_written
            target, acc = sink.view(E * N, K), len(written) > 0
            written.update(range(E))
        else:
            dw = torch.empty_like(w_all)
            target, acc = dw.view(E * N, K), False
        _launch(dy, x_pad, target, E * N, K, g.capacity, 1, 1, acc, EPI_STORE, grp.contiguous(), 0, 0, N, N,
                kbeg, kend)
        return dx, dw, None


def grouped_linear(x_pad: torch.Tensor, w_all: torch.Tensor, g: GroupedRows) -> torch.Tensor:
    return _GroupedLinear.apply(x_pad, w_all, g)
