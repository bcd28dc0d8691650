"""Attention for head widths other than 128 (256, 512, also 64: any multiple of 64) on sm_100a.

The one-kernel attention keeps S, P and O of a 128-wide head in the 512 tensor-memory columns of an SM; wider
heads do not fit, so they run as tensor-core products around a masked softmax kernel, over a chunk of query rows
at a time and only the 128-row key tiles the chunk can see under the mask:

    forward   S = Q·Kᵀ (fp32)  ->  P, lse = softmax(S)  ->  O = P·V
    backward  S again, dP = dO·Vᵀ  ->  P, dS  ->  dV += Pᵀ·dO, dK += dSᵀ·Q, dQ = dS·K

The G query heads that share a KV head are stacked along the rows of one product, so K and V tiles are gathered
once per KV head and chunk. The products are the tcgen05 GEMM of this library (`ops.gemm.gemm`), the softmax
kernels are `csrc/wide_attention.cu`; the API is the `(out, lse)` contract of the 128-wide kernels, so shard
results merge the same way. P is never kept: the backward pass recomputes it from the saved lse.

Role of dllm_parallel/core/attention/wide_head_attention.py:363-1843 (BDLM-masked wide-head attention with the
output / LSE contract), which on devices other than Hopper runs a compiled block-sparse kernel.
"""
from __future__ import annotations

import math

import torch

from ..kernels import native
from ._util import ptr, stream
from .attention import TILE, MaskLayout
from .gemm import gemm

native.register_signatures({
    "tdllm_wide_softmax": (native.c_int, [native.c_void_p] * 7 + [native.c_ll, native.c_int, native.c_int,
                                                                  native.c_ll, native.c_ll, native.c_float,
                                                                  native.c_void_p]),
    "tdllm_wide_softmax_bwd": (native.c_int, [native.c_void_p] * 10 + [native.c_ll, native.c_int, native.c_int,
                                                                       native.c_ll, native.c_ll, native.c_float,
                                                                       native.c_void_p]),
})

SCORE_BYTES = 1 << 30      # budget of the fp32 score matrix of one chunk


def wide_supported(head_dim: int) -> bool:
    return head_dim != 128 and head_dim % 64 == 0


def _chunks(layout: MaskLayout, group: int):
    """[(first query row, rows, key rows tensor)]: chunks of whole 128-row query tiles and the key rows (whole
    128-row tiles, ascending) that some row of the chunk can see."""
    key = ("wide_chunks", group)
    if key in layout._cache:
        return layout._cache[key]
    L = layout.tile_lists()
    nqt = L["nqt"]
    ptr_, idx = L["f_ptr"].cpu(), L["f_idx"].cpu()
    nk = layout.nk
    dev = layout.q_lo.device
    out, t0 = [], 0
    while t0 < nqt:
        tiles: set[int] = set()
        t1 = t0
        while t1 < nqt:
            new = tiles | set((idx[ptr_[t1]: ptr_[t1 + 1]] >> 1).tolist())
            rows = (t1 + 1 - t0) * TILE
            if t1 > t0 and rows * group * max(len(new), 1) * TILE * 4 > SCORE_BYTES:
                break
            tiles, t1 = new, t1 + 1
        kt = torch.tensor(sorted(tiles), dtype=torch.long)
        krows = (kt[:, None] * TILE + torch.arange(TILE)[None, :]).reshape(-1)
        valid = krows < nk
        out.append((t0 * TILE, (t1 - t0) * TILE, krows.clamp_max(max(nk - 1, 0)).to(dev), valid.to(dev)))
        t0 = t1
    layout._cache[key] = out
    return out


def _gather_q(t: torch.Tensor, r0: int, rows: int, h0: int, G: int) -> torch.Tensor:
    """[rows, G heads, D] slice of t (zero rows past the end) -> [G * rows, D], head-major."""
    n = t.shape[0]
    take = t[r0: min(r0 + rows, n), h0: h0 + G]
    if take.shape[0] < rows:
        take = torch.cat([take, take.new_zeros(rows - take.shape[0], G, t.shape[2])])
    return take.permute(1, 0, 2).reshape(G * rows, t.shape[2]).contiguous()


def _mask_rows(layout: MaskLayout, r0: int, rows: int):
    L = layout.tile_lists()      # padded to whole tiles: rows past nq see nothing
    return L["q_lo"][r0: r0 + rows], L["q_hi"][r0: r0 + rows], L["q_grp"][r0: r0 + rows]


def wide_attention_forward(q, k, v, layout: MaskLayout, scale: float):
    """q [nq, Hq, D], k / v [nk, Hkv, D] bf16 on the device -> (out [nq, Hq, D], lse [Hq, nq])."""
    from .attention import INT_MIN

    nq, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    lib = native.lib()
    out = torch.empty_like(q)
    lse = torch.empty(Hq, nq, dtype=torch.float32, device=q.device)
    for r0, rows, krows, valid in _chunks(layout, G):
        codes = torch.where(valid, layout.k_code.index_select(0, krows),
                            torch.full_like(krows, INT_MIN, dtype=torch.int32)).contiguous()
        lo, hi, grp = _mask_rows(layout, r0, rows)
        ns = int(krows.numel())
        live = min(rows, nq - r0)
        for h in range(Hkv):
            ks = k[:, h].index_select(0, krows)
            vs = v[:, h].index_select(0, krows)
            qc = _gather_q(q, r0, rows, h * G, G)
            s = gemm(qc, ks, out_dtype=torch.float32)                               # [G*rows, ns]
            p = torch.empty(G * rows, ns, dtype=torch.bfloat16, device=q.device)
            l = torch.empty(G * rows, dtype=torch.float32, device=q.device)
            native.check(lib.tdllm_wide_softmax(ptr(s), ptr(p), ptr(l), ptr(lo), ptr(hi), ptr(grp), ptr(codes),
                                                G * rows, rows, ns, s.stride(0), p.stride(0), float(scale),
                                                stream()), "wide_softmax")
            o = gemm(p, vs, b_mn_major=True)                                        # [G*rows, D]
            out[r0: r0 + live, h * G:(h + 1) * G] = o.view(G, rows, D)[:, :live].permute(1, 0, 2)
            lse[h * G:(h + 1) * G, r0: r0 + live] = l.view(G, rows)[:, :live]
    return out, lse


def wide_attention_backward(q, k, v, out, dout, lse, layout: MaskLayout, scale: float):
    """Gradients for the merged (out, lse) of the rows: exact per key shard without lse gradients."""
    from .attention import INT_MIN

    nq, Hq, D = q.shape
    nk, Hkv, _ = k.shape
    G = Hq // Hkv
    lib = native.lib()
    dev = q.device
    dq = torch.empty_like(q)
    dk = torch.zeros(nk, Hkv, D, dtype=torch.float32, device=dev)
    dv = torch.zeros(nk, Hkv, D, dtype=torch.float32, device=dev)
    delta = (out.float() * dout.float()).sum(-1).t().contiguous()                  # [Hq, nq]
    if lse.shape[1] != nq:
        lse = lse[:, :nq]
    for r0, rows, krows, valid in _chunks(layout, G):
        codes = torch.where(valid, layout.k_code.index_select(0, krows),
                            torch.full_like(krows, INT_MIN, dtype=torch.int32)).contiguous()
        lo, hi, grp = _mask_rows(layout, r0, rows)
        ns = int(krows.numel())
        live = min(rows, nq - r0)
        keep = valid[:, None].float()
        for h in range(Hkv):
            ks = k[:, h].index_select(0, krows)
            vs = v[:, h].index_select(0, krows)
            qc = _gather_q(q, r0, rows, h * G, G)
            doc = _gather_q(dout, r0, rows, h * G, G)
            l = torch.full((G, rows), float("-inf"), dtype=torch.float32, device=dev)
            l[:, :live] = lse[h * G:(h + 1) * G, r0: r0 + live]
            dl = torch.zeros(G, rows, dtype=torch.float32, device=dev)
            dl[:, :live] = delta[h * G:(h + 1) * G, r0: r0 + live]
            s = gemm(qc, ks, out_dtype=torch.float32)
            dp = gemm(doc, vs, out_dtype=torch.float32)
            p = torch.empty(G * rows, ns, dtype=torch.bfloat16, device=dev)
            ds = torch.empty_like(p)
            native.check(lib.tdllm_wide_softmax_bwd(ptr(s), ptr(dp), ptr(p), ptr(ds), ptr(l), ptr(dl), ptr(lo),
                                                    ptr(hi), ptr(grp), ptr(codes), G * rows, rows, ns, s.stride(0),
                                                    p.stride(0), float(scale), stream()), "wide_softmax_bwd")
            dvs = gemm(p, doc, a_mn_major=True, b_mn_major=True, out_dtype=torch.float32)     # [ns, D]
            dks = gemm(ds, qc, a_mn_major=True, b_mn_major=True, out_dtype=torch.float32)
            dk[:, h].index_add_(0, krows, dks * keep)
            dv[:, h].index_add_(0, krows, dvs * keep)
            dqc = gemm(ds, ks, b_mn_major=True)                                               # [G*rows, D]
            dq[r0: r0 + live, h * G:(h + 1) * G] = dqc.view(G, rows, D)[:, :live].permute(1, 0, 2)
    return dq, dk.to(q.dtype), dv.to(q.dtype)


class _WideAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, layout, scale):
        out, lse = wide_attention_forward(q, k, v, layout, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.layout, ctx.scale = layout, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = wide_attention_backward(q, k, v, out, dout.contiguous(), lse, ctx.layout, ctx.scale)
        return dq, dk, dv, None, None


def wide_block_attention(q, k, v, layout: MaskLayout, scale: float | None = None) -> torch.Tensor:
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _WideAttention.apply(q, k, v, layout, scale)
