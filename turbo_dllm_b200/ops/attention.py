"""Block-diffusion attention with a declarative mask.

Mask model (same predicate as the reference's `_explicit_bdlm_flex_mask`,
dllm_parallel/core/attention/context_parallel_attention.py:119-144, and its mask specs,
dllm_parallel/core/attention/masks.py:15-243):

* every query row has `(lo, hi, grp)`; every key has one `code`;
* `code >= 0` is a clean key at coordinate `code`, visible iff `lo <= code < hi`;
* `code < 0` is a noisy key of block `-(code+1)`, visible iff `code == grp`
  (`grp = 0` for clean queries, which therefore never see noisy keys).

Coordinates are `sequence_index * stride + position`, so several sequences, sliding windows
(`lo > 0`) and context-parallel shards (any subset of keys) use the same kernel.

`attention_reference` is the dense-mask fp32 oracle. On CUDA bf16 tensors the tcgen05 kernels
run; they consume per-query-tile lists of visible key tiles built once per layout
(`MaskLayout.tile_lists`).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch

from ..kernels import native
from ._util import ptr, scratch, stream, use_native

TILE = 128
INT_MIN = -(2 ** 31)

native.register_signatures({
    "tdllm_attn_fwd": (native.c_int, [native.c_void_p] * 5 + [native.c_int] * 4 + [native.c_ll] * 4
                       + [native.c_void_p] * 7 + [native.c_int, native.c_float, native.c_void_p]),
})


@dataclass
class MaskLayout:
    """Row metadata of one attention call (static for a given sequence layout)."""

    q_lo: torch.Tensor
    q_hi: torch.Tensor
    q_grp: torch.Tensor
    k_code: torch.Tensor
    _cache: dict = field(default_factory=dict, repr=False)

    @property
    def nq(self) -> int:
        return int(self.q_lo.shape[0])

    @property
    def nk(self) -> int:
        return int(self.k_code.shape[0])

    def to(self, device) -> "MaskLayout":
        return MaskLayout(self.q_lo.to(device), self.q_hi.to(device), self.q_grp.to(device),
                          self.k_code.to(device))

    def dense_mask(self) -> torch.Tensor:
        """[nq, nk] bool, True = visible."""
        code = self.k_code[None, :].long()
        lo, hi, grp = self.q_lo[:, None].long(), self.q_hi[:, None].long(), self.q_grp[:, None].long()
        return torch.where(code >= 0, (code >= lo) & (code < hi), code == grp)

    def allowed_pairs(self) -> int:
        return int(self.dense_mask().sum())

    # -- tile lists for the sm_100a kernels ---------------------------------
    def tile_lists(self) -> dict:
        if "lists" in self._cache:
            return self._cache["lists"]
        dev = self.q_lo.device
        nq, nk = self.nq, self.nk
        nqt, nkt = (nq + TILE - 1) // TILE, (nk + TILE - 1) // TILE
        nq_pad, nk_pad = nqt * TILE, nkt * TILE
        i32 = torch.int32

        def pad(t, n, value):
            out = torch.full((n,), value, dtype=i32, device=dev)
            out[: t.shape[0]] = t.to(i32)
            return out

        q_lo, q_hi, q_grp = pad(self.q_lo, nq_pad, 0), pad(self.q_hi, nq_pad, 0), pad(self.q_grp, nq_pad, 0)
        k_code = pad(self.k_code, nk_pad, INT_MIN)
        real_q = (torch.arange(nq_pad, device=dev) < nq).view(nqt, TILE)
        BIG = 2 ** 31 - 1
        lo = q_lo.view(nqt, TILE).long()
        hi = q_hi.view(nqt, TILE).long()
        grp = q_grp.view(nqt, TILE).long()
        lo_min = torch.where(real_q, lo, BIG).amin(1)
        lo_max = torch.where(real_q, lo, -1).amax(1)
        hi_min = torch.where(real_q, hi, BIG).amin(1)
        hi_max = torch.where(real_q, hi, -1).amax(1)
        q_noisy = real_q & (grp < 0)
        qg_min = torch.where(q_noisy, grp, 0).amin(1)
        qg_max = torch.where(q_noisy, grp, INT_MIN).amax(1)
        code = k_code.view(nkt, TILE).long()
        is_clean = code >= 0
        is_pad = code == INT_MIN
        is_noisy = (code < 0) & ~is_pad
        c_min = torch.where(is_clean, code, BIG).amin(1)
        c_max = torch.where(is_clean, code, -1).amax(1)
        n_min = torch.where(is_noisy, code, 0).amin(1)
        n_max = torch.where(is_noisy, code, INT_MIN).amax(1)
        all_clean = is_clean.all(1)
        vis_clean = (c_min[None, :] < hi_max[:, None]) & (c_max[None, :] >= lo_min[:, None])
        vis_noisy = (n_min[None, :] <= qg_max[:, None]) & (n_max[None, :] >= qg_min[:, None])
        visible = vis_clean | vis_noisy
        full = all_clean[None, :] & (c_max[None, :] < hi_min[:, None]) & (c_min[None, :] >= lo_max[:, None])

        def csr(vis, fl):
            idx = vis.nonzero()
            counts = vis.sum(1)
            ptr_ = torch.zeros(vis.shape[0] + 1, dtype=i32, device=dev)
            ptr_[1:] = counts.cumsum(0).to(i32)
            ent = (idx[:, 1] * 2 + (~fl[idx[:, 0], idx[:, 1]]).long()).to(i32)
            if ent.numel() == 0:
                ent = torch.zeros(1, dtype=i32, device=dev)
            order = torch.argsort(counts, descending=True, stable=True).to(i32)
            return ptr_.contiguous(), ent.contiguous(), order.contiguous()

        f_ptr, f_idx, f_order = csr(visible, full)
        b_ptr, b_idx, b_order = csr(visible.t().contiguous(), full.t().contiguous())
        lists = dict(nqt=nqt, nkt=nkt, nq_pad=nq_pad, nk_pad=nk_pad, q_lo=q_lo, q_hi=q_hi, q_grp=q_grp,
                     k_code=k_code, f_ptr=f_ptr, f_idx=f_idx, f_order=f_order, b_ptr=b_ptr, b_idx=b_idx,
                     b_order=b_order, visited_tiles=int(visible.sum()))
        self._cache["lists"] = lists
        self._cache["visible"] = (visible, full)
        return lists

    def backward_work(self, chunk_tiles: int) -> dict:
        """Work items of the one-pass backward: for chunk c of `chunk_tiles` consecutive query tiles and
        key tile kt, item c·nkt + kt lists the chunk's query tiles that see the key tile (entry = q_tile·2 +
        needs_mask). `w_order` holds the non-empty items chunk by chunk, heaviest first inside a chunk, so
        that every key tile adds to one chunk's dQ rows while those rows are still in L2."""
        key = ("work", int(chunk_tiles))
        if key in self._cache:
            return self._cache[key]
        L = self.tile_lists()
        visible, full = self._cache["visible"]
        dev = visible.device
        nqt, nkt = L["nqt"], L["nkt"]
        S = max(1, min(int(chunk_tiles), nqt)) if chunk_tiles > 0 else nqt
        nch = (nqt + S - 1) // S
        i32 = torch.int32
        vis = torch.zeros(nch * S, nkt, dtype=torch.bool, device=dev)
        vis[:nqt] = visible
        vis = vis.view(nch, S, nkt).permute(0, 2, 1).contiguous()          # [chunk, kt, s]
        idx = vis.nonzero()                                                 # sorted by (chunk, kt, s)
        qt = idx[:, 0] * S + idx[:, 2]
        ent = (qt * 2 + (~full[qt, idx[:, 1]]).long()).to(i32)
        counts = vis.sum(2).reshape(-1)                                     # [chunk * nkt]
        w_ptr = torch.zeros(nch * nkt + 1, dtype=i32, device=dev)
        w_ptr[1:] = counts.cumsum(0).to(i32)
        items = counts.nonzero().squeeze(1)
        chunk_of = items // nkt
        sort_key = chunk_of * (S + 1) + (S - counts[items])                 # chunk ascending, count descending
        w_order = items[torch.argsort(sort_key, stable=True)].to(i32)
        if ent.numel() == 0:
            ent = torch.zeros(1, dtype=i32, device=dev)
        if w_order.numel() == 0:
            w_order = torch.zeros(1, dtype=i32, device=dev)
        out = dict(w_ptr=w_ptr.contiguous(), w_idx=ent.contiguous(), w_order=w_order.contiguous(),
                   n_work=int(items.numel()), chunk_tiles=S)
        self._cache[key] = out
        return out


def attention_reference(q, k, v, layout: MaskLayout, scale: float | None = None):
    """Dense-mask attention in fp32. q [nq,Hq,D], k/v [nk,Hkv,D] -> (out [nq,Hq,D], lse [Hq,nq]).
    Rows without a visible key give out = 0 and lse = -inf."""
    nq, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hkv
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, dim=0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    mask = layout.dense_mask().to(s.device)
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(mask[None], p, torch.zeros_like(p))
    out = torch.matmul(p, vf).permute(1, 0, 2)
    return out.to(q.dtype), lse


def _rows_view(t: torch.Tensor):
    """[n, H, D] tensor with unit inner stride and head stride D -> (row stride in elements)."""
    n, H, D = t.shape
    if t.stride(2) != 1 or (H > 1 and t.stride(1) != D):
        raise ValueError("attention operands must be [rows, heads, head_dim] views with packed heads")
    return t.stride(0)


def attention_forward_native(q, k, v, layout: MaskLayout, scale: float):
    nq, Hq, D = q.shape
    nk, Hkv, _ = k.shape
    if D != 128:
        raise native.NativeKernelError("sm_100a attention kernels are built for head_dim 128")
    L = layout.tile_lists()
    out = torch.empty(nq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, L["nq_pad"], dtype=torch.float32, device=q.device)
    rc = native.lib().tdllm_attn_fwd(
        ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), nq, nk, Hq, Hkv, _rows_view(q), _rows_view(k),
        _rows_view(v), out.stride(0), ptr(L["q_lo"]), ptr(L["q_hi"]), ptr(L["q_grp"]), ptr(L["k_code"]),
        ptr(L["f_ptr"]), ptr(L["f_idx"]), ptr(L["f_order"]), L["nqt"], float(scale), stream())
    native.check(rc, "attn_fwd")
    return out, lse


SEQ_STRIDE = 1 << 24      # key/query codes are sequence * SEQ_STRIDE + position


def block_diffusion_layout(noisy_pos: torch.Tensor, noisy_group: torch.Tensor, clean_pos: torch.Tensor,
                           block_size: int, *, noisy_seq: torch.Tensor | None = None,
                           clean_seq: torch.Tensor | None = None, seq_stride: int = SEQ_STRIDE,
                           window: int | None = None, key_clean_pos: torch.Tensor | None = None,
                           key_clean_seq: torch.Tensor | None = None, clean_causal: bool = False,
                           noisy_stop: torch.Tensor | None = None) -> MaskLayout:
    """Layout for packed rows `[noisy ; clean]` attending to keys `[noisy ; clean keys]`.

    noisy_pos/noisy_group: position and unique noisy-block id of each noisy row (the id must be
    distinct across sequences and views); clean_pos: position of each clean query row.
    `key_clean_*` default to the clean query rows (self-attention); a context-parallel rank passes
    the gathered or peer-owned clean key positions instead. With `clean_causal` a clean row sees the clean
    tokens up to and including itself instead of its whole block (the clean stream then is an ordinary
    causal model whose hidden states may carry a next-token loss); noisy rows are unaffected. `window` limits clean visibility to
    the last `window` positions before the row's clean stop (sliding-window layers).
    Semantics: dllm_parallel/core/models/backbones/nemotron/model.py:3486-3520 and
    dllm_parallel/core/attention/context_parallel_attention.py:119-144.
    """
    dev = noisy_pos.device
    i64 = torch.int64
    noisy_pos, clean_pos = noisy_pos.to(i64), clean_pos.to(i64)
    ns = torch.zeros_like(noisy_pos) if noisy_seq is None else noisy_seq.to(i64)
    cs = torch.zeros_like(clean_pos) if clean_seq is None else clean_seq.to(i64)
    kpos = clean_pos if key_clean_pos is None else key_clean_pos.to(i64)
    ks = (cs if key_clean_pos is None else
          (torch.zeros_like(kpos) if key_clean_seq is None else key_clean_seq.to(i64)))
    # a noisy row sees the clean tokens before its block: blocks normally start at multiples of the block size;
    # `noisy_stop` gives the block starts explicitly (blocks counted from a response start)
    n_stop = (noisy_pos // block_size) * block_size if noisy_stop is None else noisy_stop.to(i64)
    c_stop = clean_pos + 1 if clean_causal else (clean_pos // block_size + 1) * block_size
    stop = torch.cat([n_stop, c_stop])
    seq = torch.cat([ns, cs])
    start = torch.zeros_like(stop) if window is None else (stop - window).clamp_min(0)
    q_lo = seq * seq_stride + start
    q_hi = seq * seq_stride + stop
    q_grp = torch.cat([-(noisy_group.to(i64) + 1), torch.zeros_like(clean_pos)])
    k_code = torch.cat([-(noisy_group.to(i64) + 1), ks * seq_stride + kpos])
    i32 = torch.int32
    return MaskLayout(q_lo.to(i32).to(dev), q_hi.to(i32).to(dev), q_grp.to(i32).to(dev), k_code.to(i32).to(dev))


def single_sequence_layout(seq_len: int, block_size: int, device="cpu", views: int = 1) -> MaskLayout:
    """All blocks active, `views` noisy copies (Fast-dLLM v2 uses 2) sharing one clean copy."""
    pos = torch.arange(seq_len, device=device)
    npos = pos.repeat(views)
    ngrp = (pos // block_size).repeat(views) + torch.arange(views, device=device).repeat_interleave(seq_len) * (
        seq_len // block_size)
    return block_diffusion_layout(npos, ngrp, pos, block_size)


native.register_signatures({
    "tdllm_attn_bwd": (native.c_int, [native.c_void_p] * 10 + [native.c_int] * 4 + [native.c_ll] * 8
                       + [native.c_void_p] * 10 + [native.c_int, native.c_int, native.c_float,
                                                   native.c_void_p]),
    "tdllm_attn_bwd_fused": (native.c_int, [native.c_void_p] * 11 + [native.c_int] * 4 + [native.c_ll] * 8
                             + [native.c_void_p] * 7 + [native.c_int, native.c_int, native.c_int, native.c_float,
                                                        native.c_void_p]),
})


def backward_chunk_tiles() -> int:
    """Query tiles per chunk of the one-pass backward (TDLLM_ATTN_BWD_CHUNK; 0 = one chunk). Tiles of
    128 rows touch 2 MiB of the dQ accumulator each at 32 heads; 64 per chunk measured best at 32k and 128k
    rows (the accumulator rows of a chunk mostly stay in the 126 MB L2 while all key tiles add to them)."""
    return int(os.environ.get("TDLLM_ATTN_BWD_CHUNK", "64"))


def backward_mode() -> str:
    """"fused": one pass per key tile, dQ summed in fp32 (five tensor-core products per tile pair;
    the sum over key tiles is not bitwise repeatable). "split": a dQ kernel per query tile and a dK/dV
    kernel per key tile (seven products, deterministic; needs an even number of query heads per KV head).
    TDLLM_ATTN_BWD selects; fused is the default."""
    mode = os.environ.get("TDLLM_ATTN_BWD", "fused")
    if mode not in ("fused", "split"):
        raise ValueError(f"TDLLM_ATTN_BWD must be 'fused' or 'split', got {mode!r}")
    return mode


def attention_backward_native(q, k, v, out, dout, lse, layout: MaskLayout, scale: float,
                              dqkv: torch.Tensor | None = None):
    """Returns (dq, dk, dv) as [rows, heads, 128] tensors. When q, k and v index the same rows
    (self-attention over a packed projection) the three gradients are views of one packed
    [rows, (Hq + 2·Hkv)·128] buffer, ready for the fused q/k-norm + RoPE backward."""
    nq, Hq, D = q.shape
    nk, Hkv, _ = k.shape
    L = layout.tile_lists()
    dev = q.device
    if dout.stride(2) != 1 or dout.stride(1) != D:
        dout = dout.contiguous()
    if nq == nk:
        if dqkv is None:
            dqkv = torch.empty(nq, (Hq + 2 * Hkv) * D, dtype=q.dtype, device=dev)
        dq = dqkv[:, : Hq * D].view(nq, Hq, D)
        dk = dqkv[:, Hq * D:(Hq + Hkv) * D].view(nk, Hkv, D)
        dv = dqkv[:, (Hq + Hkv) * D:].view(nk, Hkv, D)
    else:
        dq = torch.empty(nq, Hq, D, dtype=q.dtype, device=dev)
        dk = torch.empty(nk, Hkv, D, dtype=q.dtype, device=dev)
        dv = torch.empty(nk, Hkv, D, dtype=q.dtype, device=dev)
    if lse.shape[1] != L["nq_pad"]:
        padded = torch.full((Hq, L["nq_pad"]), float("-inf"), dtype=torch.float32, device=dev)
        padded[:, :nq] = lse[:, :nq]
        lse = padded
    delta = torch.empty(2, Hq, L["nq_pad"], dtype=torch.float32, device=dev)
    if backward_mode() == "fused":
        W = layout.backward_work(backward_chunk_tiles())
        acc = scratch(dev, L["nq_pad"] * Hq * D + 2 * L["nk_pad"] * Hkv * D, key="attn_bwd_acc")
        rc = native.lib().tdllm_attn_bwd_fused(
            ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(dq), ptr(dk), ptr(dv), ptr(lse), ptr(delta), ptr(acc),
            nq, nk, Hq, Hkv, _rows_view(q), _rows_view(k), _rows_view(v), _rows_view(out),
            dout.stride(0), dq.stride(0), dk.stride(0), dv.stride(0),
            ptr(L["q_lo"]), ptr(L["q_hi"]), ptr(L["q_grp"]), ptr(L["k_code"]),
            ptr(W["w_ptr"]), ptr(W["w_idx"]), ptr(W["w_order"]), W["n_work"], L["nqt"], L["nkt"], float(scale),
            stream())
        native.check(rc, "attn_bwd_fused")
        return dq, dk, dv
    rc = native.lib().tdllm_attn_bwd(
        ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(dq), ptr(dk), ptr(dv), ptr(lse), ptr(delta),
        nq, nk, Hq, Hkv, _rows_view(q), _rows_view(k), _rows_view(v), _rows_view(out),
        dout.stride(0), dq.stride(0), dk.stride(0), dv.stride(0),
        ptr(L["q_lo"]), ptr(L["q_hi"]), ptr(L["q_grp"]), ptr(L["k_code"]),
        ptr(L["f_ptr"]), ptr(L["f_idx"]), ptr(L["f_order"]), ptr(L["b_ptr"]), ptr(L["b_idx"]),
        ptr(L["b_order"]), L["nqt"], L["nkt"], float(scale), stream())
    native.check(rc, "attn_bwd")
    return dq, dk, dv


def attention_forward_kernels(q, k, v, layout: MaskLayout, scale: float):
    """(out, lse) from the device kernels for any supported head width: the one-kernel form at 128, tensor-core
    products around the masked-softmax kernels at the other multiples of 64."""
    if q.shape[-1] == 128:
        return attention_forward_native(q, k, v, layout, scale)
    from .wide_attention import wide_attention_forward

    return wide_attention_forward(q, k, v, layout, scale)


def attention_backward_kernels(q, k, v, out, dout, lse, layout: MaskLayout, scale: float):
    """(dq, dk, dv) against given (out, lse), which may be merged over key shards, for any supported head width."""
    if q.shape[-1] == 128:
        return attention_backward_native(q, k, v, out, dout, lse, layout, scale)
    from .wide_attention import wide_attention_backward

    return wide_attention_backward(q, k, v, out, dout, lse, layout, scale)


class _BlockAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, layout, scale):
        out, lse = attention_forward_native(q, k, v, layout, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.layout, ctx.scale = layout, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward_native(q, k, v, out, dout, lse, ctx.layout, ctx.scale)
        return dq, dk, dv, None, None


def block_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: MaskLayout,
                    scale: float | None = None) -> torch.Tensor:
    """q [nq,Hq,D], k/v [nk,Hkv,D] -> out [nq,Hq,D] under the layout's mask."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if use_native(q, k, v) and q.shape[-1] == 128:
        return _BlockAttention.apply(q, k, v, layout, scale)
    if use_native(q, k, v) and q.shape[-1] != 128 and q.shape[-1] % 64 == 0:
        from .wide_attention import wide_block_attention

        return wide_block_attention(q, k, v, layout, scale)
    if q.is_cuda and q.dtype == torch.bfloat16:
        raise native.NativeKernelError("bf16 CUDA attention needs head_dim 128 or another multiple of 64 "
                                       "(no silent fallback)")
    return attention_reference(q, k, v, layout, scale)[0]


def split_packed_qkv(qkv: torch.Tensor, Hq: int, Hkv: int, D: int):
    rows = qkv.shape[0]
    q = qkv[:, : Hq * D].view(rows, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(rows, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(rows, Hkv, D)
    return q, k, v


class _PackedBlockAttention(torch.autograd.Function):
    """Self-attention over a packed [rows, (Hq+2Hkv)·D] projection; the backward writes the three
    gradients into one packed buffer, so no slice-gradient copies are needed."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, D, layout, scale, precomputed=None):
        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        if precomputed is not None:
            out, lse = precomputed      # results of an earlier forward on the same inputs
            out = out.view(qkv.shape[0], Hq, D)
        else:
            out, lse = attention_forward_native(q, k, v, layout, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (Hq, Hkv, D, layout, scale)
        return out.view(qkv.shape[0], Hq * D)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        Hq, Hkv, D, layout, scale = ctx.meta
        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        dqkv = torch.empty_like(qkv)
        attention_backward_native(q, k, v, out, dout.contiguous().view(-1, Hq, D), lse, layout, scale, dqkv)
        return dqkv, None, None, None, None, None, None


def packed_block_attention(qkv: torch.Tensor, Hq: int, Hkv: int, D: int, layout: MaskLayout,
                           scale: float | None = None, store=None, key=None) -> torch.Tensor:
    """qkv [rows, (Hq+2Hkv)·D] -> [rows, Hq·D]; queries and keys are the same rows.

    `store` / `key` connect the op to activation checkpointing: during the no-grad forward of a
    checkpointed layer the output and log-sum-exp are stashed under `key`; when the layer is
    recomputed for its backward pass they are reused instead of running the forward kernel again."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if use_native(qkv) and D == 128:
        if store is not None and store.keep_attention:
            ko, kl = (key, "attn_out"), (key, "attn_lse")
            if store.recording and not torch.is_grad_enabled():
                q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
                out, lse = attention_forward_native(q, k, v, layout, scale)
                store.stash(ko, out)
                store.stash(kl, lse)
                return out.view(qkv.shape[0], Hq * D)
            if store.replaying and store.has(ko):
                pre = (store.fetch(ko), store.fetch(kl))
                return _PackedBlockAttention.apply(qkv, Hq, Hkv, D, layout, scale, pre)
        return _PackedBlockAttention.apply(qkv, Hq, Hkv, D, layout, scale)
    if use_native(qkv) and D != 128 and D % 64 == 0:
        # other head widths (64, 256, 512): tensor-core products around a masked softmax kernel (ops/wide_attention.py)
        from .wide_attention import wide_block_attention

        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        return wide_block_attention(q, k, v, layout, scale).reshape(qkv.shape[0], Hq * D)
    if qkv.is_cuda and qkv.dtype == torch.bfloat16:
        raise native.NativeKernelError("bf16 CUDA attention needs head_dim 128 or another multiple of 64 "
                                       "(no silent fallback)")
    q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
    return attention_reference(q, k, v, layout, scale)[0].reshape(qkv.shape[0], Hq * D)
