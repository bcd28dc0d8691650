"""Fused linear + cross-entropy: the `[rows, vocab]` logits are never materialised in fp32.

loss_sum = Σ_r w_r · (logsumexp_v(h_r·W_vᵀ) − h_r·W_{y_r}ᵀ) over rows with label >= 0.

* `linear_ce_reference` – vocab-tiled online log-sum-exp in plain PyTorch (CPU oracle and fp32 path).
* native path – forward: the tcgen05 GEMM's epilogue reduces every 128×256 logits tile to
  (max, Σexp, target logit) per row; a small kernel combines the tiles into lse and the loss.
  Backward: per row chunk the GEMM is recomputed with an epilogue that writes
  (softmax − onehot)·scale as bf16, followed by dH = dlogits·W and dW += dlogitsᵀ·H.
* options: `exclude_index` removes one vocabulary column from the softmax (the mask token under
  standard block diffusion), `softcap`, frozen weight (no dW).

Reference counterparts: `_TiledLinearCrossEntropy` (dllm_parallel/core/kernels/tiled_linear_cross_entropy.py:56-277),
`_ChunkedDenseLinearCrossEntropy` (:280-368) and the CUDA drivers of
dllm_parallel/core/csrc/fused_linear_ce/fused_linear_ce_cuda.cu:898-1172.
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import grad_sink, mark_grad_written, ptr, stream, use_native
from .gemm import EPI_CE_GRAD, EPI_CE_STATS, gemm

IGNORE = -100


def _softcap(x, cap):
    return cap * torch.tanh(x / cap) if cap and cap > 0 else x


def linear_ce_reference(h, w, labels, weights=None, exclude_index: int = -1, softcap: float = 0.0,
                        vocab_tile: int = 8192):
    """Differentiable (plain autograd). Returns (weighted loss sum, per-row loss)."""
    hf, wf = h.float(), w.float()
    rows, V = hf.shape[0], wf.shape[0]
    m = torch.full((rows,), float("-inf"), device=h.device)
    s = torch.zeros(rows, device=h.device)
    tgt = torch.zeros(rows, device=h.device)
    valid = labels >= 0
    safe = labels.clamp_min(0)
    for v0 in range(0, V, vocab_tile):
        v1 = min(v0 + vocab_tile, V)
        z = _softcap(hf @ wf[v0:v1].t(), softcap)
        inside = valid & (safe >= v0) & (safe < v1)
        tgt = tgt + torch.where(inside, z.gather(1, (safe - v0).clamp(0, v1 - v0 - 1)[:, None])[:, 0],
                                torch.zeros_like(tgt))
        if v0 <= exclude_index < v1:
            z = z.clone()
            z[:, exclude_index - v0] = float("-inf")
        tm = z.max(dim=1).values
        nm = torch.maximum(m, tm)
        s = s * torch.exp(m - nm) + torch.exp(z - nm[:, None]).sum(1)
        m = nm
    lse = m + torch.log(s)
    per_row = torch.where(valid, lse - tgt, torch.zeros_like(lse))
    wts = torch.ones_like(per_row) if weights is None else weights.float()
    return (per_row * wts).sum(), per_row


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, weights, exclude_index, softcap, frozen, chunk_rows):
        rows, H = h.shape
        V = w.shape[0]
        lib = native.lib()
        dev = h.device
        nt = lib.tdllm_gemm_n_tiles(V)
        stats = torch.empty(rows, nt, 3, dtype=torch.float32, device=dev)
        labels32 = labels.to(torch.int32).contiguous()
        rc = lib.tdllm_gemm_bf16(ptr(h), ptr(w), None, rows, V, H, h.stride(0), w.stride(0), 0, 0, 0, 0, 0,
                                 EPI_CE_STATS, ptr(labels32), None, None, ptr(stats), int(exclude_index),
                                 float(softcap), 0, None, 0, stream())
        native.check(rc, "linear_ce stats gemm")
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        per_row = torch.empty(rows, dtype=torch.float32, device=dev)
        out2 = torch.zeros(2, dtype=torch.float32, device=dev)
        wts = None if weights is None else weights.float().contiguous()
        native.check(lib.tdllm_ce_finalize(ptr(stats), rows, nt, ptr(labels32), ptr(wts), ptr(lse),
                                           ptr(per_row), ptr(out2), stream()), "ce_finalize")
        ctx.save_for_backward(h, w, labels32, wts, lse)
        ctx.wref = w
        ctx.opts = (int(exclude_index), float(softcap), bool(frozen), int(chunk_rows))
        ctx.mark_non_differentiable(per_row)
        return out2[0], per_row

    @staticmethod
    def backward(ctx, gsum, _gper):
        h, w, labels32, wts, lse = ctx.saved_tensors
        exclude_index, softcap, frozen, chunk_rows = ctx.opts
        rows, H = h.shape
        V = w.shape[0]
        lib = native.lib()
        dev = h.device
        valid = (labels32 >= 0).float()
        rowscale = (valid if wts is None else valid * wts) * gsum.float()
        dh = torch.empty_like(h) if ctx.needs_input_grad[0] else None
        want_dw = ctx.needs_input_grad[1] and not frozen
        sink, acc = grad_sink(ctx.wref) if want_dw else (None, False)
        dw = None
        if want_dw and sink is None:
            dw = torch.zeros(V, H, dtype=torch.float32, device=dev)
        chunk = min(rows, chunk_rows)
        dlog = torch.empty(chunk, V, dtype=torch.bfloat16, device=dev)
        first = True
        for r0 in range(0, rows, chunk):
            r1 = min(r0 + chunk, rows)
            n = r1 - r0
            hc = h[r0:r1]
            rc = lib.tdllm_gemm_bf16(ptr(hc), ptr(w), ptr(dlog), n, V, H, h.stride(0), w.stride(0), V, 0, 0,
                                     0, 0, EPI_CE_GRAD, ptr(labels32[r0:r1]), ptr(lse[r0:r1]),
                                     ptr(rowscale[r0:r1]), None, exclude_index, softcap, 0, None, 0, stream())
            native.check(rc, "linear_ce grad gemm")
            d = dlog[:n]
            if dh is not None:
                gemm(d, w, b_mn_major=True, out=dh[r0:r1])
            if want_dw:
                if sink is not None:
                    gemm(d, hc, a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc or not first)
                else:
                    gemm(d, hc, a_mn_major=True, b_mn_major=True, out=dw, accumulate=not first)
            first = False
        if want_dw and sink is not None:
            mark_grad_written(ctx.wref)
            dw = None
        elif dw is not None:
            dw = dw.to(w.dtype)
        return dh, dw, None, None, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor,
                         weights: torch.Tensor | None = None, *, exclude_index: int = -1,
                         softcap: float = 0.0, frozen_weight: bool = False, chunk_rows: int = 8192):
    """h [rows, H], w [V, H], labels [rows] (negative = ignored), weights [rows] or None.
    Returns (Σ weighted loss, per-row loss)."""
    if use_native(h, w):
        return _LinearCE.apply(h.contiguous(), w, labels, weights, exclude_index, softcap, frozen_weight,
                               chunk_rows)
    if frozen_weight:
        w = w.detach()
    return linear_ce_reference(h, w, labels, weights, exclude_index, softcap)
