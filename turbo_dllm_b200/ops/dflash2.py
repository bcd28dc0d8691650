"""Building blocks of the DFlash2 drafter and its objective.

* `grouped_dynamic_conv`: a causal convolution along the positions of each drafting block whose taps are
  a learned base kernel per channel plus a per-token, per-group correction predicted from the input.
* `frozen_linear_ce_topk`: cross-entropy through the frozen verifier head together with the
  probability of the label and the top-k candidate tokens and their logits, without ever holding the
  `[rows, vocabulary]` logits: the head GEMM runs per vocabulary block (tcgen05 GEMM on a B200), the
  running top-k is merged block by block, and the loss itself is this package's fused linear
  cross-entropy.
* `dpace_weight`: the D-PACE position weights (how much a draft position is worth given how likely
  the positions before it are to be accepted).
* `selector_schedule_factor`: warm-up / ramp of the candidate-selector loss.

Reference counterparts: dllm_parallel/core/models/backbones/dflash/dflash2.py:40-53 (convolution),
:513-533 (D-PACE weights), dllm_parallel/core/kernels/dflash_linear_topk.py:238-278
(`frozen_linear_ce_topk`), dllm_parallel/core/models/backbones/dflash/training.py:91-104 (selector schedule).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .gemm import gemm
from .linear_ce import linear_cross_entropy

DPACE_LOSSES = ("dpace", "dpace-cumulative-confidence-only", "dpace-continuation-value-only")


def grouped_dynamic_conv(x: torch.Tensor, dynamic: torch.Tensor, base: torch.Tensor, block_size: int) -> torch.Tensor:
    """out[t] = Σ_i (base[i] + dynamic[t, i, group]) · x[t - i] inside each block (x[t - i] = 0 before
    the block start).

    x: [rows, H] with rows = whole blocks of `block_size`; dynamic: [rows, taps, groups];
    base: [taps, H]. Channels are split into `groups` consecutive groups that share a correction."""
    rows, H = x.shape
    taps, groups = dynamic.shape[1], dynamic.shape[2]
    if rows % block_size or H % groups:
        raise ValueError("grouped convolution needs whole blocks and a group count that divides the width")
    xb = x.reshape(rows // block_size, block_size, H).float()
    dyn = dynamic.reshape(rows // block_size, block_size, taps, groups).float()
    gs = H // groups
    out = torch.zeros_like(xb)
    for i in range(taps):
        shifted = xb if i == 0 else F.pad(xb[:, : block_size - i], (0, 0, i, 0))
        coef = base[i].float()[None, None, :] + dyn[:, :, i, :].repeat_interleave(gs, dim=-1)
        out = out + coef * shifted
    return out.reshape(rows, H).to(x.dtype)


def dpace_weight(probability: torch.Tensor, weight_mask: torch.Tensor, *, alpha: float, kind: str) -> torch.Tensor:
    """probability, weight_mask: [..., block]. prefix_t = Π_{s<=t} ((1-α) p_s + α) over supervised
    positions; `dpace` weighs position t by Σ_{s>=t} prefix_s·mask_s (what the rest of the block is
    worth if t is right), the two ablations keep only one of the factors."""
    smooth = (1.0 - alpha) * probability + alpha
    smooth = torch.where(weight_mask > 0, smooth, torch.ones_like(smooth))
    prefix = torch.cumprod(smooth, dim=-1)
    if kind == "dpace-cumulative-confidence-only":
        return prefix
    suffix = torch.flip(torch.cumsum(torch.flip(prefix * weight_mask, dims=(-1,)), dim=-1), dims=(-1,))
    if kind == "dpace":
        return suffix
    if kind == "dpace-continuation-value-only":
        return suffix / prefix.clamp_min(torch.finfo(prefix.dtype).tiny)
    raise ValueError(f"unsupported D-PACE loss {kind!r}")


def selector_schedule_factor(step: int, total_steps: int, warmup_ratio: float, ramp_ratio: float) -> float:
    warm = int(max(1, total_steps) * warmup_ratio)
    if step < warm:
        return 0.0
    ramp = int(max(1, total_steps) * ramp_ratio)
    return 1.0 if ramp <= 0 else min(max((step - warm + 1) / ramp, 0.0), 1.0)


def transform_logits(z: torch.Tensor, multiplier: float, softcap: float | None) -> torch.Tensor:
    z = z.float() * multiplier
    return torch.tanh(z / softcap) * softcap if softcap else z


class _GatherDot(torch.autograd.Function):
    """z[n, k] = h[n] · W[ids[n, k]] for a frozen W, in row chunks so that the gathered rows of W
    (chunk × k × H) never exist for all rows at once; the backward pass gathers them again."""

    @staticmethod
    def forward(ctx, h, w, ids, chunk):
        ctx.save_for_backward(h, w, ids)
        ctx.chunk = chunk
        out = torch.empty(ids.shape, dtype=torch.float32, device=h.device)
        for r0 in range(0, h.shape[0], chunk):
            r1 = min(r0 + chunk, h.shape[0])
            out[r0:r1] = torch.einsum("nh,nkh->nk", h[r0:r1].float(), w[ids[r0:r1]].float())
        return out

    @staticmethod
    def backward(ctx, g):
        h, w, ids = ctx.saved_tensors
        dh = torch.empty_like(h)
        for r0 in range(0, h.shape[0], ctx.chunk):
            r1 = min(r0 + ctx.chunk, h.shape[0])
            dh[r0:r1] = torch.einsum("nk,nkh->nh", g[r0:r1].float(), w[ids[r0:r1]].float()).to(h.dtype)
        return dh, None, None, None


@torch.no_grad()
def _topk_candidates(h: torch.Tensor, w: torch.Tensor, top_k: int, vocab_block: int, multiplier: float,
                     softcap: float | None, row_chunk: int = 4096):
    """Ids of the k largest transformed logits per row, merged over vocabulary blocks."""
    rows, V = h.shape[0], w.shape[0]
    best_v = torch.full((rows, top_k), float("-inf"), dtype=torch.float32, device=h.device)
    best_i = torch.zeros((rows, top_k), dtype=torch.long, device=h.device)
    for r0 in range(0, rows, row_chunk):
        r1 = min(r0 + row_chunk, rows)
        for v0 in range(0, V, vocab_block):
            v1 = min(v0 + vocab_block, V)
            z = transform_logits(gemm(h[r0:r1], w[v0:v1], out_dtype=torch.float32), multiplier, softcap)
            k = min(top_k, v1 - v0)
            val, idx = z.topk(k, dim=-1)
            cat_v = torch.cat([best_v[r0:r1], val], dim=-1)
            cat_i = torch.cat([best_i[r0:r1], idx + v0], dim=-1)
            sel = cat_v.topk(top_k, dim=-1).indices
            best_v[r0:r1] = cat_v.gather(1, sel)
            best_i[r0:r1] = cat_i.gather(1, sel)
    return best_i


def frozen_linear_ce_topk(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, *, top_k: int,
                          vocab_block_size: int = 32768, output_multiplier: float = 1.0,
                          logit_softcap: float | None = None, loss_weights: torch.Tensor | None = None):
    """Cross-entropy of `softcap(multiplier · hidden Wᵀ)` against `labels` through a frozen head.

    Returns (ce_sum, ce [rows], probability [rows], topk_logits [rows, k], candidate_ids [rows, k]):
    * `ce` and `probability = exp(-ce)` are detached per-row values;
    * `ce_sum = Σ loss_weights · ce` (all ones when None) carries the gradient to `hidden`;
    * `topk_logits` are the transformed logits of the k most likely tokens, differentiable in `hidden`.
    The caller may compute `loss_weights` from a first call's probabilities (D-PACE does) and call again."""
    w = weight.detach()
    scaled = hidden * output_multiplier if output_multiplier != 1.0 else hidden
    cap = float(logit_softcap) if logit_softcap else 0.0
    ce_sum, ce = linear_cross_entropy(scaled, w, labels, loss_weights, softcap=cap, frozen_weight=True)
    ce = ce.detach()
    ids = _topk_candidates(hidden.detach(), w, top_k, vocab_block_size, output_multiplier, logit_softcap)
    raw = _GatherDot.apply(hidden, w, ids, 2048)
    return ce_sum, ce, torch.exp(-ce), transform_logits(raw, output_multiplier, logit_softcap), ids
