"""Per-head q/k RMSNorm fused with rotary position embedding on the packed QKV projection.

Input and output are [rows, (Hq + 2·Hkv)·D]; q and k heads are normalised (Qwen3 style, weight
[D], optional) and rotated by their row's position, pairing element i with i + D/2; v heads pass
through. Reference counterpart: HF `q_norm`/`k_norm` + `apply_rotary`, eager
(dllm_parallel/core/models/backbones/nemotron/model.py:3132-3211, :3192, :3249).
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import grad_sink, mark_grad_written, ptr, scratch, stream, use_native


def rope_inv_freq(head_dim: int, theta: float, device=None, rotary_dim: int | None = None) -> torch.Tensor:
    """[head_dim / 2] inverse frequencies of the pairs (i, i + head_dim/2). With `rotary_dim` < head_dim (partial
    rotary embeddings) only the first rotary_dim/2 pairs rotate, at the frequencies of a rotary_dim-wide embedding;
    the other pairs get frequency 0, i.e. the identity. The kernels need nothing else: checkpoints whose heads keep
    the rotary dimensions in front (pairs (j, j + rotary_dim/2)) are brought into this pairing by a fixed
    permutation of the head dimensions at load time (`partial_rotary_permutation`), which q·k does not see."""
    r = head_dim if rotary_dim is None else int(rotary_dim)
    if r <= 0 or r > head_dim or r % 2:
        raise ValueError(f"rotary_dim must be an even number in (0, {head_dim}], got {r}")
    freq = torch.zeros(head_dim // 2, dtype=torch.float32, device=device)
    freq[: r // 2] = 1.0 / (theta ** (torch.arange(0, r, 2, dtype=torch.float32, device=device) / r))
    return freq


def partial_rotary_permutation(head_dim: int, rotary_dim: int) -> torch.Tensor:
    """perm[new] = old: head dimension `old` of a checkpoint that rotates pairs (j, j + rotary_dim/2) of its first
    `rotary_dim` dimensions sits at `new` here, where pairs are (i, i + head_dim/2). The pass-through dimensions fill
    the rest of both halves. Identity when rotary_dim == head_dim."""
    D, R = head_dim, rotary_dim
    h, rh = D // 2, R // 2
    perm = torch.empty(D, dtype=torch.long)
    perm[:rh] = torch.arange(rh)                               # first members of the rotating pairs
    perm[h: h + rh] = torch.arange(rh, R)                      # their partners
    rest = torch.arange(R, D)
    perm[rh:h] = rest[: h - rh]
    perm[h + rh:] = rest[h - rh:]
    return perm


def qk_norm_rope_reference(qkv, pos, inv_freq, qw, kw, Hq, Hkv, D, eps):
    rows = qkv.shape[0]
    x = qkv.float().view(rows, Hq + 2 * Hkv, D)
    ang = pos.float()[:, None] * inv_freq[None, :].float()
    cos = torch.cos(ang)[:, None, :]
    sin = torch.sin(ang)[:, None, :]

    def norm(t, w):
        if w is None:
            return t
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.float()

    def rot(t):
        a, b = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    q = rot(norm(x[:, :Hq], qw))
    k = rot(norm(x[:, Hq:Hq + Hkv], kw))
    v = x[:, Hq + Hkv:]
    return torch.cat([q, k, v], dim=1).reshape(rows, -1).to(qkv.dtype)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, inv_freq, qw, kw, Hq, Hkv, D, eps):
        rows = qkv.shape[0]
        out = torch.empty_like(qkv)
        native.check(native.lib().tdllm_qk_norm_rope_fwd(
            ptr(qkv), ptr(out), ptr(pos), ptr(inv_freq), ptr(qw), ptr(kw), rows, Hq, Hkv, D, eps,
            stream()), "qk_norm_rope_fwd")
        ctx.save_for_backward(qkv, pos, inv_freq, qw, kw)
        ctx.meta = (Hq, Hkv, D, eps)
        ctx.qref, ctx.kref = qw, kw
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, pos, inv_freq, qw, kw = ctx.saved_tensors
        Hq, Hkv, D, eps = ctx.meta
        rows = qkv.shape[0]
        dout = dout.contiguous()
        din = torch.empty_like(qkv)
        dqw = dkw = None
        tq = tk = None
        fp32 = acc = False
        if qw is not None:
            sq, aq = grad_sink(ctx.qref)
            sk, ak = grad_sink(ctx.kref)
            if sq is not None and sk is not None and aq == ak:
                tq, tk, fp32, acc = sq, sk, sq.dtype == torch.float32, aq
            else:
                dqw, dkw = torch.empty_like(qw), torch.empty_like(kw)
                tq, tk = dqw, dkw
        parts = native.lib().tdllm_qk_bwd_parts()
        scr = scratch(qkv.device, (parts + 1) * 2 * D)
        native.check(native.lib().tdllm_qk_norm_rope_bwd(
            ptr(dout), ptr(qkv), ptr(din), ptr(pos), ptr(inv_freq), ptr(qw), ptr(kw), ptr(tq),
            ptr(tk), int(fp32), int(acc), ptr(scr), rows, Hq, Hkv, D, eps, stream()),
            "qk_norm_rope_bwd")
        if qw is not None and dqw is None:
            mark_grad_written(ctx.qref)
            mark_grad_written(ctx.kref)
        return din, None, None, dqw, dkw, None, None, None, None


def qk_norm_rope(qkv: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor,
                 qw: torch.Tensor | None, kw: torch.Tensor | None, Hq: int, Hkv: int, D: int,
                 eps: float = 1e-6) -> torch.Tensor:
    if not use_native(qkv):
        return qk_norm_rope_reference(qkv, pos, inv_freq, qw, kw, Hq, Hkv, D, eps)
    if pos.dtype != torch.int32:
        pos = pos.to(torch.int32)
    return _QKNormRope.apply(qkv.contiguous(), pos, inv_freq, qw, kw, Hq, Hkv, D, eps)
