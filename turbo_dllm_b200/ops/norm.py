"""RMSNorm with optional fused residual add: h = x + res; y = h * rsqrt(mean(h²)+eps) * w.

Reference counterpart: HF RMSNorm modules and TE `LayerNormLinear(normalization="RMSNorm")`
(dllm_parallel/core/models/backbones/nemotron/model.py:3866-3960).
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import grad_sink, mark_grad_written, ptr, scratch, stream, use_native


def rmsnorm_reference(x, w, eps, res=None):
    h = x if res is None else x + res
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    return (hf * rstd * w.float()).to(x.dtype), h


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        rows = x2.shape[0]
        has_res = res is not None
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if has_res else x2
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        native.check(native.lib().tdllm_rmsnorm_fwd(
            ptr(x2), ptr(res.reshape(-1, H)) if has_res else None, ptr(w), ptr(y),
            ptr(h) if has_res else None, ptr(rstd), rows, H, eps, stream()), "rmsnorm_fwd")
        ctx.save_for_backward(h, w, rstd)
        ctx.wref = w
        ctx.has_res = has_res
        ctx.shape = x.shape
        if has_res:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, w, rstd = ctx.saved_tensors
        rows, H = h.shape
        dy2 = dy.contiguous().reshape(rows, H)
        # gradient flowing into the residual stream output (h) adds to dx
        dres = dh.contiguous().reshape(rows, H) if dh is not None else None
        dx = torch.empty_like(h)
        parts = native.lib().tdllm_rmsnorm_bwd_parts()
        scr = scratch(h.device, parts * H)
        sink, acc = grad_sink(ctx.wref)
        if sink is None:
            dw = torch.empty_like(w)
            target, tfp32, tacc = dw, False, False
        else:
            dw = None
            target, tfp32, tacc = sink, sink.dtype == torch.float32, acc
        native.check(native.lib().tdllm_rmsnorm_bwd(
            ptr(dy2), ptr(h), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(target), int(tfp32),
            int(tacc), ptr(scr), rows, H, stream()), "rmsnorm_bwd")
        if sink is not None:
            mark_grad_written(ctx.wref)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_res else None), dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
            res: torch.Tensor | None = None):
    """Returns (y, h) where h = x + res is the updated residual stream (h is x when res is None)."""
    if not use_native(x):
        return rmsnorm_reference(x, w, eps, res)
    if res is None:
        return _RMSNorm.apply(x, None, w, eps), x
    y, h = _RMSNorm.apply(x, res, w, eps)
    return y, h
