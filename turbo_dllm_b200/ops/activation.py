"""SwiGLU on interleaved (gate, up) columns: out[:, j] = silu(gu[:, 2j]) * gu[:, 2j+1].

Interleaving lets the gate-up GEMM apply the activation in its epilogue (one output tile holds
both halves of every pair). Reference counterpart: Transformer Engine `ops.SwiGLU` / HF
`act_fn(gate) * up` (dllm_parallel/core/models/backbones/nemotron/model.py:4149-4160).
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import ptr, stream, use_native


def swiglu_forward(gu: torch.Tensor) -> torch.Tensor:
    rows, two_i = gu.shape
    if not use_native(gu):
        return (torch.nn.functional.silu(gu[:, 0::2].float()) * gu[:, 1::2].float()).to(gu.dtype)
    out = torch.empty(rows, two_i // 2, dtype=gu.dtype, device=gu.device)
    native.check(native.lib().tdllm_swiglu_fwd(ptr(gu), ptr(out), rows, two_i // 2, stream()),
                 "swiglu_fwd")
    return out


def swiglu_backward(dy: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    rows, two_i = gu.shape
    if not use_native(gu):
        g = gu[:, 0::2].float()
        u = gu[:, 1::2].float()
        sig = torch.sigmoid(g)
        dg = dy.float() * u * sig * (1 + g * (1 - sig))
        du = dy.float() * g * sig
        return torch.stack([dg, du], dim=-1).reshape(rows, two_i).to(gu.dtype)
    dgu = torch.empty_like(gu)
    native.check(native.lib().tdllm_swiglu_bwd(ptr(dy), ptr(gu), ptr(dgu), rows, two_i // 2, stream()),
                 "swiglu_bwd")
    return dgu


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return swiglu_forward(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return swiglu_backward(dy.contiguous(), gu)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    shape = gu.shape
    out = _SwiGLU.apply(gu.reshape(-1, shape[-1]))
    return out.view(*shape[:-1], shape[-1] // 2)
