"""Soft-label distillation through a frozen output head without keeping `[rows, V]` logits.

loss = Σ_r w_r · KL(softmax(t_r·Wᵀ) ‖ softmax(h_r·Wᵀ)) with W frozen. Rows are processed in
chunks: two tcgen05 GEMMs produce fp32 logit chunks for teacher and student, one kernel turns
them into per-row losses and the bf16 gradient of the student logits, and a third GEMM maps
that gradient back to the student hidden states — so only `chunk × V` logits exist at a time
and the gradient is computed during the forward pass (the upstream gradient is a scalar).

Counterparts: `frozen_linear_kl` (dllm_parallel/core/kernels/dflash_kl.py:72-121) and the KL kernels
of dllm_parallel/core/csrc/fused_linear_ce/fused_linear_ce_cuda.cu:367-480, :1270-1509.
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import ptr, stream, use_native
from .gemm import gemm

native.register_signatures({
    "tdllm_kl_rows": (native.c_int, [native.c_void_p] * 5 + [native.c_int, native.c_int, native.c_ll, native.c_void_p]),
})


def frozen_linear_kl_reference(h_student, h_teacher, w, weights):
    zs = h_student.float() @ w.float().t()
    zt = h_teacher.float() @ w.float().t()
    ls, lt = torch.log_softmax(zs, -1), torch.log_softmax(zt, -1)
    per = (lt.exp() * (lt - ls)).sum(-1)
    return (per * weights.float()).sum(), per


class _FrozenLinearKL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h_student, h_teacher, w, weights, chunk_rows):
        rows, H = h_student.shape
        V = w.shape[0]
        dev = h_student.device
        lib = native.lib()
        chunk = min(rows, chunk_rows)
        zs = torch.empty(chunk, V, dtype=torch.float32, device=dev)
        zt = torch.empty(chunk, V, dtype=torch.float32, device=dev)
        dlog = torch.empty(chunk, V, dtype=torch.bfloat16, device=dev)
        per = torch.empty(rows, dtype=torch.float32, device=dev)
        dh = torch.empty_like(h_student)
        wts = weights.float().contiguous()
        for r0 in range(0, rows, chunk):
            r1 = min(r0 + chunk, rows)
            n = r1 - r0
            gemm(h_student[r0:r1], w, out=zs[:n])
            gemm(h_teacher[r0:r1], w, out=zt[:n])
            native.check(lib.tdllm_kl_rows(ptr(zs), ptr(zt), ptr(wts[r0:r1]), ptr(per[r0:r1]), ptr(dlog), n, V, V,
                                           stream()), "kl_rows")
            gemm(dlog[:n], w, b_mn_major=True, out=dh[r0:r1])
        ctx.save_for_backward(dh)
        ctx.mark_non_differentiable(per)
        return (per * wts).sum(), per

    @staticmethod
    def backward(ctx, gsum, _gper):
        (dh,) = ctx.saved_tensors
        return dh * gsum.to(dh.dtype), None, None, None, None


def frozen_linear_kl(h_student: torch.Tensor, h_teacher: torch.Tensor, w: torch.Tensor, weights: torch.Tensor,
                     chunk_rows: int = 2048):
    """h_* [rows, H] (teacher carries no gradient), w [V, H] frozen, weights [rows] (0 = unsupervised).
    Returns (Σ weighted KL, per-row KL)."""
    if use_native(h_student, w):
        return _FrozenLinearKL.apply(h_student.contiguous(), h_teacher.detach().contiguous(), w.detach(), weights,
                                     chunk_rows)
    return frozen_linear_kl_reference(h_student, h_teacher.detach(), w.detach(), weights)
