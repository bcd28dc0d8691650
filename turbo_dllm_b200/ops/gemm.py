"""bf16 GEMM on tcgen05 tensor cores, and the linear layer built on it.

`gemm(a, b)` computes D[M,N] = A·B where `a` is given as [M,K] (or [K,M] with
`a_mn_major=True`) and `b` as [N,K] (or [K,N] with `b_mn_major=True`), so the forward,
input-gradient and weight-gradient products of y = x Wᵀ need no transpose copies.

The reference reaches cuBLAS through torch / Transformer Engine linears
(dllm_parallel/core/models/backbones/nemotron/model.py:3727-4190) and `cublasGemmEx`
(dllm_parallel/core/csrc/fused_linear_ce/fused_linear_ce_cuda.cu:618-791).
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import grad_sink, mark_grad_written, ptr, stream, use_native

EPI_STORE, EPI_SWIGLU, EPI_CE_STATS, EPI_CE_GRAD = 0, 1, 2, 3


def _as2d(t: torch.Tensor) -> torch.Tensor:
    return t if t.dim() == 2 else t.reshape(-1, t.shape[-1])


def gemm_reference(a, b, a_mn_major=False, b_mn_major=False):
    A = a.t() if a_mn_major else a
    B = b if b_mn_major else b.t()
    return A.float() @ B.float()


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
         accumulate: bool = False, swiglu: bool = False, max_ctas: int = 0,
         residual: torch.Tensor | None = None) -> torch.Tensor:
    """`residual` (same shape and dtype as the result) is added in the epilogue: D = A·B + residual."""
    a = _as2d(a)
    b = _as2d(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn_major else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn_major else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, dtype=out_dtype or a.dtype, device=a.device)
        accumulate = False
    if not use_native(a, b):
        res = gemm_reference(a, b, a_mn_major, b_mn_major)
        if swiglu:
            res = torch.nn.functional.silu(res[:, 0::2]) * res[:, 1::2]
        if residual is not None:
            res = res + residual.float()
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    if residual is not None:
        if accumulate or swiglu or residual.dtype != out.dtype or residual.shape != out.shape:
            raise ValueError("gemm: residual needs the result's shape and dtype, without accumulate/swiglu")
        residual = _as2d(residual)
    if a.stride(-1) != 1 or b.stride(-1) != 1 or out.stride(-1) != 1:
        raise ValueError("gemm: innermost stride must be 1")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("gemm: destination must be bf16 or fp32")
    rc = native.lib().tdllm_gemm_bf16(
        ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32),
        int(accumulate or residual is not None), EPI_SWIGLU if swiglu else EPI_STORE, None, None, None, None,
        -1, 0.0, max_ctas, ptr(residual), residual.stride(0) if residual is not None else 0, stream())
    native.check(rc, "gemm_bf16")
    return out


def _dgrad_over_tensor_parallel(dy2: torch.Tensor, w: torch.Tensor, tp) -> torch.Tensor:
    """dx = Σ_ranks dy_r · W_r for a weight split along its output rows (column-parallel linear): the
    all-reduce runs in the GEMM epilogue over peer memory when the product is large enough for that to
    pay, otherwise as an NCCL all-reduce after the GEMM."""
    import torch.distributed as dist

    fused = (tp.fused_allreduce(dy2.shape[0], w.shape[1], dy2.device)
             if (use_native(dy2, w) and w.shape[0] >= tp.fused_allreduce_min_k) else None)
    if fused is not None:
        return fused.matmul(dy2, w, b_mn_major=True)
    dx = gemm(dy2, w, b_mn_major=True)
    dist.all_reduce(dx, group=tp.group)
    return dx


class _Linear(torch.autograd.Function):
    """y = x Wᵀ with W [out, in]. The weight gradient goes straight into the parameter's
    slice of the flat gradient buffer when it has one (no .grad tensor, no extra add). With `tp`
    (column-parallel: W holds this rank's output rows, x is replicated) the input gradient is summed
    over the tensor-parallel group."""

    @staticmethod
    def forward(ctx, x, w, tp=None):
        ctx.save_for_backward(x, w)
        ctx.wref, ctx.tp = w, tp
        y = gemm(x, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = _as2d(dy.contiguous())
        x2 = _as2d(x)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = (_dgrad_over_tensor_parallel(dy2, w, ctx.tp) if ctx.tp is not None
                  else gemm(dy2, w, b_mn_major=True)).view_as(x)
        if ctx.needs_input_grad[1]:
            sink, acc = grad_sink(ctx.wref)
            if sink is not None:
                gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc)
                mark_grad_written(ctx.wref)
            else:
                dw = gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, tp=None) -> torch.Tensor:
    """`tp`: a TPContext of size > 1 makes this a column-parallel linear (see _Linear)."""
    return _Linear.apply(x, w, tp if (tp is not None and tp.size > 1) else None)


class _Replay:
    """Set while a checkpointed layer is re-run for its backward pass: the value of the layer's last
    product is then never read (the gradient of the layer output comes from outside), so the op only
    records what its backward needs and skips the GEMM."""
    skip_last_output = False


class skip_last_output:
    def __enter__(self):
        self.prev = _Replay.skip_last_output
        _Replay.skip_last_output = True

    def __exit__(self, *exc):
        _Replay.skip_last_output = self.prev


class _LinearResidual(torch.autograd.Function):
    """h = res + x Wᵀ with the add done in the GEMM epilogue (no separate pass over the stream)."""

    @staticmethod
    def forward(ctx, x, w, res, value_unused=False):
        ctx.save_for_backward(x, w)
        ctx.wref = w
        if value_unused:
            return torch.empty_like(res)
        return gemm(x, w, residual=_as2d(res)).view(res.shape)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = _as2d(dy.contiguous())
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn_major=True).view_as(x)
        if ctx.needs_input_grad[1]:
            sink, acc = grad_sink(ctx.wref)
            if sink is not None:
                gemm(dy2, _as2d(x), a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc)
                mark_grad_written(ctx.wref)
            else:
                dw = gemm(dy2, _as2d(x), a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, (dy if ctx.needs_input_grad[2] else None), None


def linear_residual(x: torch.Tensor, w: torch.Tensor, res: torch.Tensor) -> torch.Tensor:
    return _LinearResidual.apply(x, w, res)


class _RowParallelResidual(torch.autograd.Function):
    """h = res + Σ_ranks x_r W_rᵀ for a weight split along its input columns. The residual is added in
    the GEMM epilogue of rank 0 only, then one all-reduce finishes the sum; every rank receives the
    full gradient of the (replicated) residual stream."""

    @staticmethod
    def forward(ctx, x, w, res, group, rank, value_unused=False, tp=None):
        import torch.distributed as dist

        ctx.save_for_backward(x, w)
        ctx.wref = w
        if value_unused:
            return torch.empty_like(res)
        x2, r2 = _as2d(x), _as2d(res)
        # the in-kernel exchange costs a flag round trip per tile: it beats GEMM + NCCL all-reduce once a
        # tile carries enough tensor-core work (measured on 2 GPUs: 1.40 vs 1.67 ms at K = 6144 per rank,
        # 1.27 vs 0.90 ms at K = 2048 per rank, 32768 x 4096 outputs)
        fused = (tp.fused_allreduce(r2.shape[0], r2.shape[1], x.device)
                 if (tp is not None and use_native(x, w) and x2.shape[1] >= tp.fused_allreduce_min_k) else None)
        if fused is not None:   # all-reduce inside the GEMM epilogue over peer memory
            return fused.matmul(x2 if x2.is_contiguous() else x2.contiguous(), w, residual=r2).view(res.shape)
        out = gemm(x, w, residual=_as2d(res) if rank == 0 else None)
        dist.all_reduce(out, group=group)
        return out.view(res.shape)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = _as2d(dy.contiguous())
        dx = gemm(dy2, w, b_mn_major=True).view_as(x) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            sink, acc = grad_sink(ctx.wref)
            if sink is not None:
                gemm(dy2, _as2d(x), a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc)
                mark_grad_written(ctx.wref)
            else:
                dw = gemm(dy2, _as2d(x), a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, (dy if ctx.needs_input_grad[2] else None), None, None, None, None


def row_parallel_linear_residual(x, w_shard, res, tp, last: bool = False) -> torch.Tensor:
    """`tp`: parallel.tensor_parallel.TPContext (or None / size 1 for no tensor parallelism).
    `last`: this product is the layer's output (skipped when a checkpointed layer is replayed)."""
    unused = last and _Replay.skip_last_output and torch.is_grad_enabled()
    if tp is None or tp.size == 1:
        return _LinearResidual.apply(x, w_shard, res, unused)
    return _RowParallelResidual.apply(x, w_shard, res, tp.group, tp.rank, unused, tp)


class _LinearSwiGLU(torch.autograd.Function):
    """act = silu(g) * u where [g0,u0,g1,u1,...] = x W_guᵀ with interleaved gate/up rows.
    Without grad the activation is applied in the GEMM epilogue and the [rows, 2I]
    pre-activation never reaches HBM; with grad it is kept for the backward pass."""

    @staticmethod
    def forward(ctx, x, w_gu, tp=None):
        from .activation import swiglu_forward

        gu = gemm(x, w_gu)
        act = swiglu_forward(gu)
        ctx.save_for_backward(x, w_gu, gu)
        ctx.wref, ctx.tp = w_gu, tp
        return act.view(*x.shape[:-1], w_gu.shape[0] // 2)

    @staticmethod
    def backward(ctx, dact):
        from .activation import swiglu_backward

        x, w, gu = ctx.saved_tensors
        dgu = swiglu_backward(_as2d(dact.contiguous()), gu)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = (_dgrad_over_tensor_parallel(dgu, w, ctx.tp) if ctx.tp is not None
                  else gemm(dgu, w, b_mn_major=True)).view_as(x)
        if ctx.needs_input_grad[1]:
            sink, acc = grad_sink(ctx.wref)
            if sink is not None:
                gemm(dgu, _as2d(x), a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc)
                mark_grad_written(ctx.wref)
            else:
                dw = gemm(dgu, _as2d(x), a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, None


def linear_swiglu(x: torch.Tensor, w_gu: torch.Tensor, tp=None) -> torch.Tensor:
    """`tp`: a TPContext of size > 1 makes this a column-parallel projection (input gradient summed over it)."""
    if not (torch.is_grad_enabled() and (x.requires_grad or w_gu.requires_grad)):
        y = gemm(x, w_gu, swiglu=True)
        return y.view(*x.shape[:-1], w_gu.shape[0] // 2)
    return _LinearSwiGLU.apply(x, w_gu, tp if (tp is not None and tp.size > 1) else None)
