"""Tensor parallelism: Megatron-style column / row parallel projections, vocab-parallel embedding
and vocab-parallel fused linear cross-entropy, plus sequence-parallel gather / scatter.

* column-parallel (QKV, gate/up): the weight is split along its output rows; the input is
  replicated, so the forward needs no communication and the input gradient is all-reduced.
* row-parallel (O, down): the weight is split along its input columns; partial outputs are
  summed with an all-reduce. The residual stream is added in the GEMM epilogue of TP rank 0
  only, so the all-reduce produces `residual + Σ partials` without an extra pass.
* vocab-parallel embedding: masked lookup in the local vocabulary shard + all-reduce.
* vocab-parallel cross-entropy: local (max, Σexp, target) statistics from the tcgen05 GEMM
  epilogue on the local vocabulary shard, combined across ranks with one all-gather of the local
  log-sum-exp and one all-reduce of the target logit; the backward recomputes the local logits
  with the global log-sum-exp and all-reduces the hidden gradient.
* sequence parallel: rows are scattered along the sequence inside the TP group between
  blocks (reduce-scatter instead of all-reduce, all-gather before column-parallel GEMMs).

Counterparts: dllm_parallel/core/parallel/tensor_parallel/mappings.py:40-449,
layers.py:39-365, cross_entropy.py:18-276, sequence_parallel.py:22-379.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..profiling import collectives as coll

from ..ops.gemm import EPI_CE_GRAD, EPI_CE_STATS, gemm


# ---------------------------------------------------------------- mappings
class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel projection)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        coll.all_reduce(g, "tensor", group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel projection)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        coll.all_reduce(x, "tensor", group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherRowsSP(torch.autograd.Function):
    """Sequence parallel: all-gather rows forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = x.new_empty(world * x.shape[0], *x.shape[1:])
        coll.all_gather_into_tensor(out, x.contiguous(), "tensor", group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        out = g.new_empty(g.shape[0] // world, *g.shape[1:])
        if g.is_cuda:
            coll.reduce_scatter_tensor(out, g.contiguous(), "tensor", group=ctx.group)
        else:
            full = g.contiguous().clone()
            coll.all_reduce(full, "tensor", group=ctx.group)
            r = dist.get_rank(ctx.group)
            out = full[r * out.shape[0]:(r + 1) * out.shape[0]]
        return out, None


class _ScatterRowsSP(torch.autograd.Function):
    """Sequence parallel: reduce-scatter rows forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        n = x.shape[0] // world
        if x.is_cuda:
            out = x.new_empty(n, *x.shape[1:])
            coll.reduce_scatter_tensor(out, x.contiguous(), "tensor", group=group)
            return out
        full = x.contiguous().clone()
        coll.all_reduce(full, "tensor", group=group)
        r = dist.get_rank(group)
        return full[r * n:(r + 1) * n].clone()

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        out = g.new_empty(world * g.shape[0], *g.shape[1:])
        coll.all_gather_into_tensor(out, g.contiguous(), "tensor", group=ctx.group)
        return out, None


def copy_to_tensor_parallel(x, group):
    return x if group is None else _CopyToTP.apply(x, group)


def reduce_from_tensor_parallel(x, group):
    return x if group is None else _ReduceFromTP.apply(x, group)


def gather_sequence_parallel(x, group):
    return x if group is None else _GatherRowsSP.apply(x, group)


def scatter_sequence_parallel(x, group):
    return x if group is None else _ScatterRowsSP.apply(x, group)


class FusedSequenceParallelUnavailable:
    reason = ""


class TPContext:
    """Group handle plus the shard arithmetic the model needs."""

    def __init__(self, group=None, sequence_parallel: bool = False):
        self.group = group
        self.size = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.sequence_parallel = bool(sequence_parallel) and self.size > 1
        self._fused_ar: dict = {}
        # TDLLM_TP_FUSED_ALLREDUCE=0 keeps the row-parallel projections on GEMM + NCCL all-reduce
        import os

        self.fused_allreduce_enabled = os.environ.get("TDLLM_TP_FUSED_ALLREDUCE", "1") != "0"
        self.fused_allreduce_min_k = int(os.environ.get("TDLLM_TP_FUSED_ALLREDUCE_MIN_K", "4096"))

    def fused_allreduce(self, rows: int, cols: int, device):
        """Workspace of the GEMM whose epilogue all-reduces over peer memory, or None when the group
        cannot use it (CPU, no peer access, more than 8 ranks). Grown when a call brings more rows."""
        if not self.fused_allreduce_enabled or self.size < 2 or torch.device(device).type != "cuda":
            return None
        ws = self._fused_ar.get(cols)
        if ws is not None and ws is not False and ws.max_rows >= rows:
            return ws
        if ws is False:
            return None
        from .fused_allreduce import maybe_create

        if ws is not None:
            ws.close()
        ws = maybe_create(self.group, torch.device(device), rows, cols)
        self._fused_ar[cols] = ws if ws is not None else False
        return ws

    def fused_sequence_parallel(self, rows: int, cols: int, device):
        """Workspace of the fused all-gather→GEMM / GEMM→reduce-scatter kernels for activations of `rows` x
        `cols`, or None when the group cannot use them (CPU, no peer access, row shards that are not whole
        256-row tiles, TDLLM_TP_FUSED_SP=0): the caller then uses collectives around the GEMM."""
        import os

        if (self.size < 2 or torch.device(device).type != "cuda" or rows % (256 * self.size)
                or os.environ.get("TDLLM_TP_FUSED_SP", "1") == "0"
                or not getattr(self, "fused_sequence_parallel_enabled", True)):     # topology.tensor_parallel_overlap
            return None
        key = ("sp", rows, cols)
        ws = self._fused_ar.get(key)
        if ws is False:
            return None
        if ws is None:
            try:
                from .fused_sequence_parallel import FusedSequenceParallel

                ws = FusedSequenceParallel(self.group, torch.device(device), rows, cols)
            except Exception as e:   # no peer access, no kernels: keep the collective path and say why once
                FusedSequenceParallelUnavailable.reason = str(e)
                ws = False
            self._fused_ar[key] = ws
        return ws or None

    def ce_exchange(self, rows: int, device):
        """Peer-memory workspace for the cross-rank finish of vocab-parallel cross-entropy, or None."""
        if not self.fused_allreduce_enabled or self.size < 2 or torch.device(device).type != "cuda":
            return None
        ws = self._fused_ar.get("ce")
        if ws is False:
            return None
        if ws is not None and ws.max_rows >= rows:
            return ws
        from ..kernels import native
        from .fused_allreduce import CrossEntropyExchange

        if ws is not None:
            ws.close()
        try:
            ws = CrossEntropyExchange(self.group, torch.device(device), max(rows, 1024))
        except (RuntimeError, native.NativeKernelError):
            ws = None
        self._fused_ar["ce"] = ws if ws is not None else False
        return ws

    def shard(self, full: torch.Tensor, dim: int) -> torch.Tensor:
        n = full.shape[dim] // self.size
        return full.narrow(dim, self.rank * n, n)

    def vocab_range(self, vocab: int) -> tuple[int, int]:
        n = vocab // self.size
        return self.rank * n, (self.rank + 1) * n


# ------------------------------------------------------- vocab-parallel ops
class _VocabParallelEmbedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, weight, v0, v1, group):
        from ..ops._util import grad_sink

        inside = (tokens >= v0) & (tokens < v1)
        local = (tokens - v0).clamp(0, v1 - v0 - 1)
        out = weight.index_select(0, local)
        out = out * inside[:, None].to(out.dtype)
        coll.all_reduce(out, "tensor", group=group)
        ctx.save_for_backward(local, inside)
        ctx.wref = weight
        return out

    @staticmethod
    def backward(ctx, dy):
        from ..ops._util import grad_sink, mark_grad_written

        local, inside = ctx.saved_tensors
        dy = dy * inside[:, None].to(dy.dtype)
        sink, acc = grad_sink(ctx.wref)
        if sink is None:
            dw = torch.zeros_like(ctx.wref)
            dw.index_add_(0, local, dy.to(dw.dtype))
            return None, dw, None, None, None
        if not acc:
            sink.zero_()
        sink.index_add_(0, local, dy.to(sink.dtype))
        mark_grad_written(ctx.wref)
        return None, None, None, None, None


def vocab_parallel_embedding(tokens, weight_shard, tp: TPContext, vocab: int):
    v0, v1 = tp.vocab_range(vocab)
    return _VocabParallelEmbedding.apply(tokens, weight_shard, v0, v1, tp.group)


class _VocabParallelLinearCE(torch.autograd.Function):
    """Native path: h [rows,H] bf16 (replicated), w_shard [V/tp, H]."""

    @staticmethod
    def forward(ctx, h, w, labels, weights, v0, exclude_index, group, chunk_rows, tp=None):
        from ..kernels import native
        from ..ops._util import ptr, stream

        rows, H = h.shape
        Vl = w.shape[0]
        lib = native.lib()
        dev = h.device
        local_labels = torch.where((labels >= v0) & (labels < v0 + Vl), labels - v0,
                                   torch.full_like(labels, -1)).to(torch.int32).contiguous()
        ex = exclude_index - v0 if v0 <= exclude_index < v0 + Vl else -1
        nt = lib.tdllm_gemm_n_tiles(Vl)
        stats = torch.empty(rows, nt, 3, dtype=torch.float32, device=dev)
        native.check(lib.tdllm_gemm_bf16(ptr(h), ptr(w), None, rows, Vl, H, h.stride(0), w.stride(0), 0, 0, 0, 0, 0,
                                         EPI_CE_STATS, ptr(local_labels), None, None, ptr(stats), int(ex), 0.0, 0,
                                         None, 0, stream()), "vocab-parallel ce stats")
        exchange = tp.ce_exchange(rows, dev) if tp is not None else None
        if exchange is not None:   # shard statistics meet in peer memory: no collective call
            lse, tgt = exchange.finish(stats)
        else:
            s = stats.view(rows, nt, 3)
            mx = s[:, :, 0].amax(1)
            lse_local = mx + torch.log((s[:, :, 1] * torch.exp(s[:, :, 0] - mx[:, None])).sum(1))
            tgt = s[:, :, 2].sum(1)
            world = dist.get_world_size(group)
            all_lse = torch.empty(world, rows, dtype=torch.float32, device=dev)
            coll.all_gather_into_tensor(all_lse.view(-1), lse_local.contiguous(), "tensor", group=group)
            lse = torch.logsumexp(all_lse, dim=0)
            coll.all_reduce(tgt, "tensor", group=group)
        valid = labels >= 0
        per_row = torch.where(valid, lse - tgt, torch.zeros_like(lse))
        wts = torch.ones_like(per_row) if weights is None else weights.float()
        ctx.save_for_backward(h, w, local_labels, lse, (wts * valid.float()).contiguous())
        ctx.meta = (int(ex), group, int(chunk_rows))
        ctx.wref = w
        ctx.mark_non_differentiable(per_row)
        return (per_row * wts).sum(), per_row

    @staticmethod
    def backward(ctx, gsum, _g):
        from ..kernels import native
        from ..ops._util import grad_sink, mark_grad_written, ptr, stream

        h, w, local_labels, lse, rowscale = ctx.saved_tensors
        ex, group, chunk_rows = ctx.meta
        rows, H = h.shape
        Vl = w.shape[0]
        lib = native.lib()
        rowscale = (rowscale * gsum.float()).contiguous()
        dh = torch.empty_like(h)
        sink, acc = grad_sink(ctx.wref)
        dw = None if sink is not None else torch.zeros(Vl, H, dtype=torch.float32, device=h.device)
        chunk = min(rows, chunk_rows)
        dlog = torch.empty(chunk, Vl, dtype=torch.bfloat16, device=h.device)
        first = True
        for r0 in range(0, rows, chunk):
            r1 = min(r0 + chunk, rows)
            n = r1 - r0
            native.check(lib.tdllm_gemm_bf16(ptr(h[r0:r1]), ptr(w), ptr(dlog), n, Vl, H, h.stride(0), w.stride(0), Vl,
                                             0, 0, 0, 0, EPI_CE_GRAD, ptr(local_labels[r0:r1]), ptr(lse[r0:r1]),
                                             ptr(rowscale[r0:r1]), None, ex, 0.0, 0, None, 0, stream()),
                         "vocab-parallel ce grad")
            gemm(dlog[:n], w, b_mn_major=True, out=dh[r0:r1])
            if sink is not None:
                gemm(dlog[:n], h[r0:r1], a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc or not first)
            else:
                gemm(dlog[:n], h[r0:r1], a_mn_major=True, b_mn_major=True, out=dw, accumulate=not first)
            first = False
        coll.all_reduce(dh, "tensor", group=group)
        if sink is not None:
            mark_grad_written(ctx.wref)
        else:
            dw = dw.to(w.dtype)
        return dh, dw, None, None, None, None, None, None, None


def vocab_parallel_linear_cross_entropy(h, w_shard, labels, weights, tp: TPContext, vocab: int,
                                        exclude_index: int = -1, chunk_rows: int = 8192):
    """Returns (Σ weighted loss, per-row loss); identical on every TP rank."""
    from ..ops._util import use_native

    v0, v1 = tp.vocab_range(vocab)
    if use_native(h, w_shard):
        return _VocabParallelLinearCE.apply(h.contiguous(), w_shard, labels, weights, v0, exclude_index, tp.group,
                                            chunk_rows, tp)
    # reference path (CPU / fp32): gather the shards' logits statistics with autograd-aware ops
    hc = copy_to_tensor_parallel(h, tp.group)
    z = hc.float() @ w_shard.float().t()
    if v0 <= exclude_index < v1:
        z = z.clone()
        z[:, exclude_index - v0] = float("-inf")
    m_local = z.max(dim=1).values.detach()
    m = m_local.clone()
    coll.all_reduce(m, "tensor", op=dist.ReduceOp.MAX, group=tp.group)
    se = reduce_from_tensor_parallel(torch.exp(z - m[:, None]).sum(1), tp.group)
    inside = (labels >= v0) & (labels < v1)
    loc = (labels - v0).clamp(0, v1 - v0 - 1)
    zt = hc.float() @ w_shard.float().t() if v0 <= exclude_index < v1 else z
    tgt = reduce_from_tensor_parallel(torch.where(inside, zt.gather(1, loc[:, None])[:, 0], torch.zeros_like(m)),
                                      tp.group)
    valid = labels >= 0
    per_row = torch.where(valid, m + torch.log(se) - tgt, torch.zeros_like(m))
    wts = torch.ones_like(per_row) if weights is None else weights.float()
    return (per_row * wts).sum(), per_row.detach()


# ------------------------------------------------------- sequence parallelism inside the tensor-parallel group
# The residual stream is sharded along rows: rank r holds rows [r·n, (r+1)·n) of `rows = n·T`. A column-parallel
# projection first gathers the rows (all-gather → GEMM; backward: input gradient → reduce-scatter), a row-parallel
# projection ends in a reduce-scatter of its partial sums (GEMM → reduce-scatter; backward: all-gather → GEMMs).
# On CUDA with peer access both run as ONE kernel each (csrc/gemm_sm100.cu: the gather is pulled into local memory
# by extra warps of the GEMM while tiles of local rows run; the scatter is the reduce-scatter form of the
# all-reduce epilogue); elsewhere they are collectives followed / preceded by the GEMM.
# Counterparts: dllm_parallel/core/parallel/tensor_parallel/sequence_parallel.py:158-285 and the userbuffers
# overlap of dllm_parallel/core/parallel/transformer_engine.py:84-139.

def _gather_rows(x: torch.Tensor, tp: TPContext) -> torch.Tensor:
    out = x.new_empty(tp.size * x.shape[0], *x.shape[1:])
    coll.all_gather_into_tensor(out, x.contiguous(), "tensor", group=tp.group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, tp: TPContext) -> torch.Tensor:
    n = x.shape[0] // tp.size
    if x.is_cuda:
        out = x.new_empty(n, *x.shape[1:])
        coll.reduce_scatter_tensor(out, x.contiguous(), "tensor", group=tp.group)
        return out
    full = x.contiguous().clone()
    coll.all_reduce(full, "tensor", group=tp.group)
    return full[tp.rank * n:(tp.rank + 1) * n].clone()


class _TakeRowsSP(torch.autograd.Function):
    """Full (replicated) rows -> this rank's rows; backward all-gathers the ranks' row gradients."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        n = x.shape[0] // tp.size
        return x[tp.rank * n:(tp.rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _gather_rows(g, ctx.tp), None


class _GatherRowsReplicatedGrad(torch.autograd.Function):
    """This rank's rows -> all rows, for consumers that compute the SAME thing on every rank (final norm and
    the vocabulary-parallel loss, whose hidden-state gradient is already summed): backward takes the slice."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _gather_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        n = g.shape[0] // tp.size
        return g[tp.rank * n:(tp.rank + 1) * n].contiguous(), None


def take_rows_sequence_parallel(x, tp: TPContext):
    return _TakeRowsSP.apply(x, tp)


def gather_rows_replicated_grad(x, tp: TPContext):
    return _GatherRowsReplicatedGrad.apply(x, tp)


class _GatherLinearSP(torch.autograd.Function):
    """y = gather_rows(x_local) · Wᵀ for a column-parallel W (optionally with SwiGLU on interleaved gate/up)."""

    @staticmethod
    def forward(ctx, x_local, w, tp, swiglu):
        from ..ops._util import use_native
        from ..ops.activation import swiglu_forward

        fused = tp.fused_sequence_parallel(x_local.shape[0] * tp.size, x_local.shape[1], x_local.device) \
            if use_native(x_local, w) else None
        if fused is not None:
            y, x_full = fused.gather_matmul(x_local, w)
            if torch.is_grad_enabled() and not getattr(tp, "sp_saved_in_place", False):
                x_full = x_full.clone()     # the rotating buffer is reused before an un-checkpointed backward
        else:
            x_full = _gather_rows(x_local, tp)
            y = gemm(x_full, w)
        ctx.tp, ctx.wref, ctx.swiglu = tp, w, swiglu
        if swiglu:
            act = swiglu_forward(y)
            ctx.save_for_backward(x_full, w, y)
            return act
        ctx.save_for_backward(x_full, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops._util import grad_sink, mark_grad_written, use_native
        from ..ops.activation import swiglu_backward

        tp = ctx.tp
        if ctx.swiglu:
            x_full, w, gu = ctx.saved_tensors
            dy = swiglu_backward(dy.contiguous(), gu)
        else:
            x_full, w = ctx.saved_tensors
            dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            fused = tp.fused_sequence_parallel(dy.shape[0], w.shape[1], dy.device) if use_native(dy, w) else None
            if fused is not None:
                dx = fused.matmul_scatter(dy, w, b_mn_major=True)
            else:
                dx = _reduce_scatter_rows(gemm(dy, w, b_mn_major=True), tp)
        if ctx.needs_input_grad[1]:
            sink, acc = grad_sink(ctx.wref)
            if sink is not None:
                gemm(dy, x_full, a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc)
                mark_grad_written(ctx.wref)
            else:
                dw = gemm(dy, x_full, a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, None, None


class _LinearScatterResidualSP(torch.autograd.Function):
    """h_local = res_local + reduce_scatter_rows(x · W_rᵀ) for a row-parallel W (split along its input)."""

    @staticmethod
    def forward(ctx, x, w, res_local, tp, value_unused):
        from ..ops._util import use_native

        ctx.save_for_backward(x, w)
        ctx.tp, ctx.wref = tp, w
        if value_unused:
            return torch.empty_like(res_local)
        fused = tp.fused_sequence_parallel(x.shape[0], w.shape[0], x.device) if use_native(x, w) else None
        if fused is not None:
            return fused.matmul_scatter(x if x.is_contiguous() else x.contiguous(), w, residual=res_local)
        return res_local + _reduce_scatter_rows(gemm(x, w), tp)

    @staticmethod
    def backward(ctx, dy_local):
        from ..ops._util import grad_sink, mark_grad_written, use_native

        x, w = ctx.saved_tensors
        tp = ctx.tp
        dx = dw = None
        dy_local = dy_local.contiguous()
        fused = tp.fused_sequence_parallel(x.shape[0], w.shape[0], x.device) if use_native(x, w) else None
        if fused is not None and ctx.needs_input_grad[0]:
            dx, dy = fused.gather_matmul(dy_local, w, b_mn_major=True)
        else:
            dy = _gather_rows(dy_local, tp)
            if ctx.needs_input_grad[0]:
                dx = gemm(dy, w, b_mn_major=True)
        if ctx.needs_input_grad[1]:
            sink, acc = grad_sink(ctx.wref)
            if sink is not None:
                gemm(dy, x, a_mn_major=True, b_mn_major=True, out=sink, accumulate=acc)
                mark_grad_written(ctx.wref)
            else:
                dw = gemm(dy, x, a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, (dy_local if ctx.needs_input_grad[2] else None), None, None


def sp_column_linear(x_local, w, tp: TPContext, swiglu: bool = False):
    return _GatherLinearSP.apply(x_local, w, tp, swiglu)


def sp_row_linear_residual(x, w_shard, res_local, tp: TPContext, last: bool = False):
    from ..ops.gemm import _Replay

    unused = last and _Replay.skip_last_output and torch.is_grad_enabled()
    return _LinearScatterResidualSP.apply(x, w_shard, res_local, tp, unused)


def sync_partial_gradients(params, tp: TPContext) -> None:
    """Sums, over the tensor-parallel group, the gradients of replicated parameters that every rank computed
    from ITS part of the work only (`param.tp_partial`): per-head q/k norm weights see this rank's heads, and
    under sequence parallelism the layer norms see this rank's rows. One all-reduce over a packed copy.
    Counterpart of the replicated-parameter sync of dllm_parallel/core/parallel/grad_sync.py:110-187."""
    todo = [p for p in params if getattr(p, "tp_partial", False) and getattr(p, "main_grad", None) is not None]
    if not todo or tp is None or tp.size == 1:
        return
    flat = torch.cat([p.main_grad.reshape(-1).float() for p in todo])
    coll.all_reduce(flat, "tensor", group=tp.group)
    off = 0
    for p in todo:
        n = p.main_grad.numel()
        p.main_grad.copy_(flat[off:off + n].view_as(p.main_grad).to(p.main_grad.dtype))
        off += n
