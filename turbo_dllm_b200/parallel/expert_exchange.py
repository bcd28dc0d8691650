"""Expert-parallel dispatch / combine over peer memory, as autograd functions around the grouped expert GEMMs.

    x ──dispatch──▶ x_pad (owner's slab, padded expert segments) ──grouped GEMMs──▶ y_pad ──combine──▶ out

`dispatch` writes every (token, choice) row straight into the slab of the expert's owner, `combine` pulls the
expert outputs back and weights them; the backward pass runs the same two transfers in the other direction
(csrc/moe_dispatch.cu). Nothing on this path calls NCCL or reads routing data on the host: counts travel through
a symmetric table, layouts are computed on the device, and slabs have a static capacity
(`TDLLM_EP_CAPACITY_FACTOR` x the balanced load; an overflow sets the device error record instead of writing out
of bounds).

Every routed batch starts with the counts exchange, which no rank leaves before every rank has entered it. That
is what makes one set of slabs enough: a rank cannot write rows of the next batch into a peer's slab while the
peer still computes on the previous one.

Counterpart of the DeepEP buffer and its dispatch / combine autograd ops
(dllm_parallel/core/parallel/expert/deepep.py:122-555).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..kernels import native
from ..ops._util import ptr, stream
from ..ops.grouped import GroupedRows
from ..profiling.operator_trace import communication_scope
from .symm import SymmetricBarrier, SymmetricBuffer, peer_access_available

_V, _I, _LL = native.c_void_p, native.c_int, native.c_ll
native.register_signatures({
    "tdllm_ep_counts_exchange": (_I, [_V, _V, _V, _I, _I, _I, _I, _V]),
    "tdllm_ep_dispatch": (_I, [_V] * 8 + [_LL, _I, _I, _I, _LL, _I, _V]),
    "tdllm_ep_zero_pad_rows": (_I, [_V, _V, _V, _I, _I, _V]),
    "tdllm_ep_combine": (_I, [_V] * 6 + [_LL, _I, _I, _I, _I, _V]),
    "tdllm_ep_weight_grad": (_I, [_V, _V, _V, _LL, _I, _I, _V]),
})


class PeerExpertExchange:
    """Symmetric slabs and tables of one expert-parallel group (shared by all layers of a model)."""

    def __init__(self, group, device: torch.device, *, rows: int, top_k: int, hidden: int, num_experts: int):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 2 <= self.world <= 16 or num_experts % self.world or hidden % 64:
            raise RuntimeError("peer expert exchange needs 2..16 ranks, experts divisible by them, hidden % 64 == 0")
        if not peer_access_available(group):
            raise RuntimeError("GPUs of this group cannot address one another (no peer access)")
        self.E, self.el, self.k, self.H = num_experts, num_experts // self.world, top_k, hidden
        t = torch.tensor([rows], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        self.max_rows = int(t)
        factor = float(os.environ.get("TDLLM_EP_CAPACITY_FACTOR", "2.0"))
        self.cap = (int(self.max_rows * top_k * factor) + 256 * self.el + 255) // 256 * 256
        nbytes = self.cap * hidden * 2
        self.x_buf = SymmetricBuffer(nbytes, group, device)      # dispatched activations (kept for the weight gradient)
        self.dy_buf = SymmetricBuffer(nbytes, group, device)     # dispatched output gradients
        self.out_buf = SymmetricBuffer(nbytes, group, device)    # expert outputs / input gradients, pulled by sources
        self.tab = SymmetricBuffer(self.world * self.E * 4, group, device)
        self.flags = SymmetricBuffer(256, group, device)
        self.barrier = SymmetricBarrier(group, device)
        self.epoch = 0
        self.counters = torch.zeros(self.E, dtype=torch.int32, device=device)
        self.x_slab = self.x_buf.as_tensor(torch.bfloat16, self.cap * hidden).view(self.cap, hidden)
        self.dy_slab = self.dy_buf.as_tensor(torch.bfloat16, self.cap * hidden).view(self.cap, hidden)
        self.out_slab = self.out_buf.as_tensor(torch.bfloat16, self.cap * hidden).view(self.cap, hidden)
        self.tab_local = self.tab.as_tensor(torch.int32, self.world * self.E).view(self.world, self.E)

    def close(self) -> None:
        for b in (self.x_buf, self.dy_buf, self.out_buf, self.tab, self.flags, self.barrier.buf):
            b.close()

    # one routed batch: counts exchange and the layouts that follow from it
    def plan(self, experts_flat: torch.Tensor):
        lib = native.lib()
        W, E, el, r = self.world, self.E, self.el, self.rank
        counts = torch.bincount(experts_flat, minlength=E).to(torch.int32)
        self.epoch += 1
        with communication_scope("expert", "forward", "counts_exchange", E * 4 * (W - 1)):
            native.check(lib.tdllm_ep_counts_exchange(ptr(counts), self.tab.ptr_array, self.flags.ptr_array, r, W, E,
                                                      self.epoch, stream()), "ep_counts_exchange")
        tab = self.tab_local.clone().long()                         # [source, expert]
        tot = tab.sum(0)
        padded = (tot + 255) // 256 * 256
        per_owner = padded.view(W, el)
        begins = (per_owner.cumsum(1) - per_owner).reshape(E)       # first slab row of every expert, per owner
        base = (begins + tab[:r].sum(0)).contiguous()               # this rank's first slot per expert
        my_begin = begins.view(W, el)[r].contiguous()
        my_count = tot.view(W, el)[r].contiguous()
        my_padded = per_owner[r]
        ends = my_begin + my_padded
        tile_start = torch.arange(self.cap // 128, device=self.device) * 128
        mt_group = torch.searchsorted(ends, tile_start, right=True).clamp_(max=el - 1).to(torch.int32).contiguous()
        valid = tile_start < ends[-1]
        blocks_end = (my_begin + (my_count + 63) // 64 * 64) // 64
        g = GroupedRows(el, self.cap, None, mt_group, my_begin, blocks_end, valid)
        return base, my_begin, my_count, g


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, experts_flat, ex: PeerExpertExchange, state: dict):
        lib = native.lib()
        rows, H = x.shape
        base, my_begin, my_count, g = ex.plan(experts_flat)
        pos = torch.empty(rows * ex.k, dtype=torch.int32, device=x.device)
        ex.counters.zero_()
        native.check(lib.tdllm_ep_zero_pad_rows(ex.x_buf.local, ptr(my_begin), ptr(my_count), ex.el, H, stream()),
                     "ep_zero_pad_rows")
        with communication_scope("expert", "forward", "dispatch", rows * ex.k * H * 2):
            native.check(lib.tdllm_ep_dispatch(ptr(x), ptr(experts_flat), None, ptr(base), ptr(ex.counters), None,
                                               ptr(pos), ex.x_buf.ptr_array, rows, ex.k, H, ex.el, ex.cap, ex.world,
                                               stream()), "ep_dispatch")
        ex.barrier.sync()          # every source's rows are in this rank's slab
        state.update(pos=pos, g=g, my_begin=my_begin, my_count=my_count, experts=experts_flat, rows=rows)
        ctx.ex, ctx.state = ex, state
        # the slab is reused by the next routed batch: what autograd keeps must be a copy (and an autograd
        # function must hand out a tensor of its own, never the persistent view)
        return ex.x_slab.clone() if ctx.needs_input_grad[0] else ex.x_slab.detach()

    @staticmethod
    def backward(ctx, d_x_pad):
        ex, st = ctx.ex, ctx.state
        lib = native.lib()
        ex.out_slab.copy_(d_x_pad)
        ex.barrier.sync()          # every owner's input gradients are in place
        dx = torch.empty(st["rows"], ex.H, dtype=torch.bfloat16, device=d_x_pad.device)
        with communication_scope("expert", "backward", "combine", st["rows"] * ex.k * ex.H * 2):
            native.check(lib.tdllm_ep_combine(ptr(dx), None, ptr(st["experts"]), ptr(st["pos"]), ex.out_buf.ptr_array,
                                              None, st["rows"], ex.k, ex.H, ex.el, ex.world, stream()), "ep_combine")
        return dx, None, None, None


class _PeerCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_pad, weights, ex: PeerExpertExchange, state: dict):
        lib = native.lib()
        rows = state["rows"]
        ex.out_slab.copy_(y_pad)
        ex.barrier.sync()          # every owner's expert outputs are in place
        out = torch.empty(rows, ex.H, dtype=torch.bfloat16, device=y_pad.device)
        keep = (torch.empty(rows * ex.k, ex.H, dtype=torch.bfloat16, device=y_pad.device)
                if ctx.needs_input_grad[1] else None)
        w = weights.reshape(-1).float().contiguous()
        with communication_scope("expert", "forward", "combine", rows * ex.k * ex.H * 2):
            native.check(lib.tdllm_ep_combine(ptr(out), ptr(w), ptr(state["experts"]), ptr(state["pos"]),
                                              ex.out_buf.ptr_array, ptr(keep) if keep is not None else None, rows,
                                              ex.k, ex.H, ex.el, ex.world, stream()), "ep_combine")
        ctx.ex, ctx.state = ex, state
        ctx.save_for_backward(w, keep if keep is not None else w)
        ctx.has_keep = keep is not None
        ctx.wshape = weights.shape
        return out

    @staticmethod
    def backward(ctx, d_out):
        ex, st = ctx.ex, ctx.state
        lib = native.lib()
        w, keep = ctx.saved_tensors
        rows = st["rows"]
        d_out = d_out.contiguous()
        dw = None
        if ctx.needs_input_grad[1] and ctx.has_keep:
            dw = torch.empty(rows * ex.k, dtype=torch.float32, device=d_out.device)
            native.check(lib.tdllm_ep_weight_grad(ptr(d_out), ptr(keep), ptr(dw), rows, ex.k, ex.H, stream()),
                         "ep_weight_grad")
            dw = dw.view(ctx.wshape)
        native.check(lib.tdllm_ep_zero_pad_rows(ex.dy_buf.local, ptr(st["my_begin"]), ptr(st["my_count"]), ex.el, ex.H,
                                                stream()), "ep_zero_pad_rows")
        with communication_scope("expert", "backward", "dispatch", rows * ex.k * ex.H * 2):
            native.check(lib.tdllm_ep_dispatch(ptr(d_out), ptr(st["experts"]), ptr(w), None, None, ptr(st["pos"]), None,
                                               ex.dy_buf.ptr_array, rows, ex.k, ex.H, ex.el, ex.cap, ex.world, stream()),
                         "ep_dispatch")
        ex.barrier.sync()          # every source's output gradients are in this rank's slab
        return ex.dy_slab.detach(), dw, None, None


def peer_dispatch(x, experts_flat, ex: PeerExpertExchange, state: dict):
    return _PeerDispatch.apply(x, experts_flat, ex, state)


def peer_combine(y_pad, weights, ex: PeerExpertExchange, state: dict):
    return _PeerCombine.apply(y_pad, weights, ex, state)
