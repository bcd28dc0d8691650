"""DFlash drafter attention when one model replica spans several ranks.

The anchors (drafting blocks) of a batch are divided over the ranks of the replica and, with context
parallelism, so are the context rows (the conditioned target features every draft layer projects to keys and
values): rank i keeps the chunks i and 2n-1-i of 2n balanced chunks of every sequence, which evens out the
causal visibility (an anchor sees the context before it). A draft row then needs context keys that live on
other ranks. Two exchanges give the same result:

* ``kv_pull``: every rank gathers the peers' context K|V rows per layer and attends to all of them; the backward
  pass returns dK|dV to the owners (a reduce-scatter).
* ``query_rotation``: the queries travel instead. Every rank attends its own draft rows to its draft keys and
  its own context shard, and the peers' draft rows to its context shard; the partial (out, lse) pairs go back to
  the rows' owners, which merge them with the online-softmax rule. In the backward pass (dout, out, lse) travel
  the same way, each rank runs the attention backward of the peers' rows against the MERGED (out, lse) — which
  is exact without lse gradients — keeps dK|dV of its shard and returns dQ.

Which one moves fewer bytes depends on draft rows against context rows per rank; `prefer_query_rotation` counts
both (a long context with a few hundred anchors favours the queries by orders of magnitude).

Roles of dllm_parallel/core/attention/dflash_attention.py:59-189 (choice), :192-694 (the two schedules) and
dllm_parallel/core/models/backbones/dflash/training.py:130-138 (owned anchors).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch
import torch.distributed as dist

from ..ops.attention import SEQ_STRIDE, MaskLayout, attention_reference, block_attention
from ..profiling.operator_trace import communication_scope
from .context_attention import _AllGatherRows
from .layout import clean_positions_for_rank


def prefer_query_rotation(*, draft_rows: int, context_rows_per_rank: int, ranks: int, q_heads: int, kv_heads: int,
                          head_dim: int, elt: int = 2) -> bool:
    """True when rotating the queries moves fewer bytes per layer than gathering the context K|V.
    K|V: the shard is gathered in the forward pass, gathered again for the recomputation-free backward (it is
    kept, so once) and its gradient returned: 2 transfers of K and V. Queries: q out and (out, lse) back in the
    forward pass; q, dout, out, lse out and dQ back in the backward pass."""
    if ranks <= 1:
        return False
    peers = ranks - 1
    kv = 2 * peers * context_rows_per_rank * 2 * kv_heads * head_dim * elt
    row = q_heads * head_dim * elt
    lse = q_heads * 4
    queries = peers * draft_rows * ((row + row + lse) + (3 * row + lse + row))
    return queries < kv


def select_anchors(ob, index: torch.Tensor):
    """The DFlashBatch restricted to the anchors `index` (same for every sequence)."""
    b, A = ob.anchor_positions.shape
    bs = ob.draft_input_ids.shape[1] // A
    pick = lambda t: t.index_select(1, index)
    flat = lambda t: t.reshape(b, A, bs).index_select(1, index).reshape(b, -1).contiguous()
    return replace(ob, anchor_positions=pick(ob.anchor_positions), anchor_valid=pick(ob.anchor_valid),
                   block_positions=pick(ob.block_positions), teacher_source_positions=pick(ob.teacher_source_positions),
                   target_token_positions=pick(ob.target_token_positions), draft_input_ids=flat(ob.draft_input_ids),
                   supervised_mask=flat(ob.supervised_mask), position_weights=flat(ob.position_weights),
                   document_starts=pick(ob.document_starts), context_stops=pick(ob.context_stops))


def _query_codes(ob, index: torch.Tensor, block_size: int):
    """(q_lo, q_hi, q_grp) of the draft rows of the anchors `index`, packed sequence-major."""
    b, A = ob.anchor_positions.shape
    dev = ob.anchor_positions.device
    seq = torch.arange(b, device=dev)[:, None]
    grp = (seq * A + index[None, :])
    lo = seq * SEQ_STRIDE + ob.document_starts.index_select(1, index).long()
    hi = seq * SEQ_STRIDE + ob.context_stops.index_select(1, index).long()
    rep = lambda t: t[:, :, None].expand(b, index.numel(), block_size).reshape(-1).to(torch.int32)
    return rep(lo), rep(hi), rep(-(grp + 1))


@dataclass
class DraftAttentionPlan:
    """Masks of one micro-batch. Keys of `local`: [own draft rows ; own context shard]; of `pulled`: [own draft
    rows ; every rank's context shard in rank order]; `peers`: the other ranks' draft rows (rank order, this rank
    left out) against the own context shard."""

    mode: str
    draft_rows: int
    local: MaskLayout
    pulled: MaskLayout | None
    peers: MaskLayout | None
    counts: list


class DFlashContextParallel:
    def __init__(self, group, *, context_sharded: bool, mode: str = "auto", anchors_sharded: bool = True):
        """anchors_sharded=False (context parallelism without block parallelism): every rank of the replica keeps all
        anchors and only the context rows are divided; the ranks then pull the other shards' K|V, compute the same
        draft rows, and the loss of each is divided by the summed weights of all of them, so that the summed
        gradients are those of one rank."""
        self.group = group
        self.n = dist.get_world_size(group)
        self.me = dist.get_rank(group)
        self.context_sharded = bool(context_sharded) and self.n > 1
        self.anchors_sharded = bool(anchors_sharded)
        if mode not in ("auto", "kv_pull", "query_rotation"):
            raise ValueError("kernel.dflash_context_exchange must be auto, kv_pull or query_rotation")
        self.mode = mode
        self.last_mode = None

    # --------------------------------------------------------------- ownership
    def anchor_index(self, anchors: int, rank: int | None = None, device="cpu") -> torch.Tensor:
        if not self.anchors_sharded:
            return torch.arange(anchors, device=device)
        if anchors % self.n:
            raise ValueError(f"objective.max_anchors ({anchors}) must divide by the {self.n} ranks of a replica")
        return torch.arange(self.me if rank is None else rank, anchors, self.n, device=device)

    def context_positions(self, seq_len: int, rank: int | None = None, device="cpu") -> torch.Tensor:
        if not self.context_sharded:
            return torch.arange(seq_len, device=device)
        return clean_positions_for_rank(seq_len, self.n, self.me if rank is None else rank, "dual_chunk", 1, device)

    def context_rows(self, batch: int, seq_len: int, device) -> torch.Tensor:
        """Rows of a [batch * seq_len, ...] tensor that form this rank's context shard."""
        pos = self.context_positions(seq_len, device=device)
        return (torch.arange(batch, device=device)[:, None] * seq_len + pos[None, :]).reshape(-1)

    # -------------------------------------------------------------------- plan
    def plan(self, ob, block_size: int, seq_len: int, *, q_heads: int, kv_heads: int, head_dim: int) -> DraftAttentionPlan:
        b, A = ob.anchor_positions.shape
        dev = ob.anchor_positions.device
        mine = self.anchor_index(A, device=dev)
        q_lo, q_hi, q_grp = _query_codes(ob, mine, block_size)
        seq = torch.arange(b, device=dev)[:, None]
        code = lambda pos: (seq * SEQ_STRIDE + pos[None, :]).reshape(-1).to(torch.int32)
        own_ctx = code(self.context_positions(seq_len, device=dev))
        local = MaskLayout(q_lo, q_hi, q_grp, torch.cat([q_grp, own_ctx]).contiguous())
        nd = int(q_lo.numel())
        if not self.context_sharded:
            self.last_mode = "local"
            return DraftAttentionPlan("local", nd, local, None, None, [])
        shard = [code(self.context_positions(seq_len, r, dev)) for r in range(self.n)]
        counts = [int(s.numel()) for s in shard]
        mode = self.mode
        if not self.anchors_sharded:
            if mode == "query_rotation":
                raise ValueError("kernel.dflash_context_exchange=query_rotation moves the queries of the ranks' own "
                                 "anchors; without block parallelism every rank has all anchors: use kv_pull or auto")
            mode = "kv_pull"
        if mode == "auto":
            mode = ("query_rotation" if prefer_query_rotation(
                draft_rows=nd, context_rows_per_rank=max(counts), ranks=self.n, q_heads=q_heads, kv_heads=kv_heads,
                head_dim=head_dim) else "kv_pull")
        self.last_mode = mode
        if mode == "kv_pull":
            pulled = MaskLayout(q_lo, q_hi, q_grp, torch.cat([q_grp] + shard).contiguous())
            return DraftAttentionPlan(mode, nd, local, pulled, None, counts)
        others = [_query_codes(ob, self.anchor_index(A, r, dev), block_size) for r in range(self.n) if r != self.me]
        cat = lambda i: torch.cat([o[i] for o in others]).contiguous()
        peers = MaskLayout(cat(0), cat(1), cat(2), own_ctx.contiguous())
        return DraftAttentionPlan(mode, nd, local, None, peers, counts)

    # ----------------------------------------------------------------- attend
    def attend(self, plan: DraftAttentionPlan, q: torch.Tensor, kv: torch.Tensor, kv_heads: int) -> torch.Tensor:
        """q [draft rows, Hq, D]; kv [draft rows + own context rows, 2 * Hkv * D] (K | V)."""
        D = q.shape[-1]
        kd = kv_heads * D
        views = lambda t: (t[:, :kd].view(t.shape[0], kv_heads, D), t[:, kd:].view(t.shape[0], kv_heads, D))
        if plan.mode == "local":
            return block_attention(q, *views(kv), plan.local)
        nd = plan.draft_rows
        if plan.mode == "kv_pull":
            ctx_all = _AllGatherRows.apply(kv[nd:].contiguous(), self.group, plan.counts)
            return block_attention(q, *views(torch.cat([kv[:nd], ctx_all], dim=0)), plan.pulled)
        k, v = views(kv)
        if q.is_cuda and q.dtype == torch.bfloat16:
            return _QueryRotation.apply(q, k, v, self, plan)
        return self._query_rotation_composite(plan, q, k, v)

    def _exchange(self, x: torch.Tensor, label: str) -> torch.Tensor:
        """x: (n-1) equal chunks, the chunk for each other rank in rank order; returns what they sent here."""
        chunk = x.shape[0] // (self.n - 1)
        send = x.new_zeros(self.n * chunk, *x.shape[1:])
        idx = [r for r in range(self.n) if r != self.me]
        for j, r in enumerate(idx):
            send[r * chunk:(r + 1) * chunk] = x[j * chunk:(j + 1) * chunk]
        recv = torch.empty_like(send)
        with communication_scope("context_parallel", label, "all_to_all", send.numel() * send.element_size(),
                                 recv.numel() * recv.element_size()):
            dist.all_to_all_single(recv, send, group=self.group)
        return torch.cat([recv[r * chunk:(r + 1) * chunk] for r in idx])

    def _gather_peers(self, x: torch.Tensor, label: str) -> torch.Tensor:
        """Every other rank's x (equal shapes), rank order."""
        out = x.new_empty(self.n * x.shape[0], *x.shape[1:])
        with communication_scope("context_parallel", label, "all_gather", x.numel() * x.element_size(),
                                 out.numel() * out.element_size()):
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        n0 = x.shape[0]
        return torch.cat([out[r * n0:(r + 1) * n0] for r in range(self.n) if r != self.me])

    def _query_rotation_composite(self, plan, q, k, v):
        """The same schedule from differentiable pieces (fp32 reference attention, autograd through the
        collectives): the CPU path and the oracle of the kernel path."""
        nd = plan.draft_rows
        o0, l0 = attention_reference(q, k, v, plan.local)
        q_peers = _GatherPeers.apply(q, self)
        o_p, l_p = attention_reference(q_peers, k[nd:], v[nd:], plan.peers)
        packed = torch.cat([o_p.float().reshape(o_p.shape[0], -1), l_p.t()], dim=1)   # [rows, Hq*D + Hq]
        back = _ExchangeRows.apply(packed, self)
        Hq, D = q.shape[1], q.shape[2]
        outs, lses = [o0.float()], [l0.t()]
        for j in range(self.n - 1):
            part = back[j * nd:(j + 1) * nd]
            outs.append(part[:, : Hq * D].reshape(nd, Hq, D))
            lses.append(part[:, Hq * D:])
        lse = torch.stack(lses)                                      # [n, rows, Hq]
        lse = torch.where(torch.isinf(lse), torch.full_like(lse, -1.0e30), lse)
        w = torch.softmax(lse, dim=0)
        return (torch.stack(outs) * w[..., None]).sum(0).to(q.dtype)


class _GatherPeers(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp):
        ctx.cp = cp
        return cp._gather_peers(x, "forward")

    @staticmethod
    def backward(ctx, g):
        return ctx.cp._exchange(g.contiguous(), "backward").reshape(ctx.cp.n - 1, -1, *g.shape[1:]).sum(0), None


class _ExchangeRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp):
        ctx.cp = cp
        return cp._exchange(x, "forward")

    @staticmethod
    def backward(ctx, g):
        return ctx.cp._exchange(g.contiguous(), "backward"), None


class _QueryRotation(torch.autograd.Function):
    """Kernel path of the query rotation (sm_100a attention kernels; head widths 64 / 256 / 512 take the
    product-and-softmax form, which has the same (out, lse) contract)."""

    @staticmethod
    def forward(ctx, q, k, v, cp, plan):
        from ..ops.attention import attention_forward_kernels as attention_forward_native
        from ..ops.merge import MergeState

        nd, Hq, D = q.shape
        scale = 1.0 / D ** 0.5
        st = MergeState(nd, Hq, D, q.device)
        st.merge(*attention_forward_native(q, k, v, plan.local, scale))
        q_peers = cp._gather_peers(q, "forward")
        o_p, l_p = attention_forward_native(q_peers, k[nd:], v[nd:], plan.peers, scale)
        rows = q_peers.shape[0]
        o_back = cp._exchange(o_p, "forward")
        l_back = cp._exchange(l_p[:, :rows].t().contiguous(), "forward")           # [rows, Hq]
        for j in range(cp.n - 1):
            st.merge(o_back[j * nd:(j + 1) * nd], l_back[j * nd:(j + 1) * nd].t().contiguous())
        out, lse = st.finalize(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse, q_peers)
        ctx.cp, ctx.plan = cp, plan
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.attention import attention_backward_kernels as attention_backward_native

        q, k, v, out, lse, q_peers = ctx.saved_tensors
        cp, plan = ctx.cp, ctx.plan
        nd, Hq, D = q.shape
        scale = 1.0 / D ** 0.5
        dout = dout.contiguous()
        dq, dk, dv = attention_backward_native(q, k, v, out, dout, lse, plan.local, scale)
        do_p = cp._gather_peers(dout, "backward")
        o_p = cp._gather_peers(out, "backward")
        l_p = cp._gather_peers(lse[:, :nd].t().contiguous(), "backward").t().contiguous()    # [Hq, rows]
        dq_p, dk_c, dv_c = attention_backward_native(q_peers, k[nd:], v[nd:], o_p, do_p, l_p, plan.peers, scale)
        dk[nd:] += dk_c
        dv[nd:] += dv_c
        back = cp._exchange(dq_p.float(), "backward").reshape(cp.n - 1, nd, Hq, D).sum(0)
        return (dq.float() + back).to(q.dtype), dk, dv, None, None
