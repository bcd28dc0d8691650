"""Context-sharded block parallel (CSBP) attention.

A rank holds `[noisy rows of its blocks ; its clean shard]`. Queries are all of its rows; keys are
its own noisy rows plus the clean rows of EVERY rank of its context-parallel group. Only clean
K/V cross GPUs in the forward pass and only clean dK/dV in the backward pass:

  collective transport : all-gather clean K|V  → one attention call → reduce-scatter clean dK|dV
  streaming transport  : one attention call per owner shard, (out, lse) merged with the
                         online-softmax merge, gradients returned to each owner
  peer_pull transport  : the gather / scatter-reduce as stand-alone peer-memory copy kernels
  fused transport      : the transfer happens INSIDE the attention kernels. Forward: extra warps of every
                         CTA pull the peers' staged clean K|V rows into local memory while the tiles of this
                         rank's own keys run; a remote tile is loaded once its rows have arrived. Backward:
                         the epilogue of a remote key tile adds its dK/dV partial sums to the owner's fp32
                         accumulator through peer memory; one barrier, then every rank casts its own rows.
                         No staging of the gathered rows, no concatenation, no reduce-scatter call.

The all-gather and reduce-scatter are autograd functions over torch.distributed (NCCL on GPUs,
gloo on CPU ranks); the peer-memory pull kernels replace them on NVSwitch machines.

Counterparts: `fused_block_context_attention_bshd` and `_CollectiveWithLocalKVAttentionBSHD`
(dllm_parallel/core/attention/context_parallel_attention.py:443-490, :2315-2691), gather/scatter
helpers (:701-817), streaming ring variant (:1434-1669).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..ops.attention import block_attention, block_diffusion_layout, split_packed_qkv
from ..profiling.operator_trace import communication_scope
from .layout import PackedLayout, clean_positions_for_rank, runtime_clean_layout


def _register_fused_signatures() -> None:
    from ..kernels import native

    V, I, LL, F = native.c_void_p, native.c_int, native.c_ll, native.c_float
    native.register_signatures({
        "tdllm_symm_signal": (I, [V, I, I, I, V]),
        "tdllm_attn_fwd_csbp": (I, [V] * 6 + [I, I, LL, I, I] + [LL] * 4 + [V] * 7 + [I, F, V, V, V, I, I, I, V, V, I, V]),
        "tdllm_attn_bwd_fused_csbp": (I, [V] * 14 + [LL, V, LL, I, I, LL, I, I] + [LL] * 8 + [V] * 7
                                      + [I, I, I, F, V, V, V, I, I, I, V]),
    })


_register_fused_signatures()


class _AllGatherRows(torch.autograd.Function):
    """[n_local, C] → [Σ n_r, C] (ranks may hold different row counts); backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, group, counts):
        ctx.group, ctx.counts = group, counts
        world = len(counts)
        rank = dist.get_rank(group)
        nmax = max(counts)
        pad = x if x.shape[0] == nmax else torch.cat([x, x.new_zeros(nmax - x.shape[0], x.shape[1])])
        out = x.new_empty(world * nmax, x.shape[1])
        with communication_scope("context_parallel", "forward", "all_gather", pad.numel() * pad.element_size(),
                                 out.numel() * out.element_size()):
            dist.all_gather_into_tensor(out, pad.contiguous(), group=group)
        ctx.rank, ctx.nmax = rank, nmax
        if all(c == nmax for c in counts):
            return out
        return torch.cat([out[r * nmax: r * nmax + c] for r, c in enumerate(counts)])

    @staticmethod
    def backward(ctx, g):
        counts, nmax, group = ctx.counts, ctx.nmax, ctx.group
        world = len(counts)
        if all(c == nmax for c in counts):
            full = g.contiguous()
        else:
            full = g.new_zeros(world * nmax, g.shape[1])
            off = 0
            for r, c in enumerate(counts):
                full[r * nmax: r * nmax + c] = g[off: off + c]
                off += c
        out = g.new_empty(nmax, g.shape[1])
        with communication_scope("context_parallel", "backward", "reduce_scatter", full.numel() * full.element_size(),
                                 out.numel() * out.element_size()):
            if g.is_cuda:
                dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group)
            else:  # gloo: all-reduce then slice
                dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
                out = full[ctx.rank * nmax: (ctx.rank + 1) * nmax]
        return out[: counts[ctx.rank]], None, None


class WindowedExchangePlan:
    """Which clean rows a sliding-window layer moves between the members of a context group.

    A query row sees the clean positions [stop - window, stop) of its sequence, so a rank needs only the union of
    those intervals over its rows; the plan intersects every member's need with every member's ownership, which
    gives the variable split sizes of ONE all-to-all in the forward pass and of its reverse in the backward
    pass. Each member publishes its need as a per-position flag vector at set-up (an all-gather of seq_len
    bytes), so clean-replica sharing and any block schedule are covered without recomputing other ranks'
    layouts. Role of windowed_clean_exchange_plan, dllm_parallel/core/attention/layout.py:322-426."""

    def __init__(self, layout: PackedLayout, window: int, seq_len: int, batch: int, kpos1: list, group, me: int):
        dev = layout.positions.device
        self.group = group
        stop = torch.cat([(layout.noisy_pos // layout.block_size) * layout.block_size,
                          layout.clean_pos + 1 if layout.clean_causal
                          else (layout.clean_pos // layout.block_size + 1) * layout.block_size]).unique()
        delta = torch.zeros(seq_len + 1, dtype=torch.long, device=dev)          # interval union by prefix sums
        delta.index_add_(0, (stop - window).clamp_min(0), torch.ones_like(stop))
        delta.index_add_(0, stop.clamp_max(seq_len), -torch.ones_like(stop))
        need = (delta.cumsum(0)[:seq_len] > 0).to(torch.uint8)
        needs = [torch.empty_like(need) for _ in kpos1]
        dist.all_gather(needs, need, group=group)
        self.needs = [n.bool() for n in needs]
        mine = kpos1[me]                                   # positions of this rank's clean shard (one sequence)
        n1 = mine.numel()
        seq_off = torch.arange(batch, device=dev)
        send, self.send_counts = [], []
        for n in self.needs:                               # rows of mine that member d needs, all sequences
            idx1 = torch.nonzero(n[mine]).flatten() if n1 else mine
            send.append((seq_off[:, None] * n1 + idx1[None, :]).reshape(-1))
            self.send_counts.append(int(idx1.numel()) * batch)
        self.send_index = torch.cat(send) if send else torch.zeros(0, dtype=torch.long, device=dev)
        self.recv_counts, kp, ks = [], [], []
        for pos in kpos1:                                  # rows this rank receives from member j
            got = pos[self.needs[me][pos]] if pos.numel() else pos
            self.recv_counts.append(int(got.numel()) * batch)
            kp.append(got.repeat(batch))
            ks.append(seq_off.repeat_interleave(got.numel()))
        self.key_pos, self.key_seq = torch.cat(kp), torch.cat(ks)


class _AllToAllRows(torch.autograd.Function):
    """Sends x[plan.send_index] split by plan.send_counts, returns the received rows (member order); the backward
    pass sends the gradients back and sums them into the rows they came from."""

    @staticmethod
    def forward(ctx, x, plan):
        send = x.index_select(0, plan.send_index)
        out = x.new_empty(sum(plan.recv_counts), x.shape[1])
        with communication_scope("context_parallel", "forward", "all_to_all", send.numel() * send.element_size(),
                                 out.numel() * out.element_size()):
            dist.all_to_all_single(out, send, output_split_sizes=plan.recv_counts,
                                   input_split_sizes=plan.send_counts, group=plan.group)
        ctx.plan, ctx.rows = plan, x.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        plan = ctx.plan
        back = g.new_empty(sum(plan.send_counts), g.shape[1])
        with communication_scope("context_parallel", "backward", "all_to_all", g.numel() * g.element_size(),
                                 back.numel() * back.element_size()):
            dist.all_to_all_single(back, g.contiguous(), output_split_sizes=plan.send_counts,
                                   input_split_sizes=plan.recv_counts, group=plan.group)
        dx = torch.zeros(ctx.rows, g.shape[1], dtype=torch.float32, device=g.device)
        dx.index_add_(0, plan.send_index, back.float())
        return dx.to(g.dtype), None


class PeerKVExchange:
    """Clean K|V gather and gradient scatter-reduce through peer memory (csrc/comm.cu): two staging
    buffers alternate so that a fast rank never overwrites rows a slower peer is still pulling."""

    def __init__(self, group, device, counts: list[int], row_elems: int):
        import ctypes

        from ..kernels import native
        from .symm import SymmetricBarrier, SymmetricBuffer

        native.register_signatures({
            "tdllm_kv_gather": (native.c_int, [native.c_void_p] * 3 + [native.c_int] * 3 + [native.c_void_p,
                                                                                           native.c_int,
                                                                                           native.c_void_p]),
            "tdllm_kv_scatter_reduce": (native.c_int, [native.c_void_p] * 3 + [native.c_int] * 3
                                        + [native.c_void_p, native.c_int, native.c_void_p]),
        })
        self.native = native
        self.counts, self.row_elems = counts, row_elems
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.total = sum(counts)
        row_bytes = row_elems * 2
        self.row_bytes = row_bytes
        self.staging = [SymmetricBuffer(max(counts) * row_bytes, group, device) for _ in range(2)]
        self.partial = SymmetricBuffer(self.total * row_bytes, group, device)
        self.barrier = SymmetricBarrier(group, device)
        self.counts_arr = (ctypes.c_longlong * self.world)(*counts)
        self.flip = 0
        self.device = device

    def close(self) -> None:
        for b in (*self.staging, self.partial, self.barrier.buf):
            b.close()

    def gather(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops._util import ptr, stream

        buf = self.staging[self.flip]
        self.flip ^= 1
        n = self.counts[self.rank]
        buf.as_tensor(torch.bfloat16, n * self.row_elems).view(n, self.row_elems).copy_(x)
        out = torch.empty(self.total, self.row_elems, dtype=torch.bfloat16, device=self.device)
        e = self.barrier.reserve(1)
        with communication_scope("context_parallel", "forward", "peer_pull", (self.total - n) * self.row_bytes,
                                 self.total * self.row_bytes):
            self.native.check(self.native.lib().tdllm_kv_gather(
                buf.ptr_array, self.barrier.buf.ptr_array, self.counts_arr, self.rank, self.world, self.row_bytes,
                ptr(out), e, stream()), "kv_gather")
        return out

    def scatter_reduce(self, g: torch.Tensor) -> torch.Tensor:
        from ..ops._util import ptr, stream

        self.partial.as_tensor(torch.bfloat16, self.total * self.row_elems).view(self.total, self.row_elems).copy_(g)
        out = torch.empty(self.counts[self.rank], self.row_elems, dtype=torch.bfloat16, device=self.device)
        e = self.barrier.reserve(2)
        with communication_scope("context_parallel", "backward", "peer_pull_reduce",
                                 (self.world - 1) * self.counts[self.rank] * self.row_bytes):
            self.native.check(self.native.lib().tdllm_kv_scatter_reduce(
                self.partial.ptr_array, self.barrier.buf.ptr_array, self.counts_arr, self.rank, self.world,
                self.row_bytes, ptr(out), e, stream()), "kv_scatter_reduce")
        return out


class _PeerGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, exchange):
        ctx.exchange = exchange
        return exchange.gather(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.exchange.scatter_reduce(g.contiguous()), None


class FusedKVExchange:
    """State of the fused transport for one context-parallel group: two staging buffers for this rank's clean
    K|V rows (peers pull from them), two sets of fp32 dK/dV accumulators (peers add into them), ready flags,
    a barrier, and the per-tile arrival counters of the forward kernel. The two-deep alternation is safe
    because a rank can only be one attention call ahead of its slowest peer: finishing call n needs every
    peer's rows of call n, which a peer stages only after its own call n-1 has finished on its stream."""

    def __init__(self, group, device, counts: list[int], n_noisy: list[int], rows_local: int, kv_cols: int):
        import ctypes

        from ..kernels import native
        from .symm import SymmetricBarrier, SymmetricBuffer

        self.native, self.device, self.group = native, device, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.counts, self.kv_cols = counts, kv_cols
        self.n_rem = sum(c for r, c in enumerate(counts) if r != self.rank)
        self.nlt = (rows_local + 127) // 128
        self.nrt = (self.n_rem + 127) // 128
        self.acc_rows = max((n + c + 127) // 128 * 128 for n, c in zip(n_noisy, counts))
        self.staging = [SymmetricBuffer(max(max(counts), 1) * kv_cols * 2, group, device) for _ in range(2)]
        half = self.acc_rows * (kv_cols // 2) * 4
        self.acc_bytes = 2 * half
        self.acc = [SymmetricBuffer(self.acc_bytes, group, device) for _ in range(2)]   # zeroed at allocation
        self.acc_dk = [(ctypes.c_void_p * self.world)(*b.ptrs) for b in self.acc]
        self.acc_dv = [(ctypes.c_void_p * self.world)(*[p + half for p in b.ptrs]) for b in self.acc]
        self.ready = SymmetricBuffer(256, group, device)
        self.barrier = SymmetricBarrier(group, device)
        self.counts_arr = (ctypes.c_longlong * self.world)(*counts)
        self.row0_arr = (ctypes.c_longlong * self.world)(*n_noisy)
        self.tile_ready = torch.zeros(max(self.nrt, 1) + 1, dtype=torch.int32, device=device)
        self.counter = self.tile_ready[-1:]
        self.fwd_calls = 0
        self.bwd_calls = 0
        dist.barrier(group=group)

    def close(self) -> None:
        for b in (*self.staging, *self.acc, self.ready, self.barrier.buf):
            b.close()


class _FusedContextAttention(torch.autograd.Function):
    """Packed qkv of this rank's rows -> attention output, keys = own rows + the peers' clean rows."""

    @staticmethod
    def run_forward(qkv, cpa):
        """Stages this rank's travelling rows, signals the peers and runs the attention kernel that pulls theirs.
        Returns (out, lse, the peers' K|V rows as pulled)."""
        from ..ops._util import ptr, stream

        ex, c = cpa.exchange, cpa.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_noisy, rows = cpa.stage_row0, qkv.shape[0]     # rows from here on travel to the peers
        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        L = cpa.mask.tile_lists()
        ex.fwd_calls += 1
        n = ex.fwd_calls
        stage = ex.staging[n & 1]
        stage.as_tensor(torch.bfloat16, (rows - n_noisy) * ex.kv_cols).view(rows - n_noisy, ex.kv_cols).copy_(
            qkv[n_noisy:, Hq * D:])
        lib = ex.native.lib()
        ex.native.check(lib.tdllm_symm_signal(ex.ready.ptr_array, ex.rank, ex.world, n, stream()), "symm_signal")
        kv_rem = torch.empty(max(ex.n_rem, 1), ex.kv_cols, dtype=qkv.dtype, device=qkv.device)
        out = torch.empty(rows, Hq * D, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(Hq, L["nq_pad"], dtype=torch.float32, device=qkv.device)
        with communication_scope("context_parallel", "forward", "attention_with_peer_pull", ex.n_rem * ex.kv_cols * 2):
            ex.native.check(lib.tdllm_attn_fwd_csbp(
                ptr(q), ptr(k), ptr(v), ptr(kv_rem), ptr(out), ptr(lse), rows, rows, ex.n_rem, Hq, Hkv,
                qkv.stride(0), qkv.stride(0), qkv.stride(0), out.stride(0), ptr(L["q_lo"]), ptr(L["q_hi"]),
                ptr(L["q_grp"]), ptr(L["k_code"]), ptr(L["f_ptr"]), ptr(L["f_idx"]), ptr(L["f_order"]), L["nqt"],
                1.0 / D ** 0.5, stage.ptr_array, ex.ready.ptr_array, ex.counts_arr, ex.rank, ex.world, n,
                ptr(ex.counter), ptr(ex.tile_ready), n, stream()), "attn_fwd_csbp")
        return out, lse, kv_rem

    @staticmethod
    def forward(ctx, qkv, cpa, precomputed=None):
        """precomputed: (out, lse, pulled K|V) kept from the no-grad forward of a checkpointed layer; the
        recomputation then runs neither the kernel nor the pull again (every rank of the group skips alike)."""
        out, lse, kv_rem = precomputed if precomputed is not None else _FusedContextAttention.run_forward(qkv, cpa)
        ctx.save_for_backward(qkv, kv_rem, out, lse)
        ctx.cpa = cpa
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops._util import ptr, scratch, stream
        from ..ops.attention import backward_chunk_tiles

        qkv, kv_rem, out, lse = ctx.saved_tensors
        cpa = ctx.cpa
        ex, c = cpa.exchange, cpa.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        rows = qkv.shape[0]
        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        L = cpa.mask.tile_lists()
        W = cpa.mask.backward_work(backward_chunk_tiles())
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = split_packed_qkv(dqkv, Hq, Hkv, D)
        delta = torch.empty(2, Hq, L["nq_pad"], dtype=torch.float32, device=qkv.device)
        dq_acc = scratch(qkv.device, L["nq_pad"] * Hq * D, key="attn_bwd_acc")
        ex.bwd_calls += 1
        n = ex.bwd_calls
        cur, nxt = n & 1, (n + 1) & 1
        e = ex.barrier.reserve(1)
        with communication_scope("context_parallel", "backward", "attention_with_peer_add", ex.n_rem * ex.kv_cols * 4):
            ex.native.check(ex.native.lib().tdllm_attn_bwd_fused_csbp(
                ptr(q), ptr(k), ptr(v), ptr(kv_rem), ptr(out), ptr(dout), ptr(dq), ptr(dk), ptr(dv), ptr(lse),
                ptr(delta), ptr(dq_acc), ex.acc_dk[cur], ex.acc_dv[cur], ex.acc_rows, ex.acc[nxt].local, ex.acc_bytes,
                rows, rows, ex.n_rem, Hq, Hkv, qkv.stride(0), qkv.stride(0), qkv.stride(0), out.stride(0),
                dout.stride(0), dqkv.stride(0), dqkv.stride(0), dqkv.stride(0), ptr(L["q_lo"]), ptr(L["q_hi"]),
                ptr(L["q_grp"]), ptr(L["k_code"]), ptr(W["w_ptr"]), ptr(W["w_idx"]), ptr(W["w_order"]), W["n_work"],
                L["nqt"], L["nkt"], 1.0 / D ** 0.5, ex.counts_arr, ex.row0_arr, ex.barrier.buf.ptr_array, ex.rank,
                ex.world, e, stream()), "attn_bwd_fused_csbp")
        return dqkv, None, None


class _StreamingAttention(torch.autograd.Function):
    """Streaming transport: one owner shard of clean K|V is resident at a time. Forward: for every
    owner, broadcast its shard, run the attention kernel on it and fold (out, lse) into the
    online-softmax state. Backward: the shards are streamed again and each shard's backward runs
    against the MERGED (out, lse) — which yields the exact gradients without per-shard lse
    gradients — with clean dK|dV reduced to their owner."""

    @staticmethod
    def forward(ctx, qkv, cpa):
        from ..ops.attention import attention_forward_native
        from ..ops.merge import MergeState

        c = cpa.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_noisy = cpa.layout.n_noisy
        q, _, _ = split_packed_qkv(qkv, Hq, Hkv, D)
        rows = qkv.shape[0]
        st = MergeState(rows, Hq, D, qkv.device)
        scale = 1.0 / D ** 0.5
        for r in range(cpa.cp):
            if r > 0 and cpa.counts[r] == 0:
                continue        # a member without clean rows (its shard is another rank's)
            kv = cpa.shard_kv(qkv, r)
            k, v = cpa.kv_views(kv)
            st.merge(*attention_forward_native(q, k, v, cpa.shard_masks[r], scale))
        out, lse = st.finalize(qkv.dtype)
        ctx.save_for_backward(qkv, out, lse)
        ctx.cpa = cpa
        return out.reshape(rows, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        from ..ops.attention import attention_backward_native

        qkv, out, lse = ctx.saved_tensors
        cpa = ctx.cpa
        c = cpa.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_noisy = cpa.layout.n_noisy
        rows = qkv.shape[0]
        q, _, _ = split_packed_qkv(qkv, Hq, Hkv, D)
        dqkv = torch.zeros_like(qkv)
        dq_acc = torch.zeros(rows, Hq, D, dtype=torch.float32, device=qkv.device)
        dout3 = dout.contiguous().view(rows, Hq, D)
        scale = 1.0 / D ** 0.5
        for r in range(cpa.cp):
            if r > 0 and cpa.counts[r] == 0:
                continue
            kv = cpa.shard_kv(qkv, r)
            k, v = cpa.kv_views(kv)
            dq, dk, dv = attention_backward_native(q, k, v, out, dout3, lse, cpa.shard_masks[r], scale)
            dq_acc += dq.float()
            dkv = torch.cat([dk.reshape(k.shape[0], -1), dv.reshape(v.shape[0], -1)], dim=1)
            off = 0
            if r == 0:   # shard 0 also carries this rank's noisy keys
                dqkv[:n_noisy, Hq * D:] += dkv[:n_noisy]
                off = n_noisy
            clean = dkv[off:].contiguous()
            with communication_scope("context_parallel", "backward", "reduce", clean.numel() * clean.element_size()):
                dist.reduce(clean, dst=cpa.group_ranks[r], op=dist.ReduceOp.SUM, group=cpa.group)
            if r == cpa.cp_rank:
                dqkv[n_noisy:, Hq * D:] += clean
        dqkv[:, : Hq * D] = dq_acc.reshape(rows, Hq * D).to(dqkv.dtype)
        return dqkv, None


def fused_key_layout(layout: PackedLayout, kpos: list, kseq: list, cp: int, me: int, key_codes: list | None = None):
    """Mask of the fused transport. Key order: this rank's rows, padding up to a 128-row tile boundary, then
    the peers' exchanged rows in pull order (rank+1, rank+2, ...). kpos[r] / kseq[r]: positions and sequence
    indices of rank r's clean rows; key_codes[r] (token-split context parallelism): the key codes of ALL of
    rank r's rows, which then travel whole."""
    from ..ops.attention import INT_MIN, MaskLayout

    dev = layout.positions.device
    order = [(me + 1 + s) % cp for s in range(cp - 1)]
    local = layout.mask                                   # keys = own rows
    if key_codes is not None:
        pad = (-layout.rows) % 128
        k_code = torch.cat([local.k_code, torch.full((pad,), INT_MIN, dtype=torch.int32, device=dev)]
                           + [key_codes[r] for r in order])
        return MaskLayout(local.q_lo, local.q_hi, local.q_grp, k_code.contiguous())
    rem = block_diffusion_layout(layout.noisy_pos, layout.noisy_group, layout.clean_pos, layout.block_size,
                                 noisy_seq=layout.noisy_seq, clean_seq=layout.clean_seq,
                                 key_clean_pos=torch.cat([kpos[r] for r in order]),
                                 key_clean_seq=torch.cat([kseq[r] for r in order]),
                                 clean_causal=layout.clean_causal)
    rem_code = rem.k_code[layout.n_noisy:]
    pad = (-layout.rows) % 128
    k_code = torch.cat([local.k_code, torch.full((pad,), INT_MIN, dtype=torch.int32, device=dev), rem_code])
    return MaskLayout(local.q_lo, local.q_hi, local.q_grp, k_code.contiguous())


class ContextParallelAttention:
    def __init__(self, cfg: ModelConfig, layout: PackedLayout, runtime, spec, store=None):
        self.cfg, self.layout, self.rt = cfg, layout, runtime
        self.store = store                  # the model's ActivationStore (None: nothing is kept across layers)
        self.keep_pulled_rows = False
        self.debug_nonfinite = bool(spec.kernel.cp_bp_debug_nonfinite_attention)
        self.group = runtime.context_group
        cp = runtime.context_parallel_size
        seq_len, bs = spec.model.seq_len, spec.objective.block_size
        batch = spec.training.batch_size
        lay = runtime_clean_layout(spec.kernel.cp_bp_clean_kv_layout, runtime.block_parallel_size)
        dev = layout.positions.device
        # clean key coordinates in gather order: for each member of the exchange group that owns a clean shard,
        # for each sequence, its positions. Without clean-replica sharing the members are the CP ranks of this
        # chunk; with it they are all ranks of the context/block axis and only the first CP of them own rows.
        members = runtime.context_members()
        kpos, kseq, counts = [], [], []
        for _, shard, owns in members:
            pos = (clean_positions_for_rank(seq_len, cp, shard, lay, bs, dev) if owns
                   else torch.zeros(0, dtype=torch.long, device=dev))
            kpos.append(pos.repeat(batch))
            kseq.append(torch.arange(batch, device=dev).repeat_interleave(pos.numel()))
            counts.append(pos.numel() * batch)
        # Token-split context parallelism (no block axis): every rank computes a slice of the offsets of every
        # noisy block, so noisy K/V rows are exchanged too: a member contributes ALL its rows, noisy then clean.
        self.split = layout.noisy_offsets is not None
        self.key_codes = None
        self.stage_row0 = layout.n_noisy       # first local row that travels
        if self.split:
            from ..ops.attention import SEQ_STRIDE
            from .layout import noisy_rows, pure_context_offsets

            views = int(layout.noisy_view.max()) + 1 if layout.n_noisy else 1
            self.key_codes = []
            for i, (_, shard, _owns) in enumerate(members):
                _, _, _, grp = noisy_rows(seq_len=seq_len, block_size=bs, batch=batch, views=views,
                                          noisy_offsets=pure_context_offsets(bs, cp, shard), device=dev)
                self.key_codes.append(torch.cat([-(grp + 1), kseq[i] * SEQ_STRIDE + kpos[i]]).to(torch.int32))
                counts[i] += grp.numel()
            self.stage_row0 = 0
        self.counts = counts
        self._kpos1 = [p[: p.numel() // max(batch, 1)] for p in kpos]      # one sequence's positions per member
        self.group_ranks = [m[0] for m in members]
        # `cp` / `cp_rank` below: size of the exchange group and this rank's index in it
        cp = len(members)
        self.cp, self.cp_rank = cp, self.group_ranks.index(runtime.rank)
        # sliding-window layers exchange only the rows inside some local row's window, by one all-to-all
        self.window_plan = self.window_mask = None
        if layout.window_mask is not None and not self.split:
            self.window_plan = WindowedExchangePlan(layout, layout.window, seq_len, batch, self._kpos1, self.group,
                                                    self.cp_rank)
            self.window_mask = block_diffusion_layout(
                layout.noisy_pos, layout.noisy_group, layout.clean_pos, layout.block_size, noisy_seq=layout.noisy_seq,
                clean_seq=layout.clean_seq, key_clean_pos=self.window_plan.key_pos,
                key_clean_seq=self.window_plan.key_seq, window=layout.window, clean_causal=layout.clean_causal)
        elif layout.window_mask is not None:       # token-split: all rows travel anyway; only the mask narrows
            from ..ops.attention import MaskLayout

            w = layout.window_mask
            self.window_mask = MaskLayout(w.q_lo, w.q_hi, w.q_grp, torch.cat(self.key_codes).contiguous())
        self.transport = spec.kernel.cp_bp_clean_kv_transport
        self.shard_masks = None
        if self.split and self.transport in ("streaming", "peer_pull"):
            raise ValueError(f"kernel.cp_bp_clean_kv_transport={self.transport} exchanges clean rows only; context "
                             "parallelism without block parallelism divides the tokens inside every block and needs "
                             "'collective' or 'fused' (or kernel.pure_cp_token_split: false)")
        if self.transport == "streaming":
            if dev.type != "cuda":
                self.transport = "collective"   # the streaming path drives the sm_100a kernels directly
            else:
                self.shard_masks = []
                for r in range(cp):
                    m = block_diffusion_layout(layout.noisy_pos, layout.noisy_group, layout.clean_pos,
                                               layout.block_size, noisy_seq=layout.noisy_seq,
                                               clean_seq=layout.clean_seq, key_clean_pos=kpos[r],
                                               key_clean_seq=kseq[r], clean_causal=layout.clean_causal)
                    if r > 0:   # only the first shard carries the noisy keys
                        m.k_code = m.k_code[layout.n_noisy:].contiguous()
                    self.shard_masks.append(m)
        self.exchange = None
        if self.transport == "fused":
            if dev.type != "cuda" or cfg.head_dim != 128:
                raise ValueError("kernel.cp_bp_clean_kv_transport=fused needs CUDA devices with peer access "
                                 "and head_dim 128")
            self._init_fused(cfg, layout, kpos, kseq, counts, dev)
            return
        if self.transport == "peer_pull":
            if dev.type != "cuda":
                raise ValueError("kernel.cp_bp_clean_kv_transport=peer_pull needs CUDA devices with peer access")
            self.exchange = PeerKVExchange(self.group, dev, counts, 2 * cfg.num_key_value_heads * cfg.head_dim)
        if self.split:
            from ..ops.attention import MaskLayout

            m = layout.mask
            self.mask = MaskLayout(m.q_lo, m.q_hi, m.q_grp, torch.cat(self.key_codes).contiguous())
            return
        self.mask = block_diffusion_layout(layout.noisy_pos, layout.noisy_group, layout.clean_pos,
                                           layout.block_size, noisy_seq=layout.noisy_seq,
                                           clean_seq=layout.clean_seq, key_clean_pos=torch.cat(kpos),
                                           key_clean_seq=torch.cat(kseq), clean_causal=layout.clean_causal)

    def _init_fused(self, cfg, layout, kpos, kseq, counts, dev) -> None:
        self.mask = fused_key_layout(layout, kpos, kseq, self.cp, self.cp_rank, self.key_codes)
        n_noisy = [torch.zeros(1, dtype=torch.long, device=dev) for _ in range(self.cp)]
        dist.all_gather(n_noisy, torch.tensor([self.stage_row0], dtype=torch.long, device=dev), group=self.group)
        self.exchange = FusedKVExchange(self.group, dev, counts, [int(t) for t in n_noisy], layout.rows,
                                        2 * cfg.num_key_value_heads * cfg.head_dim)
        # keeping every layer's pulled rows for the recomputation costs n_rem * kv_cols * 2 bytes per layer:
        # done when that is a small part of what is free now (TDLLM_KEEP_PULLED_KV=0/1 overrides)
        import os

        need = self.exchange.n_rem * self.exchange.kv_cols * 2 * cfg.num_layers
        env = os.environ.get("TDLLM_KEEP_PULLED_KV")
        self.keep_pulled_rows = (env == "1") if env is not None else need < 0.25 * torch.cuda.mem_get_info(dev)[0]

    def shard_kv(self, qkv, r: int) -> torch.Tensor:
        """K|V rows attended in streaming step r: (noisy rows if r == 0) + owner r's clean rows."""
        c = self.cfg
        qd = c.num_attention_heads * c.head_dim
        n_noisy = self.layout.n_noisy
        if r == self.cp_rank:
            clean = qkv[n_noisy:, qd:].contiguous()
        else:
            clean = qkv.new_empty(self.counts[r], qkv.shape[1] - qd)
        with communication_scope("context_parallel", "forward", "broadcast", clean.numel() * clean.element_size()):
            dist.broadcast(clean, src=self.group_ranks[r], group=self.group)
        return torch.cat([qkv[:n_noisy, qd:], clean], dim=0) if r == 0 else clean

    def kv_views(self, kv):
        c = self.cfg
        n = kv.shape[0]
        kd = c.num_key_value_heads * c.head_dim
        return (kv[:, :kd].view(n, c.num_key_value_heads, c.head_dim),
                kv[:, kd:].view(n, c.num_key_value_heads, c.head_dim))

    def _fused(self, qkv, layer_idx):
        """The fused transport under activation checkpointing: the no-grad forward of a layer keeps (out, lse) and
        the pulled K|V rows, and the layer's recomputation reuses them instead of pulling and attending again."""
        store = self.store
        if store is not None and store.keep_attention and self.keep_pulled_rows:
            keys = [(layer_idx, "attn_out"), (layer_idx, "attn_lse"), (layer_idx, "attn_kv_pulled")]
            if store.recording and not torch.is_grad_enabled():
                res = _FusedContextAttention.run_forward(qkv, self)
                for k, t in zip(keys, res):
                    store.stash(k, t)
                return res[0]
            if store.replaying and store.has(keys[0]):
                return _FusedContextAttention.apply(qkv, self, tuple(store.fetch(k) for k in keys))
        return _FusedContextAttention.apply(qkv, self)

    def _windowed(self, qkv):
        """A sliding-window layer: noisy keys are local, clean keys are the rows the all-to-all brought."""
        c = self.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_noisy, rows = self.layout.n_noisy, qkv.shape[0]
        q, _, _ = split_packed_qkv(qkv, Hq, Hkv, D)
        if self.split:
            kv_all = _AllGatherRows.apply(qkv[:, Hq * D:].contiguous(), self.group, self.counts)
        else:
            got = _AllToAllRows.apply(qkv[n_noisy:, Hq * D:].contiguous(), self.window_plan)
            kv_all = torch.cat([qkv[:n_noisy, Hq * D:], got], dim=0)
        nk = kv_all.shape[0]
        out = block_attention(q, kv_all[:, : Hkv * D].view(nk, Hkv, D), kv_all[:, Hkv * D:].view(nk, Hkv, D),
                              self.window_mask)
        return out.reshape(rows, Hq * D)

    def __call__(self, qkv, layer_idx):
        out = self._attend(qkv, layer_idx)
        if self.debug_nonfinite and not bool(torch.isfinite(out).all()):
            # kernel.cp_bp_debug_nonfinite_attention: name the first layer whose attention output went bad
            raise FloatingPointError(f"non-finite attention output in layer {layer_idx} on rank {self.rt.rank} "
                                     f"(transport {self.transport})")
        return out

    def _attend(self, qkv, layer_idx):
        if self.window_mask is not None and self.cfg.layer_window(layer_idx) is not None:
            return self._windowed(qkv)
        if self.transport == "streaming":
            return _StreamingAttention.apply(qkv, self)
        if self.transport == "fused":
            return self._fused(qkv, layer_idx)
        c = self.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_noisy = self.layout.n_noisy
        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        rows = qkv.shape[0]
        if self.split:      # all K|V rows travel; the gathered rows include this rank's own
            kv_all = _AllGatherRows.apply(qkv[:, Hq * D:].contiguous(), self.group, self.counts)
            nk = kv_all.shape[0]
            out = block_attention(q, kv_all[:, : Hkv * D].view(nk, Hkv, D), kv_all[:, Hkv * D:].view(nk, Hkv, D),
                                  self.mask)
            return out.reshape(rows, Hq * D)
        kv_clean = qkv[n_noisy:, Hq * D:]                       # [n_clean, 2·Hkv·D], K | V
        if self.exchange is not None:
            gathered = _PeerGatherRows.apply(kv_clean.contiguous(), self.exchange)
        else:
            gathered = _AllGatherRows.apply(kv_clean.contiguous(), self.group, self.counts)
        kv_noisy = qkv[:n_noisy, Hq * D:]
        kv_all = torch.cat([kv_noisy, gathered], dim=0)
        nk = kv_all.shape[0]
        k_all = kv_all[:, : Hkv * D].view(nk, Hkv, D)
        v_all = kv_all[:, Hkv * D:].view(nk, Hkv, D)
        out = block_attention(q, k_all, v_all, self.mask)
        return out.reshape(rows, Hq * D)
