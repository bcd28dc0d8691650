"""Context-sharded block parallel (CSBP) attention.

A rank holds `[noisy rows of its blocks ; its clean shard]`. Queries are all of its rows; keys are
its own noisy rows plus the clean rows of EVERY rank of its context-parallel group. Only clean
K/V cross GPUs in the forward pass and only clean dK/dV in the backward pass:

  collective transport : all-gather clean K|V  → one attention call → reduce-scatter clean dK|dV
  streaming transport  : one attention call per owner shard, (out, lse) merged with the
                         online-softmax merge, gradients returned to each owner

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
from ..ops.attention import attention_reference, block_attention, block_diffusion_layout, split_packed_qkv
from .layout import PackedLayout, clean_positions_for_rank, runtime_clean_layout


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
        if g.is_cuda:
            dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group)
        else:  # gloo: all-reduce then slice
            dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
            out = full[ctx.rank * nmax: (ctx.rank + 1) * nmax]
        return out[: counts[ctx.rank]], None, None


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
        self.native.check(self.native.lib().tdllm_kv_gather(
            buf.ptr_array, self.barrier.buf.ptr_array, self.counts_arr, self.rank, self.world, self.row_bytes,
            ptr(out), e, stream()), "kv_gather")
        return out

    def scatter_reduce(self, g: torch.Tensor) -> torch.Tensor:
        from ..ops._util import ptr, stream

        self.partial.as_tensor(torch.bfloat16, self.total * self.row_elems).view(self.total, self.row_elems).copy_(g)
        out = torch.empty(self.counts[self.rank], self.row_elems, dtype=torch.bfloat16, device=self.device)
        e = self.barrier.reserve(2)
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
            dist.reduce(clean, dst=cpa.group_ranks[r], op=dist.ReduceOp.SUM, group=cpa.group)
            if r == cpa.cp_rank:
                dqkv[n_noisy:, Hq * D:] += clean
        dqkv[:, : Hq * D] = dq_acc.reshape(rows, Hq * D).to(dqkv.dtype)
        return dqkv, None


class ContextParallelAttention:
    def __init__(self, cfg: ModelConfig, layout: PackedLayout, runtime, spec):
        self.cfg, self.layout, self.rt = cfg, layout, runtime
        self.group = runtime.context_group
        cp = runtime.context_parallel_size
        seq_len, bs = spec.model.seq_len, spec.objective.block_size
        batch = spec.training.batch_size
        lay = runtime_clean_layout(spec.kernel.cp_bp_clean_kv_layout, runtime.block_parallel_size)
        dev = layout.positions.device
        # clean key coordinates in gather order: for each CP rank, for each sequence, its positions
        kpos, kseq, counts = [], [], []
        for r in range(cp):
            pos = clean_positions_for_rank(seq_len, cp, r, lay, bs, dev)
            kpos.append(pos.repeat(batch))
            kseq.append(torch.arange(batch, device=dev).repeat_interleave(pos.numel()))
            counts.append(pos.numel() * batch)
        self.counts = counts
        self.cp, self.cp_rank = cp, runtime.context_parallel_rank
        self.group_ranks = runtime.groups.ranks["context_block_parallel"]
        self.transport = spec.kernel.cp_bp_clean_kv_transport
        self.shard_masks = None
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
        if self.transport == "peer_pull":
            if dev.type != "cuda":
                raise ValueError("kernel.cp_bp_clean_kv_transport=peer_pull needs CUDA devices with peer access")
            self.exchange = PeerKVExchange(self.group, dev, counts, 2 * cfg.num_key_value_heads * cfg.head_dim)
        self.mask = block_diffusion_layout(layout.noisy_pos, layout.noisy_group, layout.clean_pos,
                                           layout.block_size, noisy_seq=layout.noisy_seq,
                                           clean_seq=layout.clean_seq, key_clean_pos=torch.cat(kpos),
                                           key_clean_seq=torch.cat(kseq), clean_causal=layout.clean_causal)

    def shard_kv(self, qkv, r: int) -> torch.Tensor:
        """K|V rows attended in streaming step r: (noisy rows if r == 0) + owner r's clean rows."""
        c = self.cfg
        qd = c.num_attention_heads * c.head_dim
        n_noisy = self.layout.n_noisy
        if r == self.cp_rank:
            clean = qkv[n_noisy:, qd:].contiguous()
        else:
            clean = qkv.new_empty(self.counts[r], qkv.shape[1] - qd)
        dist.broadcast(clean, src=self.group_ranks[r], group=self.group)
        return torch.cat([qkv[:n_noisy, qd:], clean], dim=0) if r == 0 else clean

    def kv_views(self, kv):
        c = self.cfg
        n = kv.shape[0]
        kd = c.num_key_value_heads * c.head_dim
        return (kv[:, :kd].view(n, c.num_key_value_heads, c.head_dim),
                kv[:, kd:].view(n, c.num_key_value_heads, c.head_dim))

    def __call__(self, qkv, layer_idx):
        if self.transport == "streaming":
            return _StreamingAttention.apply(qkv, self)
        c = self.cfg
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        n_noisy = self.layout.n_noisy
        q, k, v = split_packed_qkv(qkv, Hq, Hkv, D)
        rows = qkv.shape[0]
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
