"""Hybrid block-diffusion decoder: Gated DeltaNet linear-attention layers with gated softmax-attention
layers in between (family `qwen3_8`).

Rows are packed as in the dense model, `[noisy rows of the rank's blocks ; clean rows]`.

* A **linear-attention layer** runs the clean rows of every sequence once through the causal
  convolution and the chunked gated delta rule with `chunk = block size`, which yields the recurrent
  state in front of every block. Every noisy block then runs as its own short sequence that starts
  from the state (and from the convolution history) of the clean prefix in front of it, so a noisy
  block sees exactly the clean tokens of the earlier blocks plus its own noisy tokens: the same
  visibility as block-diffusion attention. States and histories stay in the autograd graph, so the
  loss of a noisy block reaches the clean prefix. Noisy blocks are processed in groups
  (`branch_group`) because every block carries an fp32 state of Hv x Dk x Dv.
* A **full-attention layer** is the dense layer with an output gate: a second projection of the
  normed input, passed through a sigmoid, multiplies the attention output before the O projection.

Both layer kinds end in the same SwiGLU MLP as the dense model and fit the same activation
checkpointing (`models/activation_store.py`). Projections are this package's GEMMs; the recurrence is
batched matrix products (`ops/gated_delta.py`).

Reference counterparts: `Qwen38PackedBlockDiffusionModel`
(dllm_parallel/core/models/backbones/qwen3_8/model.py:423-668), full-attention features :1291-1363,
linear-attention features :1447-1521, clean pass with boundary states :1780-1869, noisy-block pass from
those states :1894-1948, convolution :2004-2082.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops.activation import swiglu  # noqa: F401  (kept for adapters that patch the MLP)
from ..ops.gated_delta import (causal_conv_reference, chunk_size_for, expand_key_heads, gated_delta_chunked,
                               gated_rmsnorm, gdn_gate, l2_normalize)
from ..ops.gemm import linear, linear_residual, linear_swiglu, row_parallel_linear_residual
from ..ops.norm import rmsnorm
from ..ops.rope import qk_norm_rope, rope_inv_freq
from .activation_store import ActivationStore
from .config import ModelConfig
from .dense import BlockDiffusionTransformer, FlatParams, _layer_specs


def linear_layer_specs(cfg: ModelConfig, i: int):
    h, p = cfg.hidden_size, f"layers.{i}."
    return [(p + "input_norm", (h,), False), (p + "w_in", (cfg.linear_in_dim, h), True),
            (p + "conv_w", (cfg.linear_conv_channels, cfg.linear_conv_kernel), True),
            (p + "conv_b", (cfg.linear_conv_channels,), False),
            (p + "A_log", (cfg.linear_num_value_heads,), False), (p + "dt_bias", (cfg.linear_num_value_heads,), False),
            (p + "gdn_norm", (cfg.linear_value_head_dim,), False),
            (p + "w_out", (h, cfg.linear_value_dim), True), (p + "post_norm", (h,), False),
            (p + "w_gate_up", (2 * cfg.intermediate_size, h), True), (p + "w_down", (h, cfg.intermediate_size), True)]


def local_hybrid_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    """Per-rank shapes under tensor parallelism: softmax heads, linear-attention key and value heads and the FFN
    width are divided by `tp` (dllm_parallel/core/models/backbones/qwen3_8/tensor_parallel.py)."""
    if tp == 1:
        return cfg
    from dataclasses import replace

    for name in ("num_attention_heads", "num_key_value_heads", "intermediate_size", "vocab_size",
                 "linear_num_key_heads", "linear_num_value_heads"):
        if getattr(cfg, name) % tp:
            raise ValueError(f"{name} ({getattr(cfg, name)}) must divide by tensor_parallel_size {tp}")
    return replace(cfg, num_attention_heads=cfg.num_attention_heads // tp,
                   num_key_value_heads=cfg.num_key_value_heads // tp, intermediate_size=cfg.intermediate_size // tp,
                   linear_num_key_heads=cfg.linear_num_key_heads // tp,
                   linear_num_value_heads=cfg.linear_num_value_heads // tp)


def fused_projection_rows(cfg: ModelConfig, index: int, parts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(rows of the fused input projection q | k | v | z | b | a, channels of the convolution) that belong to the
    key / value heads [index * H / parts, (index + 1) * H / parts) of a layer with the FULL shapes `cfg`."""
    hk, hv = cfg.linear_num_key_heads // parts, cfg.linear_num_value_heads // parts
    kd, vd = hk * cfg.linear_key_head_dim, hv * cfg.linear_value_head_dim
    K, V, HV, cc = cfg.linear_key_dim, cfg.linear_value_dim, cfg.linear_num_value_heads, cfg.linear_conv_channels
    ar = lambda lo, n: torch.arange(lo, lo + n)
    conv = torch.cat([ar(index * kd, kd), ar(K + index * kd, kd), ar(2 * K + index * vd, vd)])
    rows = torch.cat([conv, ar(cc + index * vd, vd), ar(cc + V + index * hv, hv), ar(cc + V + HV + index * hv, hv)])
    return rows, conv


def full_layer_specs(cfg: ModelConfig, i: int):
    return _layer_specs(cfg, i) + [(f"layers.{i}.w_attn_gate", (cfg.q_dim, cfg.hidden_size), True)]


class BlockRows:
    """Where the noisy blocks and the clean sequences sit in the packed rows of a rank.

    Built once per layout. `block_seq` / `block_start` give, for every noisy block in row order, the
    sequence of the micro-batch it belongs to and its first token position. With `head_parallel`
    (a `HeadParallelPlan`) the rank's clean rows may be a shard of the sequence."""

    def __init__(self, layout, seq_len: int, head_parallel=None):
        bs = layout.block_size
        self.block_size, self.seq_len = bs, seq_len
        self.n_noisy, self.n_clean = layout.n_noisy, layout.n_clean
        self.head_parallel = head_parallel
        if self.n_noisy % bs:
            raise ValueError("noisy rows must be whole blocks")
        pos = layout.noisy_pos.view(-1, bs)
        if not bool((pos - pos[:, :1] == torch.arange(bs, device=pos.device)).all()):
            raise ValueError("noisy rows of a block must be consecutive positions")
        self.block_start = pos[:, 0].contiguous()
        self.block_seq = layout.noisy_seq.view(-1, bs)[:, 0].contiguous()
        if head_parallel is not None:
            self.batch = head_parallel.batch
            return
        if self.n_clean % seq_len:
            raise ValueError("linear-attention layers need the whole clean sequence on the rank "
                             "(context sharding redistributes heads first)")
        self.batch = self.n_clean // seq_len
        want = torch.arange(seq_len, device=pos.device).repeat(self.batch)
        if not torch.equal(layout.clean_pos.to(want.dtype), want):
            raise ValueError("clean rows must be the sequences in position order")


def _adapted_linear(layer, x, name):
    """x W^T plus the layer's low-rank update of that projection, when adapters are attached."""
    out = linear(x, getattr(layer, name))
    st = getattr(layer, "lora", None)
    pair = None if st is None else st.pair(layer.idx, name)
    if pair is None:
        return out
    from ..adapters.lora import lora_delta

    return out + lora_delta(x, pair[0], pair[1], st.scale, st.dropout)


def _adapted_mlp(layer, h):
    """SwiGLU MLP with residual, unfused so that adapters can sit on both projections."""
    from ..ops.activation import swiglu as swiglu_op

    y2, _ = rmsnorm(h, layer.post_norm, layer.cfg.rms_norm_eps)
    return h + _adapted_linear(layer, swiglu_op(_adapted_linear(layer, y2, "w_gate_up")), "w_down")


class _HeadShard:
    """Sizes and parameter slices of the key/value heads [r * H / P, (r + 1) * H / P) of one layer."""

    def __init__(self, layer: "GatedDeltaLayer", index: int = 0, parts: int = 1):
        c = layer.cfg
        if c.linear_num_key_heads % parts:
            raise ValueError(f"{c.linear_num_key_heads} linear-attention key heads cannot be split over {parts} ranks")
        self.hk, self.hv = c.linear_num_key_heads // parts, c.linear_num_value_heads // parts
        self.dk, self.dv = c.linear_key_head_dim, c.linear_value_head_dim
        kd, vd = self.hk * self.dk, self.hv * self.dv
        self.kd, self.vd = kd, vd
        if parts == 1:
            self.conv_w, self.conv_b, self.A_log, self.dt_bias = layer.conv_w, layer.conv_b, layer.A_log, layer.dt_bias
            self.columns = None
            return
        K, V, HV = c.linear_key_dim, c.linear_value_dim, c.linear_num_value_heads
        dev = layer.conv_w.device
        ar = lambda lo, n: torch.arange(lo, lo + n, device=dev)
        conv_rows = torch.cat([ar(index * kd, kd), ar(K + index * kd, kd), ar(2 * K + index * vd, vd)])
        self.conv_w, self.conv_b = layer.conv_w[conv_rows], layer.conv_b[conv_rows]
        self.A_log = layer.A_log[index * self.hv:(index + 1) * self.hv]
        self.dt_bias = layer.dt_bias[index * self.hv:(index + 1) * self.hv]
        cc = c.linear_conv_channels
        # columns of the fused input projection that belong to this shard: q | k | v | z | b | a
        self.columns = torch.cat([conv_rows, ar(cc + index * vd, vd), ar(cc + V + index * self.hv, self.hv),
                                  ar(cc + V + HV + index * self.hv, self.hv)])


class HeadParallelPlan:
    """Row bookkeeping for linear-attention layers over a context-sharded group.

    Softmax attention can leave the clean rows sharded and move K/V; a recurrence cannot, it needs every
    sequence whole. So inside a linear-attention layer the ranks of the group trade their row shards
    for head shards with one all-to-all (`parallel/head_sequence.py`): afterwards every rank holds
    all rows of the group (each rank's `[noisy ; clean]` rows, in rank order) for 1/P of the heads,
    runs the recurrence there and trades back. This object knows, for that gathered row order, where
    the noisy blocks are and how to put the clean rows into sequence order.

    Reference: dllm_parallel/core/models/backbones/qwen3_8/context_parallel.py:89-143 (head <-> sequence
    all-to-all), qwen3_8/model.py:1523-1636 (clean pass under context parallelism)."""

    def __init__(self, *, group, index: int, noisy_blocks: list, clean_positions: list, batch: int, seq_len: int,
                 block_size: int, device):
        """noisy_blocks[r]: (block_seq [n_r], block_start [n_r]) of rank r's noisy blocks in row order;
        clean_positions[r]: positions [c_r] of rank r's clean rows of ONE sequence (repeated per sequence)."""
        self.group, self.index, self.parts = group, index, len(clean_positions)
        self.row_counts = [int(nb[0].numel()) * block_size + int(cp.numel()) * batch
                           for nb, cp in zip(noisy_blocks, clean_positions)]
        noisy_rows, clean_rows, clean_key, off = [], [], [], 0
        for (bseq, bstart), cpos in zip(noisy_blocks, clean_positions):
            nn_ = int(bseq.numel()) * block_size
            noisy_rows.append(torch.arange(off, off + nn_, device=device))
            c = int(cpos.numel())
            clean_rows.append(torch.arange(off + nn_, off + nn_ + c * batch, device=device))
            seq = torch.arange(batch, device=device).repeat_interleave(c)
            clean_key.append(seq * seq_len + cpos.to(device).repeat(batch))
            off += nn_ + c * batch
        self.total_rows = off
        self.noisy_rows = torch.cat(noisy_rows)
        clean_rows, clean_key = torch.cat(clean_rows), torch.cat(clean_key)
        if clean_key.numel() != batch * seq_len or torch.unique(clean_key).numel() != batch * seq_len:
            raise ValueError("the group's clean shards must cover every position of every sequence exactly once")
        self.clean_rows = clean_rows[torch.argsort(clean_key)]      # gathered row of (sequence, position)
        self.block_seq = torch.cat([nb[0].to(device) for nb in noisy_blocks])
        self.block_start = torch.cat([nb[1].to(device) for nb in noisy_blocks])
        self.batch, self.seq_len, self.block_size = batch, seq_len, block_size


class GatedDeltaLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, branch_group: int = 64, tp=None):
        """cfg: per-rank shapes. tp: tensor-parallel context (the layer then owns 1/tp of the key / value heads: fused
        input projection column-parallel, output projection row-parallel, MLP as in the dense decoder)."""
        super().__init__()
        self.cfg, self.idx, self.branch_group = cfg, idx, branch_group
        self.tp = tp if tp is not None and tp.size > 1 else None
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        for n in ("input_norm", "w_in", "conv_w", "conv_b", "A_log", "dt_bias", "gdn_norm", "w_out", "post_norm",
                  "w_gate_up", "w_down"):
            setattr(self, n, g(n))
        if self.tp is not None:
            self.gdn_norm.tp_partial = True     # replicated weight that sees this rank's heads only
            if self.tp.sequence_parallel:       # the layer norms see this rank's rows only
                self.input_norm.tp_partial = True
                self.post_norm.tp_partial = True

    # -- pieces ------------------------------------------------------------------------------
    @staticmethod
    def _split(p: torch.Tensor, sh: _HeadShard):
        cc = 2 * sh.kd + sh.vd
        return p[..., :cc], p[..., cc:cc + sh.vd], p[..., cc + sh.vd:cc + sh.vd + sh.hv], \
            p[..., cc + sh.vd + sh.hv:cc + sh.vd + 2 * sh.hv]

    def _recurrence_inputs(self, conv: torch.Tensor, b: torch.Tensor, a: torch.Tensor, sh: _HeadShard):
        """conv: [B, T, channels] after convolution and SiLU -> q, k, v, log decay, beta."""
        B, T = conv.shape[:2]
        q = l2_normalize(conv[..., :sh.kd].reshape(B, T, sh.hk, sh.dk))
        k = l2_normalize(conv[..., sh.kd:2 * sh.kd].reshape(B, T, sh.hk, sh.dk))
        v = conv[..., 2 * sh.kd:].reshape(B, T, sh.hv, sh.dv).float()
        q, k = expand_key_heads(q, sh.hv), expand_key_heads(k, sh.hv)
        return q, k, v, gdn_gate(a, sh.A_log, sh.dt_bias), torch.sigmoid(b.float())

    def _mix_heads(self, p_noisy, p_clean, block_seq, block_start, sh: _HeadShard, bs: int):
        """p_noisy: [blocks, bs, F], p_clean: [B, S, F] (features of the heads in `sh`).
        Returns (noisy features [blocks * bs, hv * Dv], clean features [B * S, hv * Dv])."""
        c = self.cfg
        B, S, W = p_clean.shape[0], p_clean.shape[1], c.linear_conv_kernel
        C = chunk_size_for(bs)
        # ---- clean rows: one causal pass per sequence, states in front of every chunk
        qkv_c, z_c, b_c, a_c = self._split(p_clean, sh)
        conv_c = causal_conv_reference(qkv_c, sh.conv_w, sh.conv_b)
        q, k, v, g, beta = self._recurrence_inputs(conv_c, b_c, a_c, sh)
        o_c, _, states = gated_delta_chunked(q, k, v, g, beta, chunk=C, return_states=True)
        out_c = gated_rmsnorm(o_c, z_c.reshape(B, S, sh.hv, sh.dv), self.gdn_norm, c.rms_norm_eps)
        # ---- noisy blocks: short sequences from the clean state and the clean convolution history
        outs = []
        nb = p_noisy.shape[0]
        if nb:
            qkv_n, z_n, b_n, a_n = self._split(p_noisy, sh)
            flat_clean = qkv_c.reshape(B * S, -1)
            flat_states = states.reshape(B * (S // C), *states.shape[2:])
            hist_off = torch.arange(-(W - 1), 0, device=p_clean.device)
            for lo in range(0, nb, self.branch_group):
                hi = min(lo + self.branch_group, nb)
                start, seq = block_start[lo:hi], block_seq[lo:hi]
                tok = start[:, None] + hist_off[None, :]                       # [n, W-1]
                hist = flat_clean.index_select(0, (seq[:, None] * S + tok.clamp_min(0)).reshape(-1))
                hist = hist.view(hi - lo, W - 1, -1) * (tok >= 0)[..., None].to(hist.dtype)
                conv_n = causal_conv_reference(qkv_n[lo:hi], sh.conv_w, sh.conv_b, history=hist)
                q, k, v, g, beta = self._recurrence_inputs(conv_n, b_n[lo:hi], a_n[lo:hi], sh)
                s0 = flat_states.index_select(0, seq * (S // C) + start // C)
                o_n, _, _ = gated_delta_chunked(q, k, v, g, beta, initial_state=s0, chunk=C)
                outs.append(gated_rmsnorm(o_n, z_n[lo:hi].reshape(hi - lo, bs, sh.hv, sh.dv), self.gdn_norm,
                                          c.rms_norm_eps).reshape((hi - lo) * bs, -1))
        noisy = torch.cat(outs, dim=0) if outs else out_c.new_zeros(0, sh.vd)
        return noisy, out_c.reshape(B * S, -1)

    def mix(self, y: torch.Tensor | None, rows: BlockRows, projected: torch.Tensor | None = None) -> torch.Tensor:
        """y: normed rows [rows, H] -> mixer features [rows, Hv * Dv] (input of the output projection). `projected`:
        the fused input projection of ALL rows when the caller computed it (sequence parallelism gathers the rows on
        the way into that projection)."""
        bs = rows.block_size
        if projected is not None:
            p, y = projected, projected        # (y is only asked for its dtype below)
        else:
            p = linear(y, self.w_in, self.tp) if self.tp is not None else _adapted_linear(self, y, "w_in")
        plan = rows.head_parallel
        if plan is None:
            sh = _HeadShard(self)
            nn_ = rows.n_noisy
            noisy, clean = self._mix_heads(p[:nn_].view(nn_ // bs, bs, -1), p[nn_:].view(rows.batch, rows.seq_len, -1),
                                           rows.block_seq, rows.block_start, sh, bs)
            return torch.cat([noisy, clean], dim=0).to(y.dtype)
        from ..parallel.head_sequence import head_to_sequence_parallel, sequence_to_head_parallel

        shards = [_HeadShard(self, r, plan.parts) for r in range(plan.parts)]
        gathered = sequence_to_head_parallel([p[:, sh.columns] for sh in shards], plan.row_counts, plan.group)
        sh = shards[plan.index]
        p_noisy = gathered.index_select(0, plan.noisy_rows).view(-1, bs, gathered.shape[1])
        p_clean = gathered.index_select(0, plan.clean_rows).view(plan.batch, plan.seq_len, -1)
        noisy, clean = self._mix_heads(p_noisy, p_clean, plan.block_seq, plan.block_start, sh, bs)
        out = noisy.new_zeros(plan.total_rows, sh.vd)
        out = out.index_copy(0, plan.noisy_rows, noisy).index_copy(0, plan.clean_rows, clean)
        return head_to_sequence_parallel(out.to(y.dtype), plan.row_counts, plan.index, plan.group)

    def forward(self, h, positions, inv_freq, attend):
        cfg = self.cfg
        rows = attend.block_rows
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        tp = self.tp
        if getattr(self, "lora", None) is not None and tp is not None:
            return self._forward_adapted_tensor_parallel(h, y, rows)
        if getattr(self, "lora", None) is not None:
            return _adapted_mlp(self, h + _adapted_linear(self, self.mix(y, rows), "w_out"))
        if tp is not None and tp.sequence_parallel:
            # h holds this rank's rows of the residual stream: the column-parallel projections gather the rows on the
            # way in (the recurrence needs whole sequences, of this rank's heads), the row-parallel ones scatter the sum
            from ..parallel.tensor_parallel import sp_column_linear, sp_row_linear_residual

            feats = self.mix(None, rows, projected=sp_column_linear(y, self.w_in, tp))
            h = sp_row_linear_residual(feats, self.w_out, h, tp)
            y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
            return sp_row_linear_residual(sp_column_linear(y2, self.w_gate_up, tp, swiglu=True), self.w_down, h, tp, last=True)
        if tp is not None:
            h = row_parallel_linear_residual(self.mix(y, rows), self.w_out, h, tp)
            y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
            return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up, tp), self.w_down, h, tp, last=True)
        h = linear_residual(self.mix(y, rows), self.w_out, h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up), self.w_down, h, None, last=True)


    def _forward_adapted_tensor_parallel(self, h, y, rows):
        """Adapters under tensor (and sequence) parallelism: column-parallel projections add the replicated x·Aᵀ times
        this rank's B, row-parallel ones sum their partial x·Aᵀ over the ranks before the replicated B."""
        from ..adapters.lora import adapted_column_linear as column, adapted_row_linear as row

        feats = self.mix(None, rows, projected=column(self, y, "w_in"))
        h = row(self, feats, "w_out", h)
        y2, _ = rmsnorm(h, self.post_norm, self.cfg.rms_norm_eps)
        return row(self, swiglu(column(self, y2, "w_gate_up")), "w_down", h, last=True)


class GatedAttentionLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, tp=None):
        super().__init__()
        self.cfg, self.idx = cfg, idx
        self.tp = tp if tp is not None and tp.size > 1 else None
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        for n in ("input_norm", "w_qkv", "w_attn_gate", "w_o", "post_norm", "w_gate_up", "w_down"):
            setattr(self, n, g(n))
        self.q_norm = g("q_norm") if cfg.qk_norm else None
        self.k_norm = g("k_norm") if cfg.qk_norm else None
        if self.tp is not None:
            for p in (self.q_norm, self.k_norm):
                if p is not None:
                    p.tp_partial = True
            if self.tp.sequence_parallel:
                self.input_norm.tp_partial = True
                self.post_norm.tp_partial = True

    def _forward_sequence_parallel(self, h, positions, inv_freq, attend):
        """h: this rank's rows. Query / key / value and gate projections gather the rows (attention runs over all rows
        of this rank's heads), the output and down projections scatter the summed rows."""
        from ..parallel.tensor_parallel import sp_column_linear, sp_row_linear_residual

        cfg, tp = self.cfg, self.tp
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(sp_column_linear(y, self.w_qkv, tp), positions, inv_freq, self.q_norm, self.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        gate = torch.sigmoid(sp_column_linear(y, self.w_attn_gate, tp).float())
        a = (attend(qkv, self.idx).float() * gate).to(h.dtype)
        h = sp_row_linear_residual(a, self.w_o, h, tp)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return sp_row_linear_residual(sp_column_linear(y2, self.w_gate_up, tp, swiglu=True), self.w_down, h, tp, last=True)

    def _forward_tensor_parallel(self, h, positions, inv_freq, attend):
        cfg, tp = self.cfg, self.tp
        if tp.sequence_parallel:
            return self._forward_sequence_parallel(h, positions, inv_freq, attend)
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(linear(y, self.w_qkv, tp), positions, inv_freq, self.q_norm, self.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        gate = torch.sigmoid(linear(y, self.w_attn_gate, tp).float())
        a = (attend(qkv, self.idx).float() * gate).to(h.dtype)
        h = row_parallel_linear_residual(a, self.w_o, h, tp)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up, tp), self.w_down, h, tp, last=True)

    def _forward_adapted_tensor_parallel(self, h, positions, inv_freq, attend):
        from ..adapters.lora import adapted_column_linear as column, adapted_row_linear as row

        cfg = self.cfg
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(column(self, y, "w_qkv"), positions, inv_freq, self.q_norm, self.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        gate = torch.sigmoid(column(self, y, "w_attn_gate").float())
        a = (attend(qkv, self.idx).float() * gate).to(h.dtype)
        h = row(self, a, "w_o", h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row(self, swiglu(column(self, y2, "w_gate_up")), "w_down", h, last=True)

    def forward(self, h, positions, inv_freq, attend):
        if self.tp is not None and getattr(self, "lora", None) is not None:
            return self._forward_adapted_tensor_parallel(h, positions, inv_freq, attend)
        if self.tp is not None:
            return self._forward_tensor_parallel(h, positions, inv_freq, attend)
        cfg = self.cfg
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(_adapted_linear(self, y, "w_qkv"), positions, inv_freq, self.q_norm, self.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        gate = torch.sigmoid(_adapted_linear(self, y, "w_attn_gate").float())
        a = (attend(qkv, self.idx).float() * gate).to(h.dtype)
        if getattr(self, "lora", None) is not None:
            return _adapted_mlp(self, h + _adapted_linear(self, a, "w_o"))
        h = linear_residual(a, self.w_o, h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up), self.w_down, h, None, last=True)


class HybridBlockDiffusionTransformer(BlockDiffusionTransformer):
    """Same interface as the dense model (`forward(tokens, positions, attend)`, `loss`, `flat`).
    `attend.block_rows` (a `BlockRows`) must describe the packed rows; `TrainingSession` sets it."""

    def __init__(self, cfg: ModelConfig, *, dtype=torch.bfloat16, device="cpu", grad_dtype=None,
                 activation_checkpointing: bool = True, activation_offload: bool = False, seed: int = 0,
                 init_std: float = 0.02, frozen: bool = False, branch_group: int = 64, tp=None):
        nn.Module.__init__(self)
        if not cfg.is_hybrid or min(cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim,
                                    cfg.linear_value_head_dim) <= 0:
            raise ValueError("a hybrid model needs full_attention_interval and the linear_* head sizes")
        if cfg.linear_num_value_heads % cfg.linear_num_key_heads:
            raise ValueError("linear_num_value_heads must be a multiple of linear_num_key_heads")
        self.tp = tp if tp is not None and tp.size > 1 else None
        tps = self.tp.size if self.tp is not None else 1
        if self.tp is not None:
            # gathered inputs may stay in the rotating peer-memory buffers until a checkpointed layer's backward
            self.tp.sp_saved_in_place = bool(activation_checkpointing)
        self.cfg, self.lcfg = cfg, local_hybrid_config(cfg, tps)
        lcfg = self.lcfg
        self.activation_checkpointing = activation_checkpointing
        self.store = ActivationStore(torch.device(device), offload=activation_offload)
        h = cfg.hidden_size
        specs = [("embed", (cfg.vocab_size // tps, h), True), ("final_norm", (h,), False)]
        if not cfg.tie_word_embeddings:
            specs.append(("lm_head", (cfg.vocab_size // tps, h), True))
        kinds = [cfg.layer_kind(i) for i in range(cfg.num_layers)]
        for i, kind in enumerate(kinds):
            specs += full_layer_specs(lcfg, i) if kind == "full_attention" else linear_layer_specs(lcfg, i)
        first_replicated = None
        if self.tp is not None:
            # the optimizer sums squared gradients of sharded parameters over the tensor-parallel group and counts
            # replicated ones once: the per-head vectors of the linear-attention layers are sharded although they are
            # not decayed, so they go in front of the replicated norm weights
            per_head = ("conv_b", "A_log", "dt_bias")
            decayed = [sp for sp in specs if sp[2]]
            nd_sharded = [sp for sp in specs if not sp[2] and sp[0].split(".")[-1] in per_head]
            nd_repl = [sp for sp in specs if not sp[2] and sp[0].split(".")[-1] not in per_head]
            specs, first_replicated = decayed + nd_sharded + nd_repl, nd_repl[0][0]
        self.flat = FlatParams(specs, dtype, device, grad_dtype, allocate_grad=not frozen)
        if first_replicated is not None:
            self.flat.tp_sharded_numel = self.flat.offsets[first_replicated][0]
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "_"), p)
        self.embed, self.final_norm = self.flat.params["embed"], self.flat.params["final_norm"]
        self.lm_head = self.flat.params.get("lm_head", self.embed)
        self.layer_kinds = tuple(kinds)
        self.layers = nn.ModuleList(
            GatedAttentionLayer(lcfg, i, self.flat, self.tp) if kind == "full_attention"
            else GatedDeltaLayer(lcfg, i, self.flat, branch_group, self.tp) for i, kind in enumerate(kinds))
        self.register_buffer("inv_freq", rope_inv_freq(cfg.head_dim, cfg.rope_theta, device, cfg.rotary_dim), persistent=False)
        self.reset_parameters(seed, init_std)

    @torch.no_grad()
    def _reset_tensor_parallel_shards(self, seed: int, std: float) -> None:
        """The family's own sharded matrices start as slices of what a single rank draws (same per-name seeds as
        `BlockDiffusionTransformer.reset_parameters`): the fused input projection by head segments, the output
        projection by value-head columns, the attention gate by query heads."""
        import zlib

        tp, cfg, dev = self.tp, self.cfg, self.flat.data.device
        gen = torch.Generator(device=dev)
        for name, p in self.flat.params.items():
            leaf = name.split(".")[-1]
            if leaf not in ("w_in", "w_out", "w_attn_gate"):
                continue
            gen.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
            if leaf == "w_in":
                full = torch.randn((cfg.linear_in_dim, p.shape[1]), device=dev, generator=gen)
                rows, _ = fused_projection_rows(cfg, tp.rank, tp.size)
                p.zero_()
                p[: rows.numel()].copy_((full[rows.to(dev)] * std).to(p.dtype))
            elif leaf == "w_out":
                full = torch.randn((p.shape[0], p.shape[1] * tp.size), device=dev, generator=gen)
                p.copy_((tp.shard(full, 1) * std).to(p.dtype))
            else:
                full = torch.randn((p.shape[0] * tp.size, p.shape[1]), device=dev, generator=gen)
                p.copy_((tp.shard(full, 0) * std).to(p.dtype))

    @torch.no_grad()
    def reset_parameters(self, seed: int, std: float) -> None:
        super().reset_parameters(seed, std)
        hv = self.cfg.linear_num_value_heads
        tp = getattr(self, "tp", None)
        if tp is not None:
            self._reset_tensor_parallel_shards(seed, std)
        lo, n_hv = (tp.rank * (hv // tp.size), hv // tp.size) if tp is not None else (0, hv)
        for name, p in self.flat.params.items():
            leaf = name.split(".")[-1]
            if leaf == "w_in":         # rows past q | k | v | z | b | a only pad the GEMM's N; nothing reads them
                c = self.lcfg
                p[c.linear_conv_channels + c.linear_value_dim + 2 * c.linear_num_value_heads:].zero_()
            elif leaf == "conv_b":
                p.zero_()
            elif leaf == "conv_w":       # starts close to "take the current token"
                p.mul_(0.0)
                p[:, -1] = 1.0
                p[:, :-1] = 1.0 / (4 * self.cfg.linear_conv_kernel)
            elif leaf == "A_log":        # decay rates exp(A_log) spread over [1, 16] (over ALL value heads)
                p.copy_(torch.log(torch.linspace(1.0, 16.0, hv, device=p.device))[lo:lo + n_hv].to(p.dtype))
            elif leaf == "dt_bias":      # softplus^-1 of time steps spread over [1e-3, 1e-1]
                dt = torch.exp(torch.linspace(math.log(1e-3), math.log(1e-1), hv, device=p.device))
                p.copy_((dt + torch.log(-torch.expm1(-dt)))[lo:lo + n_hv].to(p.dtype))
