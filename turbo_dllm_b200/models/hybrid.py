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


def full_layer_specs(cfg: ModelConfig, i: int):
    return _layer_specs(cfg, i) + [(f"layers.{i}.w_attn_gate", (cfg.q_dim, cfg.hidden_size), True)]


class BlockRows:
    """Where the noisy blocks and the clean sequences sit in the packed rows of a rank.

    Built once per layout. `block_seq` / `block_start` give, for every noisy block in row order, the
    sequence of the micro-batch it belongs to and its first token position."""

    def __init__(self, layout, seq_len: int):
        bs = layout.block_size
        self.block_size, self.seq_len = bs, seq_len
        self.n_noisy, self.n_clean = layout.n_noisy, layout.n_clean
        if self.n_noisy % bs:
            raise ValueError("noisy rows must be whole blocks")
        pos = layout.noisy_pos.view(-1, bs)
        if not bool((pos - pos[:, :1] == torch.arange(bs, device=pos.device)).all()):
            raise ValueError("noisy rows of a block must be consecutive positions")
        self.block_start = pos[:, 0].contiguous()
        self.block_seq = layout.noisy_seq.view(-1, bs)[:, 0].contiguous()
        if self.n_clean % seq_len:
            raise ValueError("linear-attention layers need the whole clean sequence on the rank "
                             "(context sharding redistributes heads first)")
        self.batch = self.n_clean // seq_len
        want = torch.arange(seq_len, device=pos.device).repeat(self.batch)
        if not torch.equal(layout.clean_pos.to(want.dtype), want):
            raise ValueError("clean rows must be the sequences in position order")


class GatedDeltaLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, branch_group: int = 64):
        super().__init__()
        self.cfg, self.idx, self.branch_group = cfg, idx, branch_group
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        for n in ("input_norm", "w_in", "conv_w", "conv_b", "A_log", "dt_bias", "gdn_norm", "w_out", "post_norm",
                  "w_gate_up", "w_down"):
            setattr(self, n, g(n))

    # -- pieces ------------------------------------------------------------------------------
    def _split(self, p: torch.Tensor):
        c = self.cfg
        cc, vd, hv = c.linear_conv_channels, c.linear_value_dim, c.linear_num_value_heads
        return p[..., :cc], p[..., cc:cc + vd], p[..., cc + vd:cc + vd + hv], p[..., cc + vd + hv:cc + vd + 2 * hv]

    def _recurrence_inputs(self, conv: torch.Tensor, b: torch.Tensor, a: torch.Tensor):
        """conv: [B, T, channels] after convolution and SiLU -> q, k, v, log decay, beta."""
        c = self.cfg
        B, T = conv.shape[:2]
        kd = c.linear_key_dim
        q = l2_normalize(conv[..., :kd].reshape(B, T, c.linear_num_key_heads, c.linear_key_head_dim))
        k = l2_normalize(conv[..., kd:2 * kd].reshape(B, T, c.linear_num_key_heads, c.linear_key_head_dim))
        v = conv[..., 2 * kd:].reshape(B, T, c.linear_num_value_heads, c.linear_value_head_dim).float()
        q, k = expand_key_heads(q, c.linear_num_value_heads), expand_key_heads(k, c.linear_num_value_heads)
        return q, k, v, gdn_gate(a, self.A_log, self.dt_bias), torch.sigmoid(b.float())

    def mix(self, y: torch.Tensor, rows: BlockRows) -> torch.Tensor:
        """y: normed rows [rows, H] -> mixer features [rows, Hv * Dv] (input of the output projection)."""
        c = self.cfg
        bs, S, B, W = rows.block_size, rows.seq_len, rows.batch, c.linear_conv_kernel
        C = chunk_size_for(bs)
        p = linear(y, self.w_in)
        nn_ = rows.n_noisy
        # ---- clean rows: one causal pass per sequence, states in front of every chunk
        qkv_c, z_c, b_c, a_c = self._split(p[nn_:].view(B, S, -1))
        conv_c = causal_conv_reference(qkv_c, self.conv_w, self.conv_b)
        q, k, v, g, beta = self._recurrence_inputs(conv_c, b_c, a_c)
        o_c, _, states = gated_delta_chunked(q, k, v, g, beta, chunk=C, return_states=True)
        out_c = gated_rmsnorm(o_c, z_c.reshape(B, S, c.linear_num_value_heads, -1), self.gdn_norm, c.rms_norm_eps)
        outs = []
        # ---- noisy blocks: short sequences from the clean state and the clean convolution history
        nb = nn_ // bs
        if nb:
            qkv_n, z_n, b_n, a_n = self._split(p[:nn_].view(nb, bs, -1))
            flat_clean = qkv_c.reshape(B * S, -1)
            flat_states = states.reshape(B * (S // C), *states.shape[2:])
            hist_off = torch.arange(-(W - 1), 0, device=y.device)
            for lo in range(0, nb, self.branch_group):
                hi = min(lo + self.branch_group, nb)
                start, seq = rows.block_start[lo:hi], rows.block_seq[lo:hi]
                tok = start[:, None] + hist_off[None, :]                       # [n, W-1]
                hist = flat_clean.index_select(0, (seq[:, None] * S + tok.clamp_min(0)).reshape(-1))
                hist = hist.view(hi - lo, W - 1, -1) * (tok >= 0)[..., None].to(hist.dtype)
                conv_n = causal_conv_reference(qkv_n[lo:hi], self.conv_w, self.conv_b, history=hist)
                q, k, v, g, beta = self._recurrence_inputs(conv_n, b_n[lo:hi], a_n[lo:hi])
                s0 = flat_states.index_select(0, seq * (S // C) + start // C)
                o_n, _, _ = gated_delta_chunked(q, k, v, g, beta, initial_state=s0, chunk=C)
                outs.append(gated_rmsnorm(o_n, z_n[lo:hi].reshape(hi - lo, bs, c.linear_num_value_heads, -1),
                                          self.gdn_norm, c.rms_norm_eps).reshape((hi - lo) * bs, -1))
        outs.append(out_c.reshape(B * S, -1))
        return torch.cat(outs, dim=0).to(y.dtype)

    def forward(self, h, positions, inv_freq, attend):
        cfg = self.cfg
        rows = attend.block_rows
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        h = linear_residual(self.mix(y, rows), self.w_out, h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up), self.w_down, h, None, last=True)


class GatedAttentionLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams):
        super().__init__()
        self.cfg, self.idx = cfg, idx
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        for n in ("input_norm", "w_qkv", "w_attn_gate", "w_o", "post_norm", "w_gate_up", "w_down"):
            setattr(self, n, g(n))
        self.q_norm = g("q_norm") if cfg.qk_norm else None
        self.k_norm = g("k_norm") if cfg.qk_norm else None

    def forward(self, h, positions, inv_freq, attend):
        cfg = self.cfg
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(linear(y, self.w_qkv), positions, inv_freq, self.q_norm, self.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        gate = torch.sigmoid(linear(y, self.w_attn_gate).float())
        a = (attend(qkv, self.idx).float() * gate).to(h.dtype)
        h = linear_residual(a, self.w_o, h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up), self.w_down, h, None, last=True)


class HybridBlockDiffusionTransformer(BlockDiffusionTransformer):
    """Same interface as the dense model (`forward(tokens, positions, attend)`, `loss`, `flat`).
    `attend.block_rows` (a `BlockRows`) must describe the packed rows; `TrainingSession` sets it."""

    def __init__(self, cfg: ModelConfig, *, dtype=torch.bfloat16, device="cpu", grad_dtype=None,
                 activation_checkpointing: bool = True, activation_offload: bool = False, seed: int = 0,
                 init_std: float = 0.02, frozen: bool = False, branch_group: int = 64):
        nn.Module.__init__(self)
        if not cfg.is_hybrid or min(cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim,
                                    cfg.linear_value_head_dim) <= 0:
            raise ValueError("a hybrid model needs full_attention_interval and the linear_* head sizes")
        if cfg.linear_num_value_heads % cfg.linear_num_key_heads:
            raise ValueError("linear_num_value_heads must be a multiple of linear_num_key_heads")
        self.cfg, self.lcfg, self.tp = cfg, cfg, None
        self.activation_checkpointing = activation_checkpointing
        self.store = ActivationStore(torch.device(device), offload=activation_offload)
        h = cfg.hidden_size
        specs = [("embed", (cfg.vocab_size, h), True), ("final_norm", (h,), False)]
        if not cfg.tie_word_embeddings:
            specs.append(("lm_head", (cfg.vocab_size, h), True))
        kinds = [cfg.layer_kind(i) for i in range(cfg.num_layers)]
        for i, kind in enumerate(kinds):
            specs += full_layer_specs(cfg, i) if kind == "full_attention" else linear_layer_specs(cfg, i)
        self.flat = FlatParams(specs, dtype, device, grad_dtype, allocate_grad=not frozen)
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "_"), p)
        self.embed, self.final_norm = self.flat.params["embed"], self.flat.params["final_norm"]
        self.lm_head = self.flat.params.get("lm_head", self.embed)
        self.layer_kinds = tuple(kinds)
        self.layers = nn.ModuleList(
            GatedAttentionLayer(cfg, i, self.flat) if kind == "full_attention"
            else GatedDeltaLayer(cfg, i, self.flat, branch_group) for i, kind in enumerate(kinds))
        self.register_buffer("inv_freq", rope_inv_freq(cfg.head_dim, cfg.rope_theta, device), persistent=False)
        self.reset_parameters(seed, init_std)

    @torch.no_grad()
    def reset_parameters(self, seed: int, std: float) -> None:
        super().reset_parameters(seed, std)
        hv = self.cfg.linear_num_value_heads
        for name, p in self.flat.params.items():
            leaf = name.split(".")[-1]
            if leaf == "conv_b":
                p.zero_()
            elif leaf == "conv_w":       # starts close to "take the current token"
                p.mul_(0.0)
                p[:, -1] = 1.0
                p[:, :-1] = 1.0 / (4 * self.cfg.linear_conv_kernel)
            elif leaf == "A_log":        # decay rates exp(A_log) spread over [1, 16]
                p.copy_(torch.log(torch.linspace(1.0, 16.0, hv, device=p.device)).to(p.dtype))
            elif leaf == "dt_bias":      # softplus^-1 of time steps spread over [1e-3, 1e-1]
                dt = torch.exp(torch.linspace(math.log(1e-3), math.log(1e-1), hv, device=p.device))
                p.copy_((dt + torch.log(-torch.expm1(-dt))).to(p.dtype))
