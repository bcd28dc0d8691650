"""First-party block-diffusion decoder (Qwen3-style dense transformer) over packed rows.

A rank processes rows `[noisy rows of its blocks ; its clean rows]` (see `parallel.layout`).
Each layer is RMSNorm → fused QKV GEMM → per-head q/k RMSNorm + RoPE → block-diffusion
attention → O GEMM → (residual add + RMSNorm fused) → gate/up GEMM with SwiGLU → down GEMM,
built from this package's own ops so that on a B200 every step is an sm_100a kernel. All
parameters are views of one flat buffer and gradients land in one flat gradient buffer
(`FlatParams`), which is what the sharded optimizer and its collectives operate on.

The reference wraps a Hugging Face decoder instead
(`NemotronLabsDiffusionPackedBlockDiffusionModel`, dllm_parallel/core/models/backbones/nemotron/model.py:532-878,
layer body :2946-3211, loss :2046-2151); the generic causal-LM family reuses that wrapper
(dllm_parallel/core/models/backbones/causal_lm/executor.py:76-113).
"""
from __future__ import annotations

import math
from typing import Callable

import torch
import torch.nn as nn

from ..ops.attention import MaskLayout, packed_block_attention
from ..ops.embedding import embedding
from ..ops.gemm import linear, linear_residual, linear_swiglu, row_parallel_linear_residual
from ..ops.linear_ce import linear_cross_entropy
from ..ops.norm import rmsnorm
from ..ops.rope import qk_norm_rope, rope_inv_freq
from ..parallel.tensor_parallel import (TPContext, gather_rows_replicated_grad,
                                        sp_column_linear, sp_row_linear_residual, take_rows_sequence_parallel,
                                        vocab_parallel_embedding, vocab_parallel_linear_cross_entropy)
from .activation_store import ActivationStore, checkpointed_layer
from .config import ModelConfig

ALIGN = 128  # elements; keeps every parameter 256-byte aligned inside the flat buffer


class FlatParams:
    """One flat parameter buffer and one flat gradient buffer; parameters are views.

    Decayed parameters (matrices) come first, then the non-decayed ones (norm weights), so the
    optimizer handles weight decay with two contiguous ranges. `zero_grad()` only clears the
    "already written" flags: the first gradient write of a step overwrites its slice.
    """

    def __init__(self, specs: list[tuple[str, tuple[int, ...], bool]], dtype, device,
                 grad_dtype=None, allocate_grad: bool = True):
        specs = sorted(specs, key=lambda s: (not s[2],))  # stable: decay first
        offs, total = {}, 0
        for name, shape, decay in specs:
            n = math.prod(shape)
            offs[name] = (total, n, shape, decay)
            total += (n + ALIGN - 1) // ALIGN * ALIGN
        self.numel = total
        self.decay_numel = 0
        for name, (o, n, shape, decay) in offs.items():
            if decay:
                self.decay_numel = max(self.decay_numel, (o + n + ALIGN - 1) // ALIGN * ALIGN)
        self.data = torch.zeros(total, dtype=dtype, device=device)
        self.grad = torch.zeros(total if allocate_grad else 0, dtype=grad_dtype or dtype, device=device)
        self.offsets = offs
        self.params: dict[str, nn.Parameter] = {}
        for name, (o, n, shape, decay) in offs.items():
            p = nn.Parameter(self.data[o:o + n].view(shape), requires_grad=allocate_grad)
            p.main_grad = self.grad[o:o + n].view(shape) if allocate_grad else None
            p.grad_acc = False
            p.flat_offset = o
            p.decay = decay
            self.params[name] = p

    def zero_grad(self) -> None:
        for p in self.params.values():
            p.grad_acc = False
            p.grad = None
            if hasattr(p, "expert_written"):
                p.expert_written = set()

    def collect_grads(self) -> None:
        """Folds `.grad` tensors produced by plain autograd into the flat buffer and zeroes the
        slices of parameters that received no gradient at all this step."""
        for p in self.params.values():
            if hasattr(p, "expert_written"):
                # stacked expert weights: slices of experts that saw no token keep stale values
                for e in range(p.shape[0]):
                    if e not in p.expert_written:
                        p.main_grad[e].zero_()
                p.grad_acc = True
            if p.grad is not None:
                if p.grad_acc:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                p.grad_acc = True
                p.grad = None
            elif not p.grad_acc:
                p.main_grad.zero_()


def local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    """Per-rank shapes under tensor parallelism: heads and FFN width are divided by `tp`."""
    if tp == 1:
        return cfg
    from dataclasses import replace

    if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp or cfg.intermediate_size % tp or cfg.vocab_size % tp:
        raise ValueError(f"heads ({cfg.num_attention_heads}/{cfg.num_key_value_heads}), FFN width "
                         f"({cfg.intermediate_size}) and vocabulary ({cfg.vocab_size}) must divide by "
                         f"tensor_parallel_size {tp}")
    return replace(cfg, num_attention_heads=cfg.num_attention_heads // tp,
                   num_key_value_heads=cfg.num_key_value_heads // tp, intermediate_size=cfg.intermediate_size // tp)


def _layer_specs(cfg: ModelConfig, i: int):
    """cfg: per-rank (local) shapes."""
    h, p = cfg.hidden_size, f"layers.{i}."
    out = [(p + "input_norm", (h,), False), (p + "w_qkv", (cfg.qkv_dim, h), True),
           (p + "w_o", (h, cfg.q_dim), True), (p + "post_norm", (h,), False),
           (p + "w_gate_up", (2 * cfg.intermediate_size, h), True),
           (p + "w_down", (h, cfg.intermediate_size), True)]
    if cfg.qk_norm:
        out += [(p + "q_norm", (cfg.head_dim,), False), (p + "k_norm", (cfg.head_dim,), False)]
    return out


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, tp=None):
        super().__init__()
        self.cfg, self.idx, self.tp = cfg, idx, tp
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        self.input_norm, self.w_qkv, self.w_o = g("input_norm"), g("w_qkv"), g("w_o")
        self.post_norm, self.w_gate_up, self.w_down = g("post_norm"), g("w_gate_up"), g("w_down")
        self.q_norm = g("q_norm") if cfg.qk_norm else None
        self.k_norm = g("k_norm") if cfg.qk_norm else None
        if tp is not None and tp.size > 1:
            # replicated weights whose gradient a rank computes from its own heads / rows only
            for p in (self.q_norm, self.k_norm):
                if p is not None:
                    p.tp_partial = True
            if tp.sequence_parallel:
                self.input_norm.tp_partial = True
                self.post_norm.tp_partial = True

    def forward(self, h, positions, inv_freq, attend: Callable):
        """h: residual stream [rows, H] -> residual stream. Both residual adds happen in the
        epilogues of the O and down projections."""
        cfg, tp = self.cfg, self.tp
        tpg = tp.group if tp is not None and tp.size > 1 else None
        if getattr(self, "lora", None) is not None:
            return self._forward_lora(h, positions, inv_freq, attend)
        if tp is not None and tp.sequence_parallel:
            return self._forward_sequence_parallel(h, positions, inv_freq, attend)
        return self.mlp_half(self.attention_half(h, positions, inv_freq, attend))

    def attention_half(self, h, positions, inv_freq, attend: Callable):
        """Residual stream after the attention sub-layer (plain projections: no adapters, no sequence parallelism)."""
        cfg, tp = self.cfg, self.tp
        tpg = tp.group if tp is not None and tp.size > 1 else None
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = linear(y, self.w_qkv, tp) if tpg is not None else linear(y, self.w_qkv)
        qkv = qk_norm_rope(qkv, positions, inv_freq, self.q_norm, self.k_norm, cfg.num_attention_heads,
                           cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        a = attend(qkv, self.idx)          # [rows, Hq_local·D]
        return row_parallel_linear_residual(a, self.w_o, h, tp)

    def mlp_half(self, h):
        """Residual stream after the feed-forward sub-layer."""
        cfg, tp = self.cfg, self.tp
        tpg = tp.group if tp is not None and tp.size > 1 else None
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        chunk = int(getattr(self, "mlp_token_chunk", 0) or 0)
        if chunk > 0 and tpg is None and h.shape[0] > chunk:
            # kernel.mlp_token_chunk_size: the feed-forward runs over row chunks, so its [rows, 2·I] intermediate
            # never exists for more than `chunk` rows at a time
            outs = [linear_residual(linear_swiglu(y2[r: r + chunk], self.w_gate_up), self.w_down, h[r: r + chunk])
                    for r in range(0, h.shape[0], chunk)]
            return torch.cat(outs, dim=0)
        act = linear_swiglu(y2, self.w_gate_up, tp) if tpg is not None else linear_swiglu(y2, self.w_gate_up)
        return row_parallel_linear_residual(act, self.w_down, h, tp, last=True)

    def _forward_sequence_parallel(self, h, positions, inv_freq, attend):
        """h: this rank's rows of the residual stream. Norms run on local rows; the column-parallel projections
        gather the rows on their way in, the row-parallel ones scatter the sum on their way out."""
        cfg, tp = self.cfg, self.tp
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = sp_column_linear(y, self.w_qkv, tp)
        qkv = qk_norm_rope(qkv, positions, inv_freq, self.q_norm, self.k_norm, cfg.num_attention_heads,
                           cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        a = attend(qkv, self.idx)
        h = sp_row_linear_residual(a, self.w_o, h, tp)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        act = sp_column_linear(y2, self.w_gate_up, tp, swiglu=True)
        return sp_row_linear_residual(act, self.w_down, h, tp, last=True)

    def _forward_lora(self, h, positions, inv_freq, attend):
        """Same layer with low-rank updates on the adapted projections. Under tensor parallelism the low-rank
        product follows the projection: a column-parallel adapter multiplies the replicated x·Aᵀ by its B shard
        (gathered rows under sequence parallelism), a row-parallel adapter sums its x_local·A_localᵀ over the
        ranks (a [rows, r] all-reduce, or reduce-scatter of rows) and applies the replicated B."""
        from ..adapters.lora import adapted_column_linear, adapted_row_linear
        from ..ops.activation import swiglu

        cfg = self.cfg
        column = lambda x, name: adapted_column_linear(self, x, name)
        row = lambda x, name, res, last=False: adapted_row_linear(self, x, name, res, last)
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(column(y, "w_qkv"), positions, inv_freq, self.q_norm, self.k_norm, cfg.num_attention_heads,
                           cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        h = row(attend(qkv, self.idx), "w_o", h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        return row(swiglu(column(y2, "w_gate_up")), "w_down", h, last=True)


class LocalAttention:
    """Keys are the rank's own rows (single rank, or pure data parallelism)."""

    def __init__(self, cfg: ModelConfig, mask: MaskLayout, store=None, window_mask: MaskLayout | None = None):
        self.cfg, self.mask, self.store, self.window_mask = cfg, mask, store, window_mask

    def __call__(self, qkv, layer_idx):
        c = self.cfg
        mask = self.mask
        if self.window_mask is not None and c.layer_window(layer_idx) is not None:
            mask = self.window_mask         # sliding-window layer
        return packed_block_attention(qkv, c.num_attention_heads, c.num_key_value_heads, c.head_dim, mask,
                                      store=self.store, key=layer_idx)


class BlockDiffusionTransformer(nn.Module):
    checkpoint_scope = "full"     # "mlp" (training.activation_checkpointing_scope): recompute the feed-forward half only

    def __init__(self, cfg: ModelConfig, *, dtype=torch.bfloat16, device="cpu", grad_dtype=None,
                 activation_checkpointing: bool = True, activation_offload: bool = False, seed: int = 0,
                 init_std: float = 0.02, frozen: bool = False, tp: TPContext | None = None):
        super().__init__()
        self.cfg = cfg                      # global architecture
        self.tp = tp if tp is not None and tp.size > 1 else None
        tps = self.tp.size if self.tp is not None else 1
        self.lcfg = local_config(cfg, tps)  # per-rank shapes
        self.activation_checkpointing = activation_checkpointing
        if self.tp is not None:
            # gathered inputs may stay in the rotating peer-memory buffers until a checkpointed layer's backward
            self.tp.sp_saved_in_place = bool(activation_checkpointing)
        self.store = ActivationStore(torch.device(device), offload=activation_offload)
        h = cfg.hidden_size
        specs = [("embed", (cfg.vocab_size // tps, h), True), ("final_norm", (h,), False)]
        if not cfg.tie_word_embeddings:
            specs.append(("lm_head", (cfg.vocab_size // tps, h), True))
        for i in range(cfg.num_layers):
            specs += _layer_specs(self.lcfg, i)
        self.flat = FlatParams(specs, dtype, device, grad_dtype, allocate_grad=not frozen)
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "_"), p)
        self.embed = self.flat.params["embed"]
        self.final_norm = self.flat.params["final_norm"]
        self.lm_head = self.flat.params.get("lm_head", self.embed)
        self.layers = nn.ModuleList(DecoderLayer(self.lcfg, i, self.flat, self.tp) for i in range(cfg.num_layers))
        self.register_buffer("inv_freq", rope_inv_freq(cfg.head_dim, cfg.rope_theta, device, cfg.rotary_dim), persistent=False)
        self.sharded = None      # parallel.fsdp.ShardedParameters when the parameters are sharded
        self.reset_parameters(seed, init_std)

    def attach_parameter_sharding(self, sharded) -> None:
        """From now on a layer's parameters exist at full size only while the layer runs: `sharded.pre_layer(i)`
        materialises them, the checkpointed backward hands the gradients back (`activation_store`)."""
        if not self.activation_checkpointing or self.checkpoint_scope != "full":
            raise ValueError("parameter sharding needs training.activation_checkpointing over whole layers (gradients "
                             "leave a layer when its checkpointed backward ends)")
        self.sharded = sharded
        for layer in self.layers:
            layer.sharded = sharded

    @torch.no_grad()
    def reset_parameters(self, seed: int, std: float) -> None:
        """Normal(0, std) matrices, unit norm weights. Every parameter has its own seed derived from
        its name and the full (unsharded) tensor is generated before this rank's slice is taken, so
        a tensor-parallel model starts from exactly the weights of the single-rank model."""
        import zlib

        dev = self.flat.data.device
        gen = torch.Generator(device=dev)
        tp = getattr(self, "tp", None)
        cfg = self.cfg
        for name, p in self.flat.params.items():
            if not p.decay:
                p.fill_(1.0)
                continue
            gen.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
            if tp is None:
                p.copy_((torch.randn(p.shape, device=dev, generator=gen) * std).to(p.dtype))
                continue
            leaf = name.split(".")[-1]
            D, Hq, Hkv, t = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, tp.size
            if leaf in ("embed", "lm_head", "w_gate_up"):
                full = torch.randn((p.shape[0] * t, p.shape[1]), device=dev, generator=gen)
                shard = tp.shard(full, 0)
            elif leaf in ("w_o", "w_down"):
                full = torch.randn((p.shape[0], p.shape[1] * t), device=dev, generator=gen)
                shard = tp.shard(full, 1)
            elif leaf == "w_qkv":
                full = torch.randn(((Hq + 2 * Hkv) * D, p.shape[1]), device=dev, generator=gen)
                q, k, v = full[: Hq * D], full[Hq * D:(Hq + Hkv) * D], full[(Hq + Hkv) * D:]
                shard = torch.cat([tp.shard(q, 0), tp.shard(k, 0), tp.shard(v, 0)], dim=0)
            else:
                full = torch.randn(p.shape, device=dev, generator=gen)
                shard = full
            p.copy_((shard * std).to(p.dtype))

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, attend: Callable,
                soft_embeddings: torch.Tensor | None = None, soft_rows: torch.Tensor | None = None) -> torch.Tensor:
        """tokens, positions: [rows]; returns final-norm hidden states [rows, H].
        `soft_embeddings` [n, H] (detached predictions of an earlier pass) are added to the input
        embeddings of the rows `soft_rows` [n] (self-conditioning)."""
        if self.tp is not None:
            h = vocab_parallel_embedding(tokens, self.embed, self.tp, self.cfg.vocab_size)
        else:
            h = embedding(tokens, self.embed)
        if soft_embeddings is not None and soft_rows is not None and soft_rows.numel() > 0:
            h = h.index_add(0, soft_rows, soft_embeddings.to(h.dtype))
        positions = positions.to(torch.int32)
        sp = self.tp is not None and self.tp.sequence_parallel
        if sp:
            if h.shape[0] % self.tp.size:
                raise ValueError(f"sequence parallelism needs the {h.shape[0]} packed rows to divide by "
                                 f"tensor_parallel_size {self.tp.size}")
            h = take_rows_sequence_parallel(h, self.tp)
        if torch.is_grad_enabled() and not h.requires_grad:
            h = h.detach().requires_grad_(True)   # frozen embedding (adapters): keep the checkpoint chain alive
        for i, layer in enumerate(self.layers):
            if getattr(self, "sharded", None) is not None:
                self.sharded.pre_layer(i)
            if self.activation_checkpointing and torch.is_grad_enabled():
                if self.checkpoint_scope == "mlp":
                    # only the feed-forward half is recomputed: the attention half keeps its graph (its activations
                    # stay on the device), the residual stream between the halves is what the checkpoint stores
                    h = layer.attention_half(h, positions, self.inv_freq, attend)
                    h = checkpointed_layer(layer.mlp_half, h, self.store, i)
                else:
                    h = checkpointed_layer(layer, h, self.store, i, positions, self.inv_freq, attend)
            else:
                h = layer(h, positions, self.inv_freq, attend)
        if sp:
            h = gather_rows_replicated_grad(h, self.tp)
        y, _ = rmsnorm(h, self.final_norm, self.cfg.rms_norm_eps)
        return y

    def loss(self, hidden_rows: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor | None,
             exclude_mask_token: bool):
        """Σ weighted CE over rows with label >= 0 (rows are already compacted to supervised ones)."""
        ex = self.cfg.mask_token_id if exclude_mask_token else -1
        if self.tp is not None:
            return vocab_parallel_linear_cross_entropy(hidden_rows, self.lm_head, labels, weights, self.tp,
                                                       self.cfg.vocab_size, exclude_index=ex)
        return linear_cross_entropy(hidden_rows, self.lm_head, labels, weights, exclude_index=ex)


def compact_supervised_rows(hidden: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor | None):
    """Keeps only rows with a label (masked positions): the LM head runs on those alone
    (dllm_parallel/core/models/backbones/nemotron/model.py:4234)."""
    idx = (labels >= 0).nonzero(as_tuple=True)[0]
    h = hidden.index_select(0, idx)
    return h, labels.index_select(0, idx), (None if weights is None else weights.index_select(0, idx)), idx
