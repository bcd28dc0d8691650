"""DFlash diffusion speculative drafter and its frozen-target conditioning.

The drafter is a small decoder whose drafting blocks attend to (a) themselves, bidirectionally,
and (b) the *target model's* view of the context: hidden states of a few evenly spaced target
layers are concatenated, projected (`fc`) and normalised (`hidden_norm`) once, and every draft
layer projects them to keys/values with its own K/V weights. Token embeddings and the output
head are the frozen target's. The loss is a soft-label distillation against the target's
next-token distribution through the frozen head (`ops.distill.frozen_linear_kl`).

`FrozenTarget` runs the target (any dense decoder of this package) causally without grad and
captures the selected hidden states — the "online" feature source; offline feature files and
synthetic features plug in through the same `TargetFeatures` container.

Counterparts: dllm_parallel/core/models/backbones/dflash/model.py:344-517 (attention), :600-698
(conditioning), :700-860 (forward), :862-956 (loss); feature capture
dllm_parallel/core/models/backbones/dflash/feature_capture.py:83-217.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops.attention import MaskLayout, block_attention, block_diffusion_layout
from ..ops.embedding import embedding
from ..ops.gemm import linear, linear_residual, linear_swiglu
from ..ops.norm import rmsnorm
from ..ops.rope import qk_norm_rope, rope_inv_freq
from .activation_store import ActivationStore
from .config import ModelConfig
from .dense import BlockDiffusionTransformer, FlatParams


@dataclass
class TargetFeatures:
    hidden: torch.Tensor        # [B*L, n_selected * target_hidden] concatenated selected layers
    final_hidden: torch.Tensor  # [B*L, target_hidden] after the target's final norm (teacher states); may live
                                # memory-mapped on the host (offline store of a long context): rows are taken there
    hidden_is_shard: bool = False   # `hidden` already holds only this rank's context rows


def causal_layout(batch: int, seq_len: int, device) -> MaskLayout:
    """Plain causal attention as a block-diffusion layout with blocks of one token."""
    pos = torch.arange(seq_len, device=device).repeat(batch)
    seq = torch.arange(batch, device=device).repeat_interleave(seq_len)
    empty = torch.zeros(0, dtype=torch.long, device=device)
    return block_diffusion_layout(empty, empty, pos, 1, clean_seq=seq)


class FrozenTarget:
    def __init__(self, cfg: ModelConfig, layer_ids: tuple[int, ...], *, dtype, device, seed: int = 1):
        self.cfg, self.layer_ids = cfg, tuple(layer_ids)
        bad = [i for i in layer_ids if not 0 <= i < cfg.num_layers]
        if bad:
            raise ValueError(f"target_layer_ids {bad} outside the target's {cfg.num_layers} layers")
        self.model = BlockDiffusionTransformer(cfg, dtype=dtype, device=device, activation_checkpointing=False,
                                               seed=seed, frozen=True)
        self._layouts: dict = {}

    @property
    def embed(self):
        return self.model.embed

    @property
    def lm_head(self):
        return self.model.lm_head

    @torch.no_grad()
    def features(self, input_ids: torch.Tensor) -> TargetFeatures:
        from .dense import LocalAttention

        b, l = input_ids.shape
        key = (b, l)
        if key not in self._layouts:
            self._layouts[key] = causal_layout(b, l, input_ids.device)
        lay = self._layouts[key]
        m = self.model
        pos = torch.arange(l, device=input_ids.device).repeat(b).to(torch.int32)
        attend = LocalAttention(self.cfg, lay)
        h = embedding(input_ids.reshape(-1), m.embed)
        taps = []
        for i, layer in enumerate(m.layers):
            h = layer(h, pos, m.inv_freq, attend)
            if i in self.layer_ids:
                taps.append(h)
        final, _ = rmsnorm(h, m.final_norm, self.cfg.rms_norm_eps)
        return TargetFeatures(torch.cat(taps, dim=-1), final)


class DraftVocabulary:
    """A drafter that predicts a subset of the verifier's vocabulary (the `t2d` / `d2t` maps of speculative-decoding
    servers): `t2d` [V] bool marks the verifier ids the drafter can emit, draft id j stands for verifier id
    j + d2t[j] (the j-th marked id). The frozen head the losses use is the verifier head's marked rows.
    Counterpart of dllm_parallel/core/models/backbones/dflash/model.py:631-692 and
    dllm_parallel/core/models/backbones/dflash/executor.py:1022-1062."""

    def __init__(self, t2d: torch.Tensor, d2t: torch.Tensor, verifier_vocab_size: int):
        t2d = t2d.to(torch.bool).reshape(-1).cpu()
        d2t = d2t.to(torch.int64).reshape(-1).cpu()
        if t2d.numel() != verifier_vocab_size:
            raise ValueError(f"t2d has {t2d.numel()} entries, the verifier's vocabulary {verifier_vocab_size}")
        self.selected = torch.nonzero(t2d).flatten()
        if self.selected.numel() != d2t.numel() or self.selected.numel() == 0:
            raise ValueError(f"t2d marks {self.selected.numel()} ids, d2t has {d2t.numel()} entries")
        if not torch.equal(d2t, self.selected - torch.arange(d2t.numel())):
            raise ValueError("d2t does not map draft ids to the marked verifier ids (draft id j -> j + d2t[j])")
        self.t2d, self.d2t = t2d, d2t
        self.size, self.verifier_vocab_size = int(d2t.numel()), int(verifier_vocab_size)

    @classmethod
    def from_ids(cls, ids, verifier_vocab_size: int) -> "DraftVocabulary":
        """From the verifier ids to keep (any order, duplicates ignored)."""
        t2d = torch.zeros(verifier_vocab_size, dtype=torch.bool)
        t2d[torch.as_tensor(ids, dtype=torch.int64)] = True
        sel = torch.nonzero(t2d).flatten()
        return cls(t2d, sel - torch.arange(sel.numel()), verifier_vocab_size)

    @classmethod
    def load(cls, path: str, verifier_vocab_size: int) -> "DraftVocabulary":
        from safetensors.torch import load_file

        vals = load_file(path, device="cpu")
        if "t2d" not in vals or "d2t" not in vals:
            raise ValueError(f"{path} must hold the tensors t2d and d2t")
        return cls(vals["t2d"], vals["d2t"], verifier_vocab_size)

    def save(self, path: str) -> str:
        from safetensors.torch import save_file

        save_file({"t2d": self.t2d.contiguous(), "d2t": self.d2t.contiguous()}, path)
        return path

    def head_rows(self, head: torch.Tensor) -> torch.Tensor:
        """The marked rows of the verifier's output head, as one contiguous frozen matrix [size, H]."""
        return head.detach().index_select(0, self.selected.to(head.device)).contiguous()

    def to_draft_ids(self, verifier_ids: torch.Tensor) -> torch.Tensor:
        """Draft id of every verifier id, -1 where the drafter cannot emit it."""
        table = getattr(self, "_table", None)
        if table is None or table.device != verifier_ids.device:
            table = torch.full((self.verifier_vocab_size,), -1, dtype=torch.int64)
            table[self.selected] = torch.arange(self.size)
            self._table = table = table.to(verifier_ids.device)
        return table[verifier_ids]


def _draft_layer_specs(cfg: ModelConfig, i: int):
    h, p = cfg.hidden_size, f"layers.{i}."
    out = [(p + "input_norm", (h,), False), (p + "w_q", (cfg.q_dim, h), True),
           (p + "w_kv", (2 * cfg.kv_dim, h), True), (p + "w_o", (h, cfg.q_dim), True),
           (p + "post_norm", (h,), False), (p + "w_gate_up", (2 * cfg.intermediate_size, h), True),
           (p + "w_down", (h, cfg.intermediate_size), True)]
    if cfg.qk_norm:
        out += [(p + "q_norm", (cfg.head_dim,), False), (p + "k_norm", (cfg.head_dim,), False)]
    return out


class DraftMasks:
    """The two visibility layouts of a drafter with sliding-window layers: `full` (a drafting block sees its document's
    context up to its anchor) and `windowed` (only the last `sliding_window - 1` context tokens before the anchor)."""

    def __init__(self, full: MaskLayout, windowed: MaskLayout | None = None):
        self.full, self.windowed = full, windowed

    def for_layer(self, cfg: ModelConfig, idx: int) -> MaskLayout:
        if self.windowed is not None and cfg.layer_window(idx) is not None:
            return self.windowed
        return self.full


def draft_attention(q, kv, mask, cfg: ModelConfig, layer_idx: int = 0):
    """q [draft rows, Hq, D]; kv [draft rows + context rows, 2 * Hkv * D] (K | V). `mask` is the MaskLayout of a
    single-rank replica (or its `DraftMasks` pair when some layers have a sliding window), or the (exchange, plan)
    pair of a replica that spans ranks (parallel/dflash_context.py), whose context rows are this rank's shard."""
    if isinstance(mask, DraftMasks):
        mask = mask.for_layer(cfg, layer_idx)
    if isinstance(mask, tuple):
        exchange, plan = mask
        return exchange.attend(plan, q, kv, cfg.num_key_value_heads)
    nk = kv.shape[0]
    k = kv[:, : cfg.kv_dim].view(nk, cfg.num_key_value_heads, cfg.head_dim)
    v = kv[:, cfg.kv_dim:].view(nk, cfg.num_key_value_heads, cfg.head_dim)
    return block_attention(q, k, v, mask)


class DFlashLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams):
        super().__init__()
        self.cfg, self.idx = cfg, idx
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        self.input_norm, self.w_q, self.w_kv, self.w_o = g("input_norm"), g("w_q"), g("w_kv"), g("w_o")
        self.post_norm, self.w_gate_up, self.w_down = g("post_norm"), g("w_gate_up"), g("w_down")
        self.q_norm = g("q_norm") if cfg.qk_norm else None
        self.k_norm = g("k_norm") if cfg.qk_norm else None

    def forward(self, h, ctx, pos_draft, pos_all, inv_freq, mask: MaskLayout):
        c = self.cfg
        nd = h.shape[0]
        y, _ = rmsnorm(h, self.input_norm, c.rms_norm_eps)
        q = linear(y, self.w_q)
        q = qk_norm_rope(q, pos_draft, inv_freq, self.q_norm, self.k_norm, c.num_attention_heads, 0, c.head_dim,
                         c.rms_norm_eps)
        kv = linear(torch.cat([y, ctx], dim=0), self.w_kv)       # keys = [draft rows ; context rows]
        kv = qk_norm_rope(kv, pos_all, inv_freq, self.q_norm, self.k_norm, 0, c.num_key_value_heads, c.head_dim,
                          c.rms_norm_eps)
        a = draft_attention(q.view(nd, c.num_attention_heads, c.head_dim), kv, mask, c, self.idx)
        h = linear_residual(a.reshape(nd, c.q_dim), self.w_o, h)
        y2, _ = rmsnorm(h, self.post_norm, c.rms_norm_eps)
        return linear_residual(linear_swiglu(y2, self.w_gate_up), self.w_down, h)


class DFlashDraftModel(nn.Module):
    def __init__(self, cfg: ModelConfig, *, target_hidden: int, num_target_layers: int, dtype=torch.bfloat16,
                 device="cpu", seed: int = 0, init_std: float = 0.02, activation_checkpointing: bool = False):
        super().__init__()
        self.cfg = cfg
        h = cfg.hidden_size
        self.conditioning_dim = target_hidden * num_target_layers
        specs = [("fc", (h, self.conditioning_dim), True), ("hidden_norm", (h,), False), ("final_norm", (h,), False)]
        for i in range(cfg.num_layers):
            specs += _draft_layer_specs(cfg, i)
        self.flat = FlatParams(specs, dtype, device)
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "_"), p)
        self.fc, self.hidden_norm = self.flat.params["fc"], self.flat.params["hidden_norm"]
        self.final_norm = self.flat.params["final_norm"]
        self.layers = nn.ModuleList(DFlashLayer(cfg, i, self.flat) for i in range(cfg.num_layers))
        self.register_buffer("inv_freq", rope_inv_freq(cfg.head_dim, cfg.rope_theta, device, cfg.rotary_dim), persistent=False)
        self.store = ActivationStore(torch.device(device), offload=False)
        BlockDiffusionTransformer.reset_parameters(self, seed, init_std)

    def condition(self, target_hidden_concat: torch.Tensor) -> torch.Tensor:
        """concat(selected target layers) -> fc -> RMSNorm: the context the draft layers attend to."""
        ctx = linear(target_hidden_concat, self.fc)
        out, _ = rmsnorm(ctx, self.hidden_norm, self.cfg.rms_norm_eps)
        return out

    def forward(self, draft_embeds, ctx_features, pos_draft, pos_ctx, mask: MaskLayout):
        ctx = self.condition(ctx_features)
        pos_d = pos_draft.to(torch.int32)
        pos_all = torch.cat([pos_d, pos_ctx.to(torch.int32)])
        h = draft_embeds
        for layer in self.layers:
            h = layer(h, ctx, pos_d, pos_all, self.inv_freq, mask)
        y, _ = rmsnorm(h, self.final_norm, self.cfg.rms_norm_eps)
        return y


def dflash_mask_layout(batch_obj, seq_len: int, block_size: int, seq_stride: int = 1 << 24, *, window: int | None = None,
                       context_rows: torch.Tensor | None = None) -> MaskLayout:
    """Draft rows (queries and first keys) then the context keys: all B·L rows, or the rows `context_rows` (flat
    indices b·L + position) when the context was compacted. `window`: a drafting block sees only the last
    `window - 1` context tokens before its anchor (the anchor's own token is the window's newest entry:
    dllm_parallel/core/attention/dflash_attention.py:853-875); its own block stays fully visible."""
    a = batch_obj.anchor_positions
    b, A = a.shape
    dev = a.device
    seq = torch.arange(b, device=dev)[:, None].expand(b, A)
    grp = (seq * A + torch.arange(A, device=dev)[None, :])
    start, stop = batch_obj.document_starts.long(), batch_obj.context_stops.long()
    if window is not None:
        start = torch.maximum(start, stop - max(1, int(window) - 1))
    lo = seq * seq_stride + start
    hi = seq * seq_stride + stop
    rep = lambda t: t[:, :, None].expand(b, A, block_size).reshape(-1)
    q_lo, q_hi, q_grp = rep(lo), rep(hi), -(rep(grp) + 1)
    ctx_code = (torch.arange(b, device=dev)[:, None] * seq_stride + torch.arange(seq_len, device=dev)[None, :]).reshape(-1)
    if context_rows is not None:
        ctx_code = ctx_code.index_select(0, context_rows)
    i32 = torch.int32
    return MaskLayout(q_lo.to(i32), q_hi.to(i32), q_grp.to(i32), torch.cat([q_grp, ctx_code]).to(i32))


def window_context_rows(batch_obj, seq_len: int, window: int, min_rows: int = 128) -> torch.Tensor:
    """Flat indices (b·L + position, ascending) of the context rows that some valid anchor's window reaches. When every
    layer of the drafter has the window, all other rows have no influence and no gradient (the conditioning
    projection, norms, rotary embedding and K|V projection act row by row) and are left out of the step
    (dllm_parallel/core/models/backbones/dflash/model.py:1098-1215). At least `min_rows` rows are kept, so no
    projection runs on a degenerate row count; extra rows are invisible to every query."""
    stop = batch_obj.context_stops.long()
    start = torch.maximum(batch_obj.document_starts.long(), stop - max(1, int(window) - 1))
    b, A = stop.shape
    # coverage count by difference array: +1 at start, -1 at stop (invalid anchors have start == stop == seq_len)
    diff = torch.zeros(b, seq_len + 1, dtype=torch.int32, device=stop.device)
    one = torch.ones_like(start, dtype=torch.int32)
    diff.scatter_add_(1, start.clamp_max(seq_len), one)
    diff.scatter_add_(1, stop.clamp_max(seq_len), -one)
    keep = diff[:, :seq_len].cumsum(1) > 0
    short = min(min_rows, b * seq_len) - int(keep.sum())
    if short > 0:
        spare = (~keep).reshape(-1).nonzero(as_tuple=True)[0][:short]
        keep.view(-1)[spare] = True
    return keep.reshape(-1).nonzero(as_tuple=True)[0]
