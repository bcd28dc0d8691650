"""DFlash2 drafter: the DFlash decoder with block-local dynamic convolutions around the attention and
MLP sub-layers, and a low-rank candidate selector on top of the frozen verifier head.

Layer: `x, k_a = conv_a.prepare(norm(h))`, attention over `[draft ; context]`, `h += conv_a.finish(o, k_a)`,
and the same around the MLP. `prepare` predicts per-token corrections of both convolutions' taps from
its input (one small projection), applies the first convolution and hands the second set of taps to
`finish`. At initialisation the base kernels are the identity tap and the projections are zero, so a
fresh DFlash2 layer computes exactly what a DFlash layer computes.

Selector: for each draft position the verifier head yields k candidate tokens with unary logits; the
selector adds a pairwise term `(P[prev] ∘ (U h)) · S[cand]` (codebooks P, S of rank r over the
verifier vocabulary) so that a serving stack can walk the k x k lattice of consecutive candidates.
`greedy_path` is that walk; training scores the candidates after the true predecessor.

Counterparts: dllm_parallel/core/models/backbones/dflash/dflash2.py:257-329 (grouped convolution), :331-387
(layer), :389-471 (selector), :473-511 (model).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.attention import MaskLayout
from ..ops.dflash2 import grouped_dynamic_conv, transform_logits
from ..ops.gemm import linear, linear_swiglu
from ..ops.norm import rmsnorm
from ..ops.rope import qk_norm_rope, rope_inv_freq
from .activation_store import ActivationStore
from .config import ModelConfig
from .dense import BlockDiffusionTransformer, FlatParams
from .dflash import DFlashDraftModel, _draft_layer_specs, draft_attention


def _conv_specs(cfg: ModelConfig, prefix: str, taps: int, groups: int):
    h = cfg.hidden_size
    rows = (2 * taps * groups + 7) // 8 * 8      # projection rows, padded for the GEMM's 16-byte rows
    return [(prefix + "_base", (2, taps, h), False), (prefix + "_proj", (rows, h), True)]


class GroupedConv:
    """Views of one convolution pair's parameters plus the two steps of the layer."""

    def __init__(self, base: torch.Tensor, proj: torch.Tensor, taps: int, groups: int, block_size: int):
        self.base, self.proj, self.taps, self.groups, self.block_size = base, proj, taps, groups, block_size

    def prepare(self, x: torch.Tensor):
        n = 2 * self.taps * self.groups
        coef = linear(x, self.proj)[:, :n].reshape(x.shape[0], 2, self.taps, self.groups)
        return grouped_dynamic_conv(x, coef[:, 0], self.base[0], self.block_size), coef[:, 1]

    def finish(self, x: torch.Tensor, coef: torch.Tensor):
        return grouped_dynamic_conv(x, coef, self.base[1], self.block_size)


class DFlash2Layer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, *, taps: int, groups: int, block_size: int):
        super().__init__()
        self.cfg, self.idx = cfg, idx
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        for n in ("input_norm", "w_q", "w_kv", "w_o", "post_norm", "w_gate_up", "w_down"):
            setattr(self, n, g(n))
        self.q_norm = g("q_norm") if cfg.qk_norm else None
        self.k_norm = g("k_norm") if cfg.qk_norm else None
        self.attention_conv = GroupedConv(g("attn_conv_base"), g("attn_conv_proj"), taps, groups, block_size)
        self.mlp_conv = GroupedConv(g("mlp_conv_base"), g("mlp_conv_proj"), taps, groups, block_size)

    def forward(self, h, ctx, pos_draft, pos_all, inv_freq, mask: MaskLayout):
        c = self.cfg
        nd = h.shape[0]
        y, _ = rmsnorm(h, self.input_norm, c.rms_norm_eps)
        y, k_attn = self.attention_conv.prepare(y)
        q = qk_norm_rope(linear(y, self.w_q), pos_draft, inv_freq, self.q_norm, self.k_norm, c.num_attention_heads, 0,
                         c.head_dim, c.rms_norm_eps)
        kv = linear(torch.cat([y, ctx], dim=0), self.w_kv)
        kv = qk_norm_rope(kv, pos_all, inv_freq, self.q_norm, self.k_norm, 0, c.num_key_value_heads, c.head_dim,
                          c.rms_norm_eps)
        a = draft_attention(q.view(nd, c.num_attention_heads, c.head_dim), kv, mask, c, self.idx)
        h = h + self.attention_conv.finish(linear(a.reshape(nd, c.q_dim), self.w_o), k_attn)
        y2, _ = rmsnorm(h, self.post_norm, c.rms_norm_eps)
        y2, k_mlp = self.mlp_conv.prepare(y2)
        return h + self.mlp_conv.finish(linear(linear_swiglu(y2, self.w_gate_up), self.w_down), k_mlp)


class CandidateSelector:
    """Low-rank predecessor-conditioned scorer over the verifier head's top-k candidates."""

    def __init__(self, predecessor: torch.Tensor, successor: torch.Tensor, projection: torch.Tensor, top_k: int):
        self.predecessor, self.successor, self.projection, self.top_k = predecessor, successor, projection, top_k

    def _context(self, hidden, predecessor_ids):
        return self.predecessor[predecessor_ids].float() * (hidden.float() @ self.projection.float().t())

    def score_candidates(self, *, candidate_ids, unary_logits, hidden_states, predecessor_ids):
        """candidate_ids, unary_logits: [n, k]; hidden_states: [n, H]; predecessor_ids: [n] -> [n, k]."""
        ctx = self._context(hidden_states, predecessor_ids)
        return unary_logits.float() + torch.einsum("nr,nkr->nk", ctx, self.successor[candidate_ids].float())

    def build_lattice(self, *, candidate_ids, unary_logits, hidden_states, anchor_token_ids):
        """[b, L, k] candidates per position -> scores [b, L, k_prev, k]: every candidate after every
        candidate of the position before (the anchor token before position 0)."""
        b, L, k = candidate_ids.shape
        prev = torch.cat([anchor_token_ids[:, None, None].expand(b, 1, k), candidate_ids[:, :-1]], dim=1)
        proj = hidden_states.float() @ self.projection.float().t()               # [b, L, r]
        ctx = self.predecessor[prev].float() * proj[:, :, None]                   # [b, L, k_prev, r]
        pair = torch.einsum("blpr,blcr->blpc", ctx, self.successor[candidate_ids].float())
        return unary_logits.float()[:, :, None] + pair

    @torch.no_grad()
    def greedy_path(self, *, candidate_ids, unary_logits, hidden_states, anchor_token_ids):
        prev, path = anchor_token_ids, []
        for t in range(candidate_ids.shape[1]):
            s = self.score_candidates(candidate_ids=candidate_ids[:, t], unary_logits=unary_logits[:, t],
                                      hidden_states=hidden_states[:, t], predecessor_ids=prev)
            prev = candidate_ids[:, t].gather(1, s.argmax(-1, keepdim=True))[:, 0]
            path.append(prev)
        return torch.stack(path, dim=1)


class DFlash2DraftModel(DFlashDraftModel):
    def __init__(self, cfg: ModelConfig, *, target_hidden: int, num_target_layers: int, block_size: int,
                 conv_kernel_size: int, conv_group_size: int, selector_rank: int, selector_top_k: int,
                 verifier_vocab_size: int, output_multiplier: float = 1.0,
                 final_logit_softcapping: float | None = None, dtype=torch.bfloat16, device="cpu", seed: int = 0,
                 init_std: float = 0.02):
        nn.Module.__init__(self)
        h = cfg.hidden_size
        if not 1 <= conv_kernel_size <= block_size:
            raise ValueError("dflash2_conv_kernel_size must lie in [1, block_size]")
        if conv_group_size < 1 or h % conv_group_size:
            raise ValueError("dflash2_conv_group_size must divide hidden_size")
        if selector_rank < 1 or selector_top_k < 1:
            raise ValueError("dflash2_selector_rank and dflash2_selector_top_k must be positive")
        self.cfg, self.block_size = cfg, block_size
        self.output_multiplier, self.final_logit_softcapping = output_multiplier, final_logit_softcapping
        self.conditioning_dim = target_hidden * num_target_layers
        groups = h // conv_group_size
        specs = [("fc", (h, self.conditioning_dim), True), ("hidden_norm", (h,), False), ("final_norm", (h,), False),
                 ("selector_predecessor", (verifier_vocab_size, selector_rank), True),
                 ("selector_successor", (verifier_vocab_size, selector_rank), True),
                 ("selector_proj", (selector_rank, h), True)]
        for i in range(cfg.num_layers):
            specs += _draft_layer_specs(cfg, i)
            specs += _conv_specs(cfg, f"layers.{i}.attn_conv", conv_kernel_size, groups)
            specs += _conv_specs(cfg, f"layers.{i}.mlp_conv", conv_kernel_size, groups)
        self.flat = FlatParams(specs, dtype, device)
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "_"), p)
        g = self.flat.params
        self.fc, self.hidden_norm, self.final_norm = g["fc"], g["hidden_norm"], g["final_norm"]
        self.layers = nn.ModuleList(DFlash2Layer(cfg, i, self.flat, taps=conv_kernel_size, groups=groups,
                                                 block_size=block_size) for i in range(cfg.num_layers))
        self.register_buffer("inv_freq", rope_inv_freq(cfg.head_dim, cfg.rope_theta, device, cfg.rotary_dim), persistent=False)
        self.store = ActivationStore(torch.device(device), offload=False)
        BlockDiffusionTransformer.reset_parameters(self, seed, init_std)
        with torch.no_grad():
            for name, p in g.items():
                if name.endswith("_conv_base"):      # identity tap
                    p.zero_()
                    p[:, 0] = 1.0
                elif name.endswith("_conv_proj") or name == "selector_successor":
                    p.zero_()
        self.candidate_selector = CandidateSelector(g["selector_predecessor"], g["selector_successor"],
                                                    g["selector_proj"], selector_top_k)
        self.selector_objective_enabled = True

    def transform_unary_logits(self, logits: torch.Tensor) -> torch.Tensor:
        return transform_logits(logits, self.output_multiplier, self.final_logit_softcapping)
