"""LoRA adapters on the decoder's projections.

`apply_lora(model, rank, alpha, targets)` freezes the base parameters, creates one low-rank pair
(A [r, in], B [out, r]; B starts at zero) for every targeted projection — roles `attention`
(w_qkv, w_o), `mlp` (w_gate_up, w_down) and `experts` (stacked expert weights) — in a flat
adapter buffer of its own, and hooks the layers: y = x·Wᵀ + (alpha/r)·(x·Aᵀ)·Bᵀ. Only the adapter
buffer is optimised and checkpointed (`adapter_model_only`); `merge_lora` folds the adapters into
the base weights for export. Under tensor parallelism the adapter of a column-parallel projection
shards B with the weight and the adapter of a row-parallel projection shards A; the low-rank
product of a row-parallel adapter is all-reduced with the main output.

Counterparts: dllm_parallel/core/adapters/lora.py:26-130 (LoRALinear), :133-317 (sequence-parallel
variant), :320-450 (grouped expert LoRA), :453-543 (apply_lora).
"""
from __future__ import annotations

import torch

from ..models.dense import FlatParams
from ..ops.gemm import linear

# `attention` also names the mixer projections of the hybrid family's layers (fused input projection and
# output projection of a linear-attention layer, output gate of a gated softmax-attention layer);
# a layer only gets adapters for the projections it has
ROLE_TARGETS = {"attention": ("w_qkv", "w_o", "w_in", "w_out", "w_attn_gate"), "mlp": ("w_gate_up", "w_down"),
                "experts": ()}


class LoRAState:
    def __init__(self, flat: FlatParams, scale: float, dropout: float):
        self.flat, self.scale, self.dropout = flat, scale, dropout

    def pair(self, layer_idx: int, name: str):
        a = self.flat.params.get(f"layers.{layer_idx}.{name}.lora_A")
        if a is None:
            return None
        return a, self.flat.params[f"layers.{layer_idx}.{name}.lora_B"]


def lora_delta(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scale: float, dropout: float = 0.0,
               token_mask: torch.Tensor | None = None) -> torch.Tensor:
    if dropout > 0 and torch.is_grad_enabled():
        x = torch.nn.functional.dropout(x, dropout)
    d = linear(linear(x, a), b) * scale
    if token_mask is not None:
        d = d * token_mask[:, None].to(d.dtype)
    return d


def apply_lora(model, *, rank: int, alpha: float | None = None, dropout: float = 0.0,
               targets=("attention", "mlp"), seed: int = 0) -> LoRAState:
    if rank <= 0:
        raise ValueError("LoRA rank must be positive")
    bad = sorted(set(targets) - set(ROLE_TARGETS))
    if bad:
        raise ValueError(f"unknown LoRA target roles {bad}; known: {sorted(ROLE_TARGETS)}")
    names = [n for role in targets for n in ROLE_TARGETS[role]]
    r8 = (rank + 7) // 8 * 8            # GEMM operands need 16-byte rows; extra rows stay zero
    specs = []
    for i, layer in enumerate(model.layers):
        for n in names:
            w = getattr(layer, n, None)
            if w is None:
                continue
            out_f, in_f = w.shape
            specs += [(f"layers.{i}.{n}.lora_A", (r8, in_f), True), (f"layers.{i}.{n}.lora_B", (out_f, r8), True)]
    if not specs:
        raise ValueError("no projection matches the requested LoRA targets")
    base = model.flat
    flat = FlatParams(specs, base.data.dtype, base.data.device)
    gen = torch.Generator(device=base.data.device)
    gen.manual_seed(seed + 4242)
    with torch.no_grad():
        for name, p in flat.params.items():
            if name.endswith("lora_A"):
                p.zero_()
                p[:rank].copy_((torch.randn((rank, p.shape[1]), device=p.device, generator=gen)
                                * (1.0 / rank ** 0.5)).to(p.dtype))
            else:
                p.zero_()
    for p in base.params.values():
        p.requires_grad_(False)
    state = LoRAState(flat, (alpha if alpha is not None else float(rank)) / rank, dropout)
    for layer in model.layers:
        layer.lora = state
    model.lora = state
    return state


@torch.no_grad()
def merge_lora(model) -> None:
    """W += scale · B·A for every adapted projection (after which the adapters can be dropped)."""
    st = getattr(model, "lora", None)
    if st is None:
        return
    for i, layer in enumerate(model.layers):
        for n in (n for names in ROLE_TARGETS.values() for n in names):
            pair = st.pair(i, n)
            if pair is None:
                continue
            a, b = pair
            w = getattr(layer, n)
            w.add_((b.float() @ a.float() * st.scale).to(w.dtype))
