"""LoRA adapters on the decoder's projections.

`apply_lora(model, rank, alpha, targets)` freezes the base parameters, creates one low-rank pair
(A [r, in], B [out, r]; B starts at zero) for every targeted projection — roles `attention`
(w_qkv, w_o), `mlp` (w_gate_up, w_down) and `experts` (stacked expert weights) — in a flat
adapter buffer of its own, and hooks the layers: y = x·Wᵀ + (alpha/r)·(x·Aᵀ)·Bᵀ. Only the adapter
buffer is optimised and checkpointed (`adapter_model_only`); `merge_lora` folds the adapters into
the base weights for export. Under tensor parallelism the adapter of a column-parallel projection
shards B with the weight and the adapter of a row-parallel projection shards A (the other halves are
replicated); the [rows, r] product of a row-parallel adapter is summed over the ranks (all-reduce, or
reduce-scatter of rows under sequence parallelism) before the replicated B applies, and under
sequence parallelism the replicated halves see this rank's rows only, so their gradients are summed
over the group with the other partial gradients. Role `experts` adds one pair per local expert on the
stacked gate/up and down weights of a mixture-of-experts layer, in an adapter buffer of its own that
is sharded with the experts; those layers then run their experts one by one (not through the grouped
GEMM or the peer-memory exchange).

Counterparts: dllm_parallel/core/adapters/lora.py:26-130 (LoRALinear), :133-317 (sequence-parallel
variant), :320-450 (grouped expert LoRA), :453-543 (apply_lora).
"""
from __future__ import annotations

import contextlib
import contextvars

import torch

from ..models.dense import FlatParams
from ..ops.gemm import linear

# `attention` also names the mixer projections of the hybrid family's layers (fused input projection and
# output projection of a linear-attention layer, output gate of a gated softmax-attention layer);
# a layer only gets adapters for the projections it has
ROLE_TARGETS = {"attention": ("w_qkv", "w_o", "w_in", "w_out", "w_attn_gate"), "mlp": ("w_gate_up", "w_down"),
                "experts": ()}
# tensor parallelism: a column-parallel projection is split along its outputs (B follows the weight, A is replicated),
# a row-parallel one along its inputs (A follows the weight, B is replicated)
ROW_PARALLEL = ("w_o", "w_down", "w_out")


EXPERT_TARGETS = ("experts_gate_up", "experts_down")     # stacked [E_local, out, in] weights of an expert bank


class LoRAState:
    def __init__(self, flat: FlatParams, scale: float, dropout: float, flat_experts: FlatParams | None = None):
        self.flat, self.scale, self.dropout = flat, scale, dropout
        self.flat_experts = flat_experts      # per-expert adapter pairs (sharded with the experts), or None

    def expert_pair(self, layer_idx: int, name: str):
        if self.flat_experts is None:
            return None
        a = self.flat_experts.params.get(f"layers.{layer_idx}.{name}.lora_A")
        return None if a is None else (a, self.flat_experts.params[f"layers.{layer_idx}.{name}.lora_B"])

    def pair(self, layer_idx: int, name: str):
        a = self.flat.params.get(f"layers.{layer_idx}.{name}.lora_A")
        if a is None:
            return None
        return a, self.flat.params[f"layers.{layer_idx}.{name}.lora_B"]


_TOKEN_MASK: contextvars.ContextVar = contextvars.ContextVar("turbo_dllm_b200_lora_token_mask", default=None)


@contextlib.contextmanager
def lora_token_mask(mask: "torch.Tensor | bool | None"):
    """Inside the block the low-rank updates act only on the rows `mask` selects ([rows] bool; False: on no row;
    None: on every row). Context-local, so the recomputation of a checkpointed layer sees the mask of the code that
    replays it (dllm_parallel/core/adapters/lora.py:26-47)."""
    if mask is not None and not isinstance(mask, (torch.Tensor, bool)):
        raise TypeError("the LoRA token mask is a tensor, a bool or None")
    token = _TOKEN_MASK.set(mask)
    try:
        yield
    finally:
        _TOKEN_MASK.reset(token)


def current_lora_token_mask():
    return _TOKEN_MASK.get()


def lora_delta(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scale: float, dropout: float = 0.0,
               token_mask: torch.Tensor | None = None) -> torch.Tensor:
    if token_mask is None:
        token_mask = current_lora_token_mask()
    if token_mask is False:
        return torch.zeros((x.shape[0], b.shape[0]), dtype=x.dtype, device=x.device)
    if token_mask is True:
        token_mask = None
    if dropout > 0 and torch.is_grad_enabled():
        x = torch.nn.functional.dropout(x, dropout)
    low = linear(x, a)
    if token_mask is not None:
        if token_mask.numel() != x.shape[0]:
            raise ValueError(f"the LoRA token mask has {token_mask.numel()} entries for {x.shape[0]} rows")
        low = low * token_mask.reshape(-1, 1).to(low.dtype)     # unselected rows: no update, no adapter gradient
    return linear(low, b) * scale


def adapted_column_linear(layer, x: torch.Tensor, name: str) -> torch.Tensor:
    """x·Wᵀ of a column-parallel (or unsharded) projection `layer.<name>` plus its low-rank update. `layer` carries
    `lora` (a LoRAState or None), `tp` (tensor-parallel context or None) and `idx`. Under tensor parallelism A is
    replicated and B follows the weight's rows: the replicated x·Aᵀ (gathered rows under sequence parallelism) is
    multiplied by this rank's B."""
    from ..parallel.tensor_parallel import copy_to_tensor_parallel, gather_sequence_parallel, sp_column_linear

    st, tp = getattr(layer, "lora", None), getattr(layer, "tp", None)
    w = getattr(layer, name)
    pair = None if st is None else st.pair(layer.idx, name)
    g = tp.group if tp is not None and tp.size > 1 else None
    if g is None:
        out = linear(x, w)
        return out if pair is None else out + lora_delta(x, pair[0], pair[1], st.scale, st.dropout)
    sp = tp.sequence_parallel
    base = sp_column_linear(x, w, tp) if sp else linear(x, w, tp)
    if pair is None:
        return base
    low = linear(torch.nn.functional.dropout(x, st.dropout) if st.dropout > 0 and torch.is_grad_enabled() else x, pair[0])
    low = gather_sequence_parallel(low, g) if sp else copy_to_tensor_parallel(low, g)
    return base + linear(low, pair[1]) * st.scale


def adapted_row_linear(layer, x: torch.Tensor, name: str, residual: torch.Tensor, last: bool = False) -> torch.Tensor:
    """residual + x·Wᵀ of a row-parallel (or unsharded) projection plus its low-rank update. Under tensor parallelism A
    follows the weight's columns and B is replicated: the ranks' partial x_local·A_localᵀ are summed (all-reduce, or
    reduce-scatter of rows under sequence parallelism) before B applies."""
    from ..ops.gemm import row_parallel_linear_residual
    from ..parallel.tensor_parallel import (reduce_from_tensor_parallel, scatter_sequence_parallel,
                                            sp_row_linear_residual)

    st, tp = getattr(layer, "lora", None), getattr(layer, "tp", None)
    w = getattr(layer, name)
    pair = None if st is None else st.pair(layer.idx, name)
    g = tp.group if tp is not None and tp.size > 1 else None
    if g is None:
        out = residual + linear(x, w)
        return out if pair is None else out + lora_delta(x, pair[0], pair[1], st.scale, st.dropout)
    sp = tp.sequence_parallel
    out = (sp_row_linear_residual(x, w, residual, tp, last=last) if sp
           else row_parallel_linear_residual(x, w, residual, tp, last=last))
    if pair is None:
        return out
    low = linear(torch.nn.functional.dropout(x, st.dropout) if st.dropout > 0 and torch.is_grad_enabled() else x, pair[0])
    low = scatter_sequence_parallel(low, g) if sp else reduce_from_tensor_parallel(low, g)
    return out + linear(low, pair[1]) * st.scale


def apply_lora(model, *, rank: int, alpha: float | None = None, dropout: float = 0.0,
               targets=("attention", "mlp"), seed: int = 0, tp=None) -> LoRAState:
    """tp: the model's tensor-parallel context (None or size 1: one rank holds whole projections). Under tensor
    parallelism the adapters take the LOCAL shapes of the projections, and their start values are the matching
    slices of what a single rank would draw, so a tensor-parallel run starts from the same adapted model."""
    if rank <= 0:
        raise ValueError("LoRA rank must be positive")
    bad = sorted(set(targets) - set(ROLE_TARGETS))
    if bad:
        raise ValueError(f"unknown LoRA target roles {bad}; known: {sorted(ROLE_TARGETS)}")
    tp_size = tp.size if tp is not None else 1
    tp_rank = tp.rank if tp is not None else 0
    if tp_size > 1 and dropout > 0:
        raise ValueError("adapter.dropout must be 0 under tensor parallelism (ranks would draw different masks "
                         "for replicated rows)")
    names = [n for role in targets for n in ROLE_TARGETS[role]]
    r8 = (rank + 7) // 8 * 8            # GEMM operands need 16-byte rows; extra rows stay zero
    sharded, replicated, order = [], [], []
    for i, layer in enumerate(model.layers):
        for n in names:
            w = getattr(layer, n, None)
            if w is None:
                continue
            out_f, in_f = w.shape
            a = (f"layers.{i}.{n}.lora_A", (r8, in_f), True)
            b = (f"layers.{i}.{n}.lora_B", (out_f, r8), True)
            row = n in ROW_PARALLEL
            (sharded if row or tp_size == 1 else replicated).append(a)
            (replicated if row and tp_size > 1 else sharded).append(b)
            order.append((a[0], in_f, row))
    expert_specs = []
    if "experts" in targets:
        for i, layer in enumerate(model.layers):
            bank = getattr(layer, "experts", None)
            if bank is None:
                continue
            for n, w in (("experts_gate_up", bank.w_gu), ("experts_down", bank.w_down)):
                e_local, out_f, in_f = w.shape
                expert_specs += [(f"layers.{i}.{n}.lora_A", (e_local, r8, in_f), True),
                                 (f"layers.{i}.{n}.lora_B", (e_local, out_f, r8), True)]
        if not expert_specs:
            raise ValueError("adapter target 'experts' needs a mixture-of-experts model")
    if not order:
        raise ValueError("no projection matches the requested LoRA targets" if not expert_specs else
                         "expert adapters come with at least one of the roles attention / mlp (the replicated and "
                         "the expert-sharded adapters are two optimizer buffers)")
    base = model.flat
    flat = FlatParams(sharded + replicated, base.data.dtype, base.data.device)
    if tp_size > 1:
        # the optimizer sums the squared gradients of the sharded part over the tensor-parallel group and counts
        # the replicated part once
        flat.tp_sharded_numel = flat.offsets[replicated[0][0]][0] if replicated else flat.numel
    gen = torch.Generator(device=base.data.device)
    gen.manual_seed(seed + 4242)
    with torch.no_grad():
        flat.data.zero_()
        for name, in_f, row in order:            # the order a single rank draws in; B starts at zero
            p = flat.params[name]
            full_in = in_f * tp_size if row else in_f
            draw = (torch.randn((rank, full_in), device=p.device, generator=gen) * (1.0 / rank ** 0.5)).to(p.dtype)
            p[:rank].copy_(draw[:, tp_rank * in_f:(tp_rank + 1) * in_f] if row and tp_size > 1 else draw)
    if tp_size > 1 and getattr(tp, "sequence_parallel", False):
        # rows are divided over the ranks: a replicated adapter matrix sees this rank's rows only
        for spec in replicated:
            flat.params[spec[0]].tp_partial = True
    flat_experts = None
    if expert_specs:
        flat_experts = FlatParams(expert_specs, base.data.dtype, base.data.device)
        ep_rank = getattr(model.layers[0].experts, "ep_rank", 0)
        egen = torch.Generator(device=base.data.device)
        egen.manual_seed(seed + 977 + 131 * ep_rank)          # experts differ per expert-parallel rank
        if tp_size > 1 and getattr(tp, "sequence_parallel", False):
            # the experts (and their pairs) are replicated over the tensor-parallel ranks, which route their own rows
            for p in flat_experts.params.values():
                p.tp_partial = True
        with torch.no_grad():
            flat_experts.data.zero_()
            for name, p in flat_experts.params.items():
                p.expert_written = set()
                if name.endswith("lora_A"):
                    p[:, :rank].copy_((torch.randn((p.shape[0], rank, p.shape[2]), device=p.device, generator=egen)
                                       * (1.0 / rank ** 0.5)).to(p.dtype))
    for p in base.params.values():
        p.requires_grad_(False)
    state = LoRAState(flat, (alpha if alpha is not None else float(rank)) / rank, dropout, flat_experts)
    for layer in model.layers:
        layer.lora = state
        if getattr(layer, "experts", None) is not None:
            layer.experts.lora = state if flat_experts is not None else None
    model.lora = state
    return state


def lora_merge_plan(model) -> list[dict]:
    """What `merge_lora` will do, checked before anything is written: one entry per adapted projection with the
    target's name and shape, the adapter shapes and the kind (`linear`: W += s·B·A; `grouped`: per expert
    W[e] += s·B[e]·A[e]). Raises when an adapter does not fit its target.
    Role of the validated merge plan of dllm_parallel/core/models/backbones/diffusiongemma/export.py:63-376."""
    st = getattr(model, "lora", None)
    if st is None:
        return []
    plan = []
    for i, layer in enumerate(model.layers):
        for n in (n for names in ROLE_TARGETS.values() for n in names):
            pair = st.pair(i, n)
            if pair is None:
                continue
            a, b = pair
            w = getattr(layer, n)
            if b.shape[0] != w.shape[0] or a.shape[1] != w.shape[1] or a.shape[0] != b.shape[1]:
                raise ValueError(f"layers.{i}.{n}: adapter A{tuple(a.shape)} / B{tuple(b.shape)} does not fit "
                                 f"the weight {tuple(w.shape)}")
            plan.append({"target": f"layers.{i}.{n}", "kind": "linear", "weight": list(w.shape),
                         "A": list(a.shape), "B": list(b.shape), "scale": st.scale})
        bank = getattr(layer, "experts", None)
        if bank is not None:
            for n, w in (("experts_gate_up", bank.w_gu), ("experts_down", bank.w_down)):
                pair = st.expert_pair(i, n)
                if pair is None:
                    continue
                a, b = pair
                if (a.shape[0] != w.shape[0] or b.shape[0] != w.shape[0] or b.shape[1] != w.shape[1]
                        or a.shape[2] != w.shape[2] or a.shape[1] != b.shape[2]):
                    raise ValueError(f"layers.{i}.{n}: expert adapters A{tuple(a.shape)} / B{tuple(b.shape)} do not "
                                     f"fit the stacked weight {tuple(w.shape)}")
                plan.append({"target": f"layers.{i}.{n}", "kind": "grouped", "weight": list(w.shape),
                             "A": list(a.shape), "B": list(b.shape), "scale": st.scale})
    return plan


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
        bank = getattr(layer, "experts", None)
        if bank is not None:
            for n, w in (("experts_gate_up", bank.w_gu), ("experts_down", bank.w_down)):
                pair = st.expert_pair(i, n)
                if pair is not None:         # per expert: W[e] += scale * B[e] @ A[e]
                    w.add_((torch.bmm(pair[1].float(), pair[0].float()) * st.scale).to(w.dtype))
