"""DFlash drafter-distillation objective: anchors, drafting blocks, supervision and weights.

For every sequence `max_anchors` anchor positions are sampled among positions that are
supervised and have a successor in the same document. An anchor at position a opens a drafting
block of `block_size` slots at positions a .. a+bs-1: slot 0 carries the anchor's real token, the
other slots the mask token. Slot j is supervised with the token at its own position (teacher
distribution taken from the target model's output at position-1), unless it crosses the end of
the sequence or of the anchor's document; slot 0 is never supervised (unless
`sample_from_anchor`, where slot j predicts position a+j+1 from the teacher at a+j). Position
weights decay exponentially with the slot index (`decay_gamma`). Each drafting block attends
bidirectionally to itself and to the target context `[document_start, anchor)`.

Semantics follow dllm_parallel/core/objectives/dflash.py:122-230 (prepare), :311-350 (anchor
sampling), :394-510 (weights, reference loss); attention masks dllm_parallel/core/attention/masks.py:246-313.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

STATE_VERSION = 1


@dataclass
class DFlashBatch:
    anchor_positions: torch.Tensor        # [B, A]
    anchor_valid: torch.Tensor            # [B, A] bool
    block_positions: torch.Tensor         # [B, A, bs] clamped to the sequence
    teacher_source_positions: torch.Tensor  # [B, A, bs]
    target_token_positions: torch.Tensor  # [B, A, bs]
    draft_input_ids: torch.Tensor         # [B, A*bs]
    supervised_mask: torch.Tensor         # [B, A*bs] bool
    position_weights: torch.Tensor        # [B, A*bs] float32
    document_starts: torch.Tensor         # [B, A] int32 (seq_len for invalid anchors)
    context_stops: torch.Tensor           # [B, A] int32

    @property
    def valid_supervised_tokens(self) -> torch.Tensor:
        return self.supervised_mask.sum(dim=1, dtype=torch.float32)


def document_starts(document_ids: torch.Tensor) -> torch.Tensor:
    """Start position of the contiguous document segment each position belongs to."""
    b, l = document_ids.shape
    change = torch.ones_like(document_ids, dtype=torch.bool)
    change[:, 1:] = document_ids[:, 1:] != document_ids[:, :-1]
    pos = torch.arange(l, device=document_ids.device).expand(b, l)
    return torch.where(change, pos, torch.zeros_like(pos)).cummax(dim=1).values


def position_weights(block_size: int, gamma: float | None, sample_from_anchor: bool, device) -> torch.Tensor:
    idx = torch.arange(block_size, dtype=torch.float32, device=device)
    if gamma is None or gamma <= 0:
        return torch.ones(block_size, device=device)
    first = 0.0 if sample_from_anchor else 1.0      # first supervised slot has weight 1
    return torch.exp(-(idx - first).clamp_min(0) / gamma)


class DFlashObjectiveRuntime:
    name = "dflash_distillation"

    def __init__(self, *, block_size: int, max_anchors: int, mask_token_id: int, seed: int, device="cpu",
                 anchor_sampling: str = "uniform", anchor_group_size: int = 0, sample_from_anchor: bool = False,
                 decay_gamma: float | None = None):
        if anchor_sampling not in ("uniform", "locality"):
            raise ValueError(f"unknown anchor_sampling {anchor_sampling!r}")
        self.block_size, self.max_anchors, self.mask_token_id = block_size, max_anchors, mask_token_id
        self.anchor_sampling, self.anchor_group_size = anchor_sampling, anchor_group_size
        self.sample_from_anchor, self.decay_gamma = sample_from_anchor, decay_gamma
        self.device = torch.device(device)
        self.generator = torch.Generator(device=self.device)
        self.generator.manual_seed(int(seed))
        self.seed = int(seed)
        self.batches_sampled = 0

    # ----------------------------------------------------------- sampling
    def _sample_anchors(self, valid: torch.Tensor):
        """valid [B, L] bool -> (positions [B, A] ascending, valid [B, A])."""
        b, l = valid.shape
        a = self.max_anchors
        scores = torch.rand((b, l), device=self.device, generator=self.generator)
        if self.anchor_sampling == "locality" and self.anchor_group_size > 1:
            # anchors come in groups of consecutive strides: pick group leaders, then expand
            g = self.anchor_group_size
            leaders = max(a // g, 1)
            lead_scores = torch.where(valid, scores, torch.full_like(scores, -1.0))
            lead = lead_scores.topk(leaders, dim=1).indices
            offs = torch.arange(g, device=self.device) * self.block_size
            pos = (lead[:, :, None] + offs[None, None, :]).reshape(b, -1)[:, :a].clamp_max(l - 1)
            ok = valid.gather(1, pos)
            if pos.shape[1] < a:
                pad = a - pos.shape[1]
                pos = torch.cat([pos, pos.new_zeros(b, pad)], 1)
                ok = torch.cat([ok, ok.new_zeros(b, pad)], 1)
        else:
            masked = torch.where(valid, scores, torch.full_like(scores, -1.0))
            top = masked.topk(min(a, l), dim=1)
            pos, ok = top.indices, top.values >= 0
            if pos.shape[1] < a:
                pad = a - pos.shape[1]
                pos = torch.cat([pos, pos.new_zeros(b, pad)], 1)
                ok = torch.cat([ok, ok.new_zeros(b, pad)], 1)
        key = torch.where(ok, pos, torch.full_like(pos, l))   # invalid anchors sort last
        order = key.argsort(dim=1)
        return pos.gather(1, order), ok.gather(1, order)

    def prepare(self, input_ids: torch.Tensor, loss_mask: torch.Tensor | None = None,
                document_ids: torch.Tensor | None = None) -> DFlashBatch:
        if input_ids.ndim != 2:
            raise ValueError("input_ids must be [batch, seq]")
        b, l = input_ids.shape
        dev = input_ids.device
        loss_mask = torch.ones_like(input_ids, dtype=torch.bool) if loss_mask is None else loss_mask.to(dev, torch.bool)
        document_ids = torch.zeros_like(input_ids) if document_ids is None else document_ids.to(dev, torch.int64)
        starts = document_starts(document_ids)
        # a valid anchor has a supervised successor inside the same document
        nxt_same = torch.zeros_like(loss_mask)
        nxt_same[:, :-1] = (starts[:, 1:] == starts[:, :-1]) & loss_mask[:, 1:]
        anchors, valid = self._sample_anchors(nxt_same)
        offs = torch.arange(self.block_size, device=dev)
        block_pos = anchors[:, :, None] + offs
        target_pos = block_pos + 1 if self.sample_from_anchor else block_pos
        safe_block = block_pos.clamp_max(l - 1)
        safe_target = target_pos.clamp_max(l - 1)
        teacher_src = safe_block if self.sample_from_anchor else (safe_target - 1).clamp_min(0)
        draft = torch.full((b, self.max_anchors, self.block_size), self.mask_token_id, dtype=input_ids.dtype, device=dev)
        draft[:, :, 0] = input_ids.gather(1, anchors)
        sup = loss_mask.gather(1, safe_target.reshape(b, -1)).reshape(b, self.max_anchors, self.block_size)
        anchor_doc = starts.gather(1, anchors)
        tgt_doc = starts.gather(1, safe_target.reshape(b, -1)).reshape(b, self.max_anchors, self.block_size)
        sup &= target_pos < l
        sup &= tgt_doc == anchor_doc[:, :, None]
        sup &= valid[:, :, None]
        if not self.sample_from_anchor:
            sup[:, :, 0] = False
        w = position_weights(self.block_size, self.decay_gamma, self.sample_from_anchor, dev)
        w = w.view(1, 1, -1).expand_as(sup).to(torch.float32)
        invalid = torch.full_like(anchors, l)
        self.batches_sampled += 1
        return DFlashBatch(
            anchor_positions=anchors, anchor_valid=valid, block_positions=safe_block,
            teacher_source_positions=teacher_src, target_token_positions=safe_target,
            draft_input_ids=draft.reshape(b, -1).contiguous(), supervised_mask=sup.reshape(b, -1).contiguous(),
            position_weights=w.reshape(b, -1).contiguous(),
            document_starts=torch.where(valid, anchor_doc, invalid).to(torch.int32),
            context_stops=torch.where(valid, anchors, invalid).to(torch.int32))

    def state_dict(self) -> dict[str, Any]:
        return {"kind": self.name, "version": STATE_VERSION, "seed": self.seed,
                "generator_state": self.generator.get_state().cpu(), "batches_sampled": self.batches_sampled}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if state.get("kind") != self.name or state.get("version") != STATE_VERSION:
            raise ValueError("objective state is not a DFlash state of this version")
        self.generator.set_state(state["generator_state"].cpu())
        self.batches_sampled = int(state["batches_sampled"])


def reference_dflash_loss(student_logits, teacher_logits, supervised_mask, weights, kind: str = "speculators_kl"):
    """Dense oracle. logits [rows, V]; mask/weights [rows]. Returns Σ w·loss over supervised rows."""
    m = supervised_mask.bool()
    if kind == "speculators_kl":
        ls = torch.log_softmax(student_logits.float(), -1)
        lt = torch.log_softmax(teacher_logits.float(), -1)
        per = (lt.exp() * (lt - ls)).sum(-1)
    elif kind == "paper_ce":
        per = torch.nn.functional.cross_entropy(student_logits.float(), teacher_logits.argmax(-1), reduction="none")
    else:
        raise ValueError(f"unknown dflash loss {kind!r}")
    return (per * weights.float() * m.float()).sum(), per
