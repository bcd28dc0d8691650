"""DFlash drafter-distillation task: frozen target forward → anchors and drafting blocks →
draft forward over [draft rows ; conditioned context] → soft-label KL through the frozen head.

Counterparts: DFlashTrainingTask (dllm_parallel/core/models/backbones/dflash/training.py:29-197),
`distributed_dflash_loss` (dllm_parallel/core/models/backbones/dflash/model.py:862-956).
"""
from __future__ import annotations

import torch

from ..models.config import PRESETS, ModelConfig
from ..models.dflash import DFlashDraftModel, FrozenTarget, TargetFeatures, dflash_mask_layout
from ..objectives.dflash import DFlashObjectiveRuntime
from ..ops.distill import frozen_linear_kl
from ..ops.embedding import embedding
from ..ops.linear_ce import linear_cross_entropy


class DFlashTask:
    def __init__(self, spec, cfg: ModelConfig, *, dtype, device, seed: int, dp_rank: int):
        m, o = spec.model, spec.objective
        self.spec, self.cfg, self.device = spec, cfg, device
        target_cfg = PRESETS.get(m.verifier_id or "")
        if target_cfg is None:
            raise ValueError(f"model.verifier_id {m.verifier_id!r} is not a built-in target preset "
                             f"({', '.join(k for k in PRESETS)}); offline features need data.target_features=offline")
        if spec.data.target_features == "offline":
            raise NotImplementedError("offline target-feature stores are read by data.dflash_features")
        if m.max_layers is not None and spec.data.target_features == "synthetic":
            pass
        self.target = FrozenTarget(target_cfg, tuple(m.target_layer_ids), dtype=dtype, device=device, seed=seed + 1)
        self.model = DFlashDraftModel(cfg, target_hidden=target_cfg.hidden_size,
                                      num_target_layers=len(m.target_layer_ids), dtype=dtype, device=device, seed=seed)
        max_anchors = o.max_anchors or max(m.seq_len // (o.block_size or 16) // 2, 1)
        self.objective = DFlashObjectiveRuntime(
            block_size=o.block_size or 16, max_anchors=max_anchors, mask_token_id=target_cfg.mask_token_id,
            seed=seed + 7919 * (dp_rank + 1), device=device, anchor_sampling=o.anchor_sampling,
            anchor_group_size=o.anchor_group_size, sample_from_anchor=o.sample_from_anchor, decay_gamma=o.decay_gamma)
        self.loss_kind = o.dflash_loss
        self.synthetic = spec.data.target_features == "synthetic"

    def target_features(self, input_ids: torch.Tensor) -> TargetFeatures:
        if self.synthetic:  # random features of the right shape: exercises the drafter without a target pass
            b, l = input_ids.shape
            g = torch.Generator(device=self.device)
            g.manual_seed(int(input_ids.sum()) % (2 ** 31))
            th = self.target.cfg.hidden_size
            dt = self.model.flat.data.dtype
            hid = torch.randn(b * l, th * len(self.target.layer_ids), device=self.device, generator=g).to(dt)
            return TargetFeatures(hid, torch.randn(b * l, th, device=self.device, generator=g).to(dt))
        return self.target.features(input_ids)

    def forward_backward(self, batch, denominator=None):
        ids = batch.input_ids
        b, l = ids.shape
        ob = self.objective.prepare(ids, batch.supervision_mask)
        feats = self.target_features(ids)
        bs = self.objective.block_size
        mask = dflash_mask_layout(ob, l, bs)
        draft_tok = ob.draft_input_ids.reshape(-1)
        draft_emb = embedding(draft_tok, self.target.embed)
        pos_draft = ob.block_positions.reshape(-1)
        pos_ctx = torch.arange(l, device=ids.device).repeat(b)
        hidden = self.model(draft_emb, feats.hidden, pos_draft, pos_ctx, mask)
        sup = ob.supervised_mask.reshape(-1)
        w = ob.position_weights.reshape(-1) * sup.float()
        rows = sup.nonzero(as_tuple=True)[0]
        seq_off = (torch.arange(b, device=ids.device) * l)[:, None, None]
        src = (ob.teacher_source_positions + seq_off).reshape(-1)
        h_s = hidden.index_select(0, rows)
        h_t = feats.final_hidden.index_select(0, src.index_select(0, rows))
        wr = w.index_select(0, rows)
        if self.loss_kind == "speculators_kl":
            loss_sum, _ = frozen_linear_kl(h_s, h_t, self.target.lm_head, wr)
        else:  # paper_ce: hard labels = the data token at the target position
            tgt = (ob.target_token_positions + seq_off).reshape(-1).index_select(0, rows)
            labels = ids.reshape(-1).index_select(0, tgt)
            loss_sum, _ = linear_cross_entropy(h_s, self.target.lm_head, labels, wr, frozen_weight=True)
        denom = wr.sum().clamp_min(1.0) if denominator is None else denominator
        (loss_sum / denom).backward()
        return loss_sum.detach(), int(rows.numel()), denom
