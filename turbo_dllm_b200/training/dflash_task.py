"""DFlash drafter-distillation task: frozen target forward → anchors and drafting blocks →
draft forward over [draft rows ; conditioned context] → soft-label KL through the frozen head.

With `model.dflash2_*` set the drafter is the DFlash2 architecture (block-local dynamic convolutions,
candidate selector) and the losses `dflash` / `dpace*` apply: hard-label cross-entropy through the
frozen head with position weights that are either the sampled decay weights (`dflash`) or the D-PACE
weights computed from the drafter's own label probabilities, optionally mixed with a total-variation
term (`lk_loss_type`), plus the selector's cross-entropy over the head's top-k candidates.

Counterparts: DFlashTrainingTask (dllm_parallel/core/models/backbones/dflash/training.py:29-197),
`distributed_dflash_loss` (dllm_parallel/core/models/backbones/dflash/model.py:862-956,
dllm_parallel/core/models/backbones/dflash/dflash2.py:552-701).
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
    def __init__(self, spec, cfg: ModelConfig, *, dtype, device, seed: int, dp_rank: int, exchange=None,
                 replicas: int | None = None):
        """exchange: a parallel.dflash_context.DFlashContextParallel when one replica spans several ranks (they
        divide the anchors and, with context parallelism, the context rows); replicas: data-parallel size."""
        m, o = spec.model, spec.objective
        self.spec, self.cfg, self.device = spec, cfg, device
        self.exchange, self.replicas = exchange, replicas
        import os
        from dataclasses import replace

        self.offline = spec.data.target_features == "offline"
        hf_dir = m.verifier_id if (m.verifier_id and os.path.isdir(m.verifier_id)) else None
        target_cfg = PRESETS.get(m.verifier_id or "")
        if hf_dir is not None:
            # a Hugging Face checkpoint directory on disk: its config gives the shapes, its tensors the weights
            from ..models.hf_loader import load_hf_config

            target_cfg = load_hf_config(hf_dir)
        if target_cfg is None:
            raise ValueError(f"model.verifier_id {m.verifier_id!r} is neither a built-in target preset "
                             f"({', '.join(k for k in PRESETS)}) nor a Hugging Face checkpoint directory")
        layer_ids = tuple(m.target_layer_ids)
        full_layers = target_cfg.num_layers
        if self.offline:
            # hidden states come from the feature store: only the verifier's embedding and head are needed
            target_cfg = replace(target_cfg, num_layers=0)
        self.target = FrozenTarget(target_cfg, () if self.offline else layer_ids, dtype=dtype, device=device,
                                   seed=seed + 1)
        self.target.layer_ids = layer_ids
        if hf_dir is not None:
            from ..models.hf_loader import load_hf_weights

            load_hf_weights(self.target.model, hf_dir)
        # model.draft_vocab_path: the drafter predicts a subset of the verifier's vocabulary; the frozen head of the
        # losses is then the verifier head's rows of that subset
        self.draft_vocab = None
        self.head = self.target.lm_head
        if m.draft_vocab_path:
            from ..models.dflash import DraftVocabulary

            self.draft_vocab = DraftVocabulary.load(m.draft_vocab_path, target_cfg.vocab_size)
            if self.draft_vocab.size % 8:
                raise ValueError(f"the draft vocabulary has {self.draft_vocab.size} ids; the logit rows of the loss "
                                 "kernels need a multiple of 8")
            self.head = self.draft_vocab.head_rows(self.target.lm_head)
        self.feature_store = None
        if self.offline:
            from ..data.dflash_features import FeatureStore

            self.feature_store = FeatureStore(spec.data.target_feature_path, verify=True)
            man = self.feature_store.manifest
            if list(man.get("target_layer_ids", [])) != list(layer_ids) or int(man.get("seq_len", 0)) != m.seq_len:
                raise ValueError(f"feature store {spec.data.target_feature_path} was captured for target layers "
                                 f"{man.get('target_layer_ids')} at seq_len {man.get('seq_len')}; the run asks for "
                                 f"{list(layer_ids)} at {m.seq_len}")
            if any(i >= full_layers for i in layer_ids):
                raise ValueError(f"target_layer_ids {layer_ids} outside the verifier's {full_layers} layers")
        self.is_dflash2 = bool(m.dflash2_conv_kernel_size or m.dflash2_selector_rank)
        if self.is_dflash2:
            from ..models.dflash2 import DFlash2DraftModel

            self.model = DFlash2DraftModel(
                cfg, target_hidden=target_cfg.hidden_size, num_target_layers=len(m.target_layer_ids),
                block_size=o.block_size or 16, conv_kernel_size=m.dflash2_conv_kernel_size or 1,
                conv_group_size=m.dflash2_conv_group_size or cfg.hidden_size,
                selector_rank=m.dflash2_selector_rank or 1, selector_top_k=m.dflash2_selector_top_k or 1,
                verifier_vocab_size=target_cfg.vocab_size, dtype=dtype, device=device, seed=seed)
        else:
            self.model = DFlashDraftModel(cfg, target_hidden=target_cfg.hidden_size,
                                          num_target_layers=len(m.target_layer_ids), dtype=dtype, device=device,
                                          seed=seed)
        from ..models.hf_loader import pretrained_directory

        start = None if m.random_init else pretrained_directory(m.id)
        if start is not None:
            # model.id names a drafter checkpoint on disk (module-style tensor names): continue from its weights
            if self.is_dflash2:
                raise ValueError("continuing from a drafter checkpoint is built for the DFlash drafter; a DFlash2 run "
                                 "resumes from its training checkpoints")
            from ..models.export import load_speculators_checkpoint

            load_speculators_checkpoint(self.model, start)
        from ..ops.dflash2 import DPACE_LOSSES

        if o.dflash_loss in ("dflash",) + DPACE_LOSSES and not self.is_dflash2:
            raise ValueError(f"objective.dflash_loss={o.dflash_loss} needs the DFlash2 drafter "
                             "(model.dflash2_conv_kernel_size, model.dflash2_selector_rank, ...)")
        if o.lk_loss_type not in (None, "alpha", "lambda", "tv"):
            raise ValueError("objective.lk_loss_type must be unset, alpha, lambda or tv")
        self.effective_selector_loss_alpha = float(o.selector_loss_alpha)
        self.last_objective_metrics: dict = {}
        max_anchors = o.max_anchors or max(m.seq_len // (o.block_size or 16) // 2, 1)
        self.objective = DFlashObjectiveRuntime(
            block_size=o.block_size or 16, max_anchors=max_anchors, mask_token_id=target_cfg.mask_token_id,
            seed=seed + 7919 * (dp_rank + 1), device=device, anchor_sampling=o.anchor_sampling,
            anchor_group_size=o.anchor_group_size, sample_from_anchor=o.sample_from_anchor, decay_gamma=o.decay_gamma)
        self.loss_kind = o.dflash_loss
        self.synthetic = spec.data.target_features == "synthetic"
        # sliding-window drafters: leave out context rows no window reaches (TDLLM_DFLASH_COMPACT_CONTEXT=0 keeps them)
        self.compact_context = os.environ.get("TDLLM_DFLASH_COMPACT_CONTEXT", "1") != "0"
        self.last_context_rows = None
        if cfg.has_sliding_layers and exchange is not None:
            raise ValueError("sliding-window drafter layers are built for replicas on one rank "
                             "(context_parallel_size = block_parallel_size = 1)")

    def set_optimizer_step(self, step: int, total_steps: int) -> None:
        """Warm-up and ramp of the selector loss (fractions of the run's optimizer steps)."""
        from ..ops.dflash2 import selector_schedule_factor

        o = self.spec.objective
        self.effective_selector_loss_alpha = float(o.selector_loss_alpha) * selector_schedule_factor(
            int(step), int(total_steps), float(o.selector_warmup_ratio), float(o.selector_ramp_ratio))

    def target_features(self, input_ids: torch.Tensor, batch=None) -> TargetFeatures:
        if self.offline:
            feats = getattr(batch, "features", None)
            if feats is None:
                raise ValueError("data.target_features=offline needs batches of the feature-store data runtime")
            dt = self.model.flat.data.dtype
            fh = feats["final_hidden"]
            fh = fh.reshape(-1, fh.shape[-1])
            return TargetFeatures(feats["hidden"].reshape(-1, feats["hidden"].shape[-1]).to(dt),
                                  fh if fh.device != self.model.flat.data.device else fh.to(dt),
                                  bool(feats.get("hidden_is_shard", False)))
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
        feats = self.target_features(ids, batch)
        bs = self.objective.block_size
        ex = self.exchange
        if ex is None:
            ctx_features = feats.hidden
            pos_ctx = torch.arange(l, device=ids.device).repeat(b)
            window = self.cfg.sliding_window if self.cfg.has_sliding_layers else None
            if window is None:
                mask = dflash_mask_layout(ob, l, bs)
            else:
                from ..models.dflash import DraftMasks, window_context_rows

                every_layer = all(self.cfg.layer_window(i) is not None for i in range(self.cfg.num_layers))
                keep = window_context_rows(ob, l, window) if every_layer and self.compact_context else None
                windowed = dflash_mask_layout(ob, l, bs, window=window, context_rows=keep)
                mask = DraftMasks(windowed if every_layer else dflash_mask_layout(ob, l, bs), windowed)
                if keep is not None:      # rows no window reaches take no part in the step
                    ctx_features = ctx_features.index_select(0, keep)
                    pos_ctx = pos_ctx.index_select(0, keep)
                    self.last_context_rows = int(keep.numel())
        else:
            # this rank's anchors of the (replica-wide identical) sample, and its shard of the context rows
            from ..parallel.dflash_context import select_anchors

            c = self.cfg
            plan = ex.plan(ob, bs, l, q_heads=c.num_attention_heads, kv_heads=c.num_key_value_heads,
                           head_dim=c.head_dim)
            ob = select_anchors(ob, ex.anchor_index(ob.anchor_positions.shape[1], device=ids.device))
            mask = (ex, plan)
            ctx_features = (feats.hidden if feats.hidden_is_shard
                            else feats.hidden.index_select(0, ex.context_rows(b, l, ids.device)))
            pos_ctx = ex.context_positions(l, device=ids.device).repeat(b)
        draft_tok = ob.draft_input_ids.reshape(-1)
        draft_emb = embedding(draft_tok, self.target.embed)
        pos_draft = ob.block_positions.reshape(-1)
        hidden = self.model(draft_emb, ctx_features, pos_draft, pos_ctx, mask)
        sup = ob.supervised_mask.reshape(-1)
        w = ob.position_weights.reshape(-1) * sup.float()
        rows = sup.nonzero(as_tuple=True)[0]
        seq_off = (torch.arange(b, device=ids.device) * l)[:, None, None]
        src = (ob.teacher_source_positions + seq_off).reshape(-1)
        h_s = hidden.index_select(0, rows)
        want = src.index_select(0, rows)
        fh = feats.final_hidden
        if fh.device != hidden.device:      # memory-mapped on the host: only the needed teacher rows are read
            h_t = fh.index_select(0, want.to(fh.device)).to(hidden.device, hidden.dtype)
        else:
            h_t = fh.index_select(0, want)
        wr = w.index_select(0, rows)
        if self.loss_kind == "speculators_kl":
            loss_sum, _ = frozen_linear_kl(h_s, h_t, self.head, wr)
        elif self.is_dflash2 and self.loss_kind != "paper_ce":
            tgt_all = ids.reshape(-1).index_select(0, (ob.target_token_positions + seq_off).reshape(-1))
            loss_sum, denom = self._dflash2_loss(h_s, rows, tgt_all, sup, ob.position_weights.reshape(-1))
            (loss_sum / denom).backward()
            return loss_sum.detach(), int(rows.numel()), denom
        else:  # paper_ce: hard labels = the data token at the target position
            tgt = (ob.target_token_positions + seq_off).reshape(-1).index_select(0, rows)
            labels = ids.reshape(-1).index_select(0, tgt)
            if self.draft_vocab is not None:    # tokens the drafter cannot emit are not supervised
                labels = self.draft_vocab.to_draft_ids(labels)
                wr = wr * (labels >= 0).to(wr.dtype)
                labels = labels.clamp_min(0)
            loss_sum, _ = linear_cross_entropy(h_s, self.head, labels, wr, frozen_weight=True)
        if denominator is None:
            wsum = wr.sum()
            if ex is not None:            # the anchors of this micro-batch are spread over the replica's ranks
                torch.distributed.all_reduce(wsum, group=ex.group)
            denom = wsum.clamp_min(1.0)
        else:
            denom = denominator
        (loss_sum / denom).backward()
        return loss_sum.detach(), int(rows.numel()), denom

    def _dflash2_loss(self, hidden, rows, targets_all, supervised, position_weights):
        """hidden [n, H]: supervised draft rows `rows`; targets_all / supervised / position_weights:
        per draft row in block order. Returns (loss numerator with gradient, detached denominator)."""
        from ..ops.dflash2 import DPACE_LOSSES, dpace_weight, frozen_linear_ce_topk

        o, model = self.spec.objective, self.model
        bs = self.objective.block_size
        sel = model.candidate_selector
        selector_on = bool(model.selector_objective_enabled) and self.effective_selector_loss_alpha > 0.0
        labels = targets_all.index_select(0, rows)
        head = self.target.lm_head
        kw = dict(top_k=sel.top_k if selector_on else 1, vocab_block_size=int(o.dflash_vocab_block_size),
                  output_multiplier=model.output_multiplier, logit_softcap=model.final_logit_softcapping)
        with torch.no_grad():      # label probabilities first: the position weights depend on them
            _, _, prob, _, _ = frozen_linear_ce_topk(hidden.detach(), head, labels, **kw)
        mask = supervised.reshape(-1, bs).float()
        full_p = torch.zeros_like(mask).view(-1).index_copy_(0, rows, prob).view(-1, bs)
        if self.loss_kind == "dflash":
            weights = mask * position_weights.reshape(-1, bs).float()
        else:
            weights = mask * dpace_weight(full_p, mask, alpha=float(o.dpace_alpha), kind=self.loss_kind)
        w_rows = weights.reshape(-1).index_select(0, rows)
        # cross-entropy / total-variation mix. d(1 - p)/dh = p * d(ce)/dh, so the total-variation
        # term is a cross-entropy whose row weights carry the detached probability.
        # sums over all data-parallel ranks: weighted supervised count, accepted probability mass, supervised count
        stats = torch.stack([w_rows.sum(), (full_p * mask).sum(), mask.sum()]).detach().clone()
        world = 1
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            world = torch.distributed.get_world_size()
            if world > 1:
                torch.distributed.all_reduce(stats)
        ce_share = 1.0
        if o.lk_loss_type == "tv":
            ce_share = 0.0
        elif o.lk_loss_type == "lambda":
            acceptance = stats[1] / stats[2].clamp_min(1.0)
            ce_share = float(o.kl_scale) * float(torch.exp(-float(o.kl_decay) * acceptance))
        eff = w_rows * (ce_share + (1.0 - ce_share) * prob)
        grad_carrier, ce, _, unary, cand = frozen_linear_ce_topk(hidden, head, labels, loss_weights=eff, **kw)
        value = (ce_share * ce + (1.0 - ce_share) * (1.0 - prob)) * w_rows
        token_num = value.sum() + (grad_carrier - grad_carrier.detach())
        selector_num = token_num.new_zeros(())
        covered = torch.zeros_like(labels, dtype=torch.bool)
        if selector_on:
            blocks = targets_all.reshape(-1, bs)
            predecessor = torch.cat([blocks[:, :1], blocks[:, :-1]], dim=-1).reshape(-1).index_select(0, rows)
            stop = bool(o.selector_stop_gradient)
            matches = cand.eq(labels[:, None])
            covered = matches.any(-1)
            scores = sel.score_candidates(candidate_ids=cand, unary_logits=unary.detach() if stop else unary,
                                          hidden_states=hidden.detach() if stop else hidden,
                                          predecessor_ids=predecessor)
            sel_ce = torch.nn.functional.cross_entropy(scores.float(), matches.long().argmax(-1), reduction="none")
            sel_w = w_rows * covered.float()
            selector_num = (sel_ce * sel_w).sum()
            self.last_objective_metrics["selector_loss"] = (selector_num.detach() / sel_w.sum().clamp_min(1.0))
        self.last_objective_metrics.update(target_probability=prob.mean(), selector_coverage=covered.float().mean())
        # the session averages per-rank losses over the ranks: dividing by (global count / ranks) makes that
        # average the global sum over the global count
        denom = (stats[0] / (self.replicas or world)).clamp_min(torch.finfo(torch.float32).tiny)
        return token_num + self.effective_selector_loss_alpha * selector_num, denom
