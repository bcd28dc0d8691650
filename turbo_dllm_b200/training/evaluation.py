"""Masked-token accuracy evaluation on held-out batches (no gradient, fixed seed).

Every evaluation batch is corrupted with the run's objective under its own generator
(`evaluation.seed`), the model predicts the masked positions and accuracy / mean loss are reduced
over data-parallel ranks. Counterpart of `_evaluate_masked_token_accuracy`
(dllm_parallel/training/block_diffusion_trainer.py:1981-2107).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.dense import compact_supervised_rows
from ..objectives.runtime import build_objective_runtime


@torch.no_grad()
def evaluate_masked_token_accuracy(session, batches: int, seed: int = 314159) -> dict:
    if batches <= 0 or session.task is not None:
        return {}
    spec = session.spec
    objective = build_objective_runtime(spec, mask_token_id=session.cfg.mask_token_id, seed=seed,
                                        vocab_size=session.cfg.vocab_size, device=session.device)
    saved = session.objective
    session.objective = objective
    correct = torch.zeros((), dtype=torch.float64, device=session.device)
    total = torch.zeros_like(correct)
    loss_sum = torch.zeros_like(correct)
    try:
        for _ in range(batches):
            batch = session.data.next_batch()
            cb = objective.corrupt(batch.input_ids, supervision_mask=batch.supervision_mask)
            tokens, labels, weights = session.assemble_rows(cb)
            hidden = session.model(tokens, session.layout.positions, session.attend)
            h, l, w, _ = compact_supervised_rows(hidden, labels, weights)
            if session.model.tp is None:
                logits = h.float() @ session.model.lm_head.float().t()
                if objective.exclude_mask_token:
                    logits[:, session.cfg.mask_token_id] = float("-inf")
                correct += (logits.argmax(-1) == l).sum()
            ls, _ = session.model.loss(h, l, None, objective.exclude_mask_token)
            loss_sum += ls.double()
            total += l.numel()
    finally:
        session.objective = saved
    if dist.is_initialized() and dist.get_world_size() > 1:
        for t in (correct, total, loss_sum):
            dist.all_reduce(t)
    n = max(float(total), 1.0)
    return {"eval_masked_tokens": float(total), "eval_masked_token_accuracy": float(correct) / n,
            "eval_loss": float(loss_sum) / n}
