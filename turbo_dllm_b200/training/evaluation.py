"""Masked-token accuracy evaluation (no gradient, fixed seed) on `evaluation.dataset_path` when it is set, else on
the next batches of the training stream.

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
    data = session.data
    if spec.evaluation.dataset_path:
        # held-out data: `evaluation.dataset_path` (a prepared artifact, a flat token file or a text file), read with
        # the evaluation seed and sharded over the data-parallel ranks like the training data
        from ..data.artifact_runtimes import build_artifact_runtime

        held_out = spec.with_overrides({"data": {"input_mode": "dataset", "dataset_path": spec.evaluation.dataset_path,
                                                 "optimizer_step_unit": "microbatch"},
                                        "launch": {"seed": int(seed)}})
        data = build_artifact_runtime(held_out, device=session.device, dp_rank=getattr(session, "dp_rank", 0),
                                      dp_size=session.dp_size)
    saved = session.objective
    session.objective = objective
    correct = torch.zeros((), dtype=torch.float64, device=session.device)
    total = torch.zeros_like(correct)
    loss_sum = torch.zeros_like(correct)
    try:
        for _ in range(batches):
            batch = data.next_batch()
            cb = objective.corrupt(batch.input_ids, supervision_mask=batch.supervision_mask)
            tokens, labels, weights = session.assemble_rows(cb)
            hidden = session.model(tokens, session.layout.positions, session.attend)
            h, l, w, _ = compact_supervised_rows(hidden, labels, weights)
            tp = session.model.tp
            logits = h.float() @ session.model.lm_head.float().t()       # this rank's slice of the vocabulary under TP
            v0 = tp.vocab_range(session.cfg.vocab_size)[0] if tp is not None else 0
            if objective.exclude_mask_token and v0 <= session.cfg.mask_token_id < v0 + logits.shape[1]:
                logits[:, session.cfg.mask_token_id - v0] = float("-inf")
            best, arg = logits.max(-1) if logits.shape[0] else (logits.new_zeros(0), l.new_zeros(0))
            arg = arg + v0
            if tp is not None:
                # vocabulary-parallel argmax: the largest logit over the ranks, ties to the smallest token id
                top = best.clone()
                dist.all_reduce(top, op=dist.ReduceOp.MAX, group=tp.group)
                arg = torch.where(best == top, arg, torch.full_like(arg, session.cfg.vocab_size))
                dist.all_reduce(arg, op=dist.ReduceOp.MIN, group=tp.group)
            correct += (arg == l).sum()
            ls, _ = session.model.loss(h, l, None, objective.exclude_mask_token)
            loss_sum += ls.double()
            total += l.numel()
    finally:
        session.objective = saved
    if dist.is_initialized() and dist.get_world_size() > 1:
        for t in (correct, total, loss_sum):
            dist.all_reduce(t)
            if session.model.tp is not None:     # every tensor-parallel rank holds the same three numbers
                t /= session.model.tp.size
    n = max(float(total), 1.0)
    return {"eval_masked_tokens": float(total), "eval_masked_token_accuracy": float(correct) / n,
            "eval_loss": float(loss_sum) / n}
