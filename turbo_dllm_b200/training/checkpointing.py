"""Checkpoint policy: where to resume from and when to save.

Explicit `load_checkpoint_dir` wins; `auto_resume` picks the newest COMPLETE checkpoint of the
save directory (metadata.json is published last, so its presence means every rank shard exists).
Saves trigger on the step interval, on the first / final step, and when elapsed time crosses a
configured fraction of `training.max_duration_seconds`.

Counterpart of dllm_parallel/training/checkpointing.py:19-88.
"""
from __future__ import annotations

import json
import os

_fraction_state: dict[str, set] = {}


def resolve_load_checkpoint(spec) -> tuple[str | None, str]:
    ck = spec.checkpointing
    if ck.load_checkpoint_dir:
        return ck.load_checkpoint_dir, ck.checkpoint_tag
    if ck.auto_resume and ck.save_checkpoint_dir:
        meta = os.path.join(ck.save_checkpoint_dir, "metadata.json")
        if os.path.exists(meta):
            try:
                data = json.load(open(meta))
            except (OSError, ValueError):
                return None, ck.checkpoint_tag
            tag = data.get("latest_tag")
            if tag and os.path.isdir(os.path.join(ck.save_checkpoint_dir, tag)):
                return ck.save_checkpoint_dir, "latest"
    return None, ck.checkpoint_tag


def should_save(spec, step: int, total_steps: int, elapsed_seconds: float) -> bool:
    ck = spec.checkpointing
    if not ck.save_checkpoint_dir:
        return False
    if ck.save_first_step and step == 1:
        return True
    if ck.save_final and step == total_steps:
        return True
    if ck.save_checkpoint_interval and step % ck.save_checkpoint_interval == 0:
        return True
    limit = spec.training.max_duration_seconds
    if limit and ck.save_duration_fractions:
        done = _fraction_state.setdefault(ck.save_checkpoint_dir, set())
        for frac in sorted(ck.save_duration_fractions):
            if frac not in done and elapsed_seconds >= frac * limit:
                done.add(frac)
                return True
    return False


def duration_tag(fraction: float, step: int) -> str:
    return f"duration_{int(round(fraction * 100)):03d}pct_step_{step:08d}"


def step_tag(step: int) -> str:
    return f"step_{step:08d}"
