"""Checkpoint policy: where to resume from and when to save.

Explicit `load_checkpoint_dir` wins; `auto_resume` picks the newest COMPLETE checkpoint of the
save directory (metadata.json is published last, so its presence means every rank shard exists).
Saves trigger on the step interval, on the first / final step, and when elapsed time crosses a
configured fraction of `training.max_duration_seconds`.

Time-based decisions ("a duration fraction is due", "the duration limit is reached") are taken by rank 0
from ITS clock and broadcast (`StepControl`), so every rank saves and stops on the same step; a rank that
acted on its own clock would enter the checkpoint barriers, or leave the loop, alone.

Counterpart of dllm_parallel/training/checkpointing.py:19-88 and the rank-0-driven duration control of
dllm_parallel/training/block_diffusion_trainer.py:1557-1570, :2971-3017.
"""
from __future__ import annotations

import json
import os

from dataclasses import dataclass


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


def step_due(spec, step: int, total_steps: int) -> bool:
    """Step-count triggers: identical on every rank by construction."""
    ck = spec.checkpointing
    if not ck.save_checkpoint_dir:
        return False
    if ck.save_first_step and step == 1:
        return True
    if ck.save_final and step == total_steps:
        return True
    return bool(ck.save_checkpoint_interval and step % ck.save_checkpoint_interval == 0)


@dataclass
class StepVerdict:
    save: bool            # write a checkpoint after this step
    tag: str | None       # its tag (None = the step tag)
    stop: bool            # leave the training loop after this step (duration limit reached)


class StepControl:
    """Per-run save/stop decisions shared by all ranks. `decide` must be called by every rank after
    every step; rank 0 evaluates the clock-dependent rules and the verdict is broadcast over
    `group` (the gloo control group; any group that contains every rank works)."""

    def __init__(self, spec, total_steps: int, *, rank: int = 0, world: int = 1, group=None, device=None,
                 clock=None):
        import time

        self.spec, self.total_steps = spec, total_steps
        self.rank, self.world, self.group, self.device = rank, world, group, device
        self.clock = clock or time.monotonic
        self.t0 = self.clock()
        self.saved_fractions: set[float] = set()

    def elapsed(self) -> float:
        return self.clock() - self.t0

    def _local(self, step: int) -> tuple[int, int, int]:
        """(save, fraction in percent or -1, stop) as seen by this rank's clock."""
        spec, ck = self.spec, self.spec.checkpointing
        save = step_due(spec, step, self.total_steps)
        pct, stop = -1, False
        limit = spec.training.max_duration_seconds
        if limit:
            el = self.elapsed()
            if ck.save_checkpoint_dir and ck.save_duration_fractions:
                due = [f for f in sorted(ck.save_duration_fractions) if f not in self.saved_fractions and el >= f * limit]
                if due:
                    pct = int(round(due[-1] * 100))
                    save = True
            if el >= limit:
                stop = True
                if ck.save_checkpoint_dir and ck.save_final:
                    save = True      # leaving on the duration limit counts as the final step
        return int(save), pct, int(stop)

    def decide(self, step: int) -> StepVerdict:
        import torch
        import torch.distributed as dist

        save, pct, stop = self._local(step) if self.rank == 0 or self.world == 1 else (0, -1, 0)
        if self.world > 1 and dist.is_initialized():
            gloo = self.group is not None and dist.get_backend(self.group) == "gloo"
            t = torch.tensor([save, pct, stop], dtype=torch.int64,
                             device="cpu" if gloo or self.device is None else self.device)
            src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
            dist.broadcast(t, src=src, group=self.group)
            save, pct, stop = (int(x) for x in t.tolist())
        tag = None
        if pct >= 0:
            limit = self.spec.training.max_duration_seconds or 0
            for f in self.spec.checkpointing.save_duration_fractions or ():
                if int(round(f * 100)) <= pct:
                    self.saved_fractions.add(f)     # every rank records what rank 0 decided
            if not step_due(self.spec, step, self.total_steps) and not stop:
                tag = duration_tag(pct / 100.0, step)
            del limit
        return StepVerdict(bool(save), tag, bool(stop))


def should_save(spec, step: int, total_steps: int, elapsed_seconds: float = 0.0) -> bool:
    """Single-rank convenience: step triggers only (time-based triggers go through StepControl)."""
    return step_due(spec, step, total_steps)


def duration_tag(fraction: float, step: int) -> str:
    return f"duration_{int(round(fraction * 100)):03d}pct_step_{step:08d}"


def step_tag(step: int) -> str:
    return f"step_{step:08d}"
