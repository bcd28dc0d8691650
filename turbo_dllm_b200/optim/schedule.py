"""Learning-rate and weight-decay schedules driven by the run spec.

constant / linear / cosine / inverse_square_root with linear warm-up, plus a constant / linear /
cosine weight-decay schedule; resumable through state_dict.
Counterpart of RunSpecLRScheduler (dllm_parallel/training/optimizer_setup.py:22-220).
"""
from __future__ import annotations

import math


class RunSpecLRScheduler:
    def __init__(self, *, base_lr: float, scheduler_type: str = "constant", warmup_steps: int = 0,
                 decay_steps: int | None = None, min_lr: float = 0.0, total_steps: int | None = None,
                 weight_decay: float = 0.0, weight_decay_style: str = "constant",
                 weight_decay_start: float | None = None, weight_decay_end: float | None = None,
                 weight_decay_steps: int | None = None):
        if scheduler_type not in ("constant", "linear", "cosine", "inverse_square_root"):
            raise ValueError(f"unknown scheduler type {scheduler_type!r}")
        if weight_decay_style not in ("constant", "linear", "cosine"):
            raise ValueError(f"unknown weight decay style {weight_decay_style!r}")
        self.base_lr, self.kind, self.warmup = float(base_lr), scheduler_type, int(warmup_steps)
        self.decay_steps = int(decay_steps) if decay_steps is not None else (total_steps or 0)
        self.min_lr = float(min_lr)
        self.wd, self.wd_style = float(weight_decay), weight_decay_style
        self.wd_start = self.wd if weight_decay_start is None else float(weight_decay_start)
        self.wd_end = self.wd if weight_decay_end is None else float(weight_decay_end)
        self.wd_steps = int(weight_decay_steps) if weight_decay_steps is not None else self.decay_steps
        self.step_count = 0

    @classmethod
    def from_run_spec(cls, spec) -> "RunSpecLRScheduler":
        s, o = spec.scheduler, spec.optimizer
        return cls(base_lr=o.lr, scheduler_type=s.type, warmup_steps=s.warmup_steps, decay_steps=s.decay_steps,
                   min_lr=s.min_lr, total_steps=spec.training.steps, weight_decay=o.weight_decay,
                   weight_decay_style=s.weight_decay_style, weight_decay_start=s.weight_decay_start,
                   weight_decay_end=s.weight_decay_end, weight_decay_steps=s.weight_decay_steps)

    def lr_at(self, step: int) -> float:
        """Learning rate used by optimizer step number `step` (1-based)."""
        if self.warmup > 0 and step <= self.warmup:
            return self.base_lr * step / self.warmup
        if self.kind == "constant":
            return self.base_lr
        if self.kind == "inverse_square_root":
            return max(self.min_lr, self.base_lr * math.sqrt(max(self.warmup, 1) / max(step, 1)))
        span = max(self.decay_steps - self.warmup, 1)
        frac = min(max(step - self.warmup, 0) / span, 1.0)
        if self.kind == "linear":
            coeff = 1.0 - frac
        else:
            coeff = 0.5 * (1.0 + math.cos(math.pi * frac))
        return self.min_lr + (self.base_lr - self.min_lr) * coeff

    def wd_at(self, step: int) -> float:
        if self.wd_style == "constant" or self.wd_steps <= 0:
            return self.wd if self.wd_style == "constant" else self.wd_end
        frac = min(max(step, 0) / self.wd_steps, 1.0)
        coeff = frac if self.wd_style == "linear" else 0.5 * (1.0 - math.cos(math.pi * frac))
        return self.wd_start + (self.wd_end - self.wd_start) * coeff

    def step(self) -> tuple[float, float]:
        self.step_count += 1
        return self.lr_at(self.step_count), self.wd_at(self.step_count)

    def state_dict(self) -> dict:
        return {"step_count": self.step_count, "base_lr": self.base_lr, "kind": self.kind}

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(state["step_count"])
