"""SystemTrace: a bounded window of optimizer steps traced on every rank.

Configured by the `profiler` section of the run spec. At `system_trace_start_step` every rank
synchronises, then either starts a Kineto profile (CPU + CUDA activities, exported as
`rank_{r}.trace.json.gz`) or brackets the window with cudaProfilerStart/Stop for an external nsys
capture. Inside the window each step is a `dllm.step.N` range and each phase a `dllm.phase.*`
range (zero_grad, data, forward, loss, backward, gradient_sync, gradient_clip, optimizer).

Counterpart of dllm_parallel/core/profiling/system_trace.py:27-158.
"""
from __future__ import annotations

import contextlib
import os

from .operator_trace import BACKEND_ENV

PHASES = ("zero_grad", "data", "forward", "loss", "backward", "gradient_sync", "gradient_clip", "optimizer")


class SystemTrace:
    def __init__(self, *, enabled: bool, backend: str = "kineto", directory: str | None = None, start_step: int = 1,
                 steps: int = 1, rank: int = 0, barrier=None):
        if backend not in ("kineto", "nsys"):
            raise ValueError(f"unknown system trace backend {backend!r}")
        self.enabled, self.backend = bool(enabled), backend
        self.directory = directory or os.path.join(os.environ.get("DLLM_RUN_DIR", "."), "system_trace")
        self.start_step, self.steps, self.rank = int(start_step), int(steps), int(rank)
        self.barrier = barrier
        self.active = False
        self._prof = None
        self._step_ctx = None
        self.exported: str | None = None

    @classmethod
    def from_run_spec(cls, spec, rank: int, barrier=None) -> "SystemTrace":
        p = spec.profiler
        return cls(enabled=p.system_trace, backend=p.system_trace_backend, directory=p.system_trace_dir,
                   start_step=p.system_trace_start_step, steps=p.system_trace_steps, rank=rank, barrier=barrier)

    def _sync(self):
        import torch

        if self.barrier is not None:
            self.barrier()
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def begin_step(self, step: int) -> None:
        if not self.enabled:
            return
        import torch

        if step == self.start_step and not self.active:
            self._sync()
            os.environ[BACKEND_ENV] = self.backend
            os.makedirs(self.directory, exist_ok=True)
            if self.backend == "kineto":
                acts = [torch.profiler.ProfilerActivity.CPU]
                if torch.cuda.is_available():
                    acts.append(torch.profiler.ProfilerActivity.CUDA)
                self._prof = torch.profiler.profile(activities=acts, acc_events=True)
                self._prof.__enter__()
            elif torch.cuda.is_available():
                torch.cuda.cudart().cudaProfilerStart()
            self.active = True
        if self.active:
            self._step_ctx = self._range(f"dllm.step.{step}")
            self._step_ctx.__enter__()

    def _range(self, label: str):
        import torch

        if self.backend == "nsys" and torch.cuda.is_available():
            return torch.cuda.nvtx.range(label)
        return torch.profiler.record_function(label)

    def phase(self, name: str):
        if not self.active:
            return contextlib.nullcontext()
        if name not in PHASES:
            raise ValueError(f"unknown phase {name!r}")
        return self._range(f"dllm.phase.{name}")

    def end_step(self, step: int) -> None:
        if not self.active:
            return
        import torch

        if self._step_ctx is not None:
            self._step_ctx.__exit__(None, None, None)
            self._step_ctx = None
        if step >= self.start_step + self.steps - 1:
            self._sync()
            if self.backend == "kineto" and self._prof is not None:
                self._prof.__exit__(None, None, None)
                self.exported = os.path.join(self.directory, f"rank_{self.rank}.trace.json.gz")
                self._prof.export_chrome_trace(self.exported)
                self._prof = None
            elif torch.cuda.is_available():
                torch.cuda.cudart().cudaProfilerStop()
            os.environ.pop(BACKEND_ENV, None)
            self.active = False
            self.enabled = False


class PhaseTimer:
    """Host-side milliseconds per step phase (`profiler.phase_timing`), reported as `phase_ms` in step events.
    With `phase_timing_sync` the device is synchronised at both ends of every phase, so the figures are
    device-inclusive (and the step slower); without it they show where the host spends its time while the
    device runs behind. Each phase also opens the trace's `dllm.phase.*` range when a trace window is open.
    Counterpart of the phase bookkeeping in dllm_parallel/training/block_diffusion_trainer.py:1292-1536."""

    def __init__(self, device=None):
        self.device = device
        self.enabled = False
        self.sync = False
        self.ms: dict[str, float] = {}

    def configure(self, enabled: bool, sync: bool = False) -> None:
        self.enabled, self.sync = bool(enabled), bool(sync)

    def _device_sync(self) -> None:
        if self.sync and self.device is not None and getattr(self.device, "type", "cpu") == "cuda":
            import torch

            torch.cuda.synchronize(self.device)

    @contextlib.contextmanager
    def phase(self, name: str, trace: "SystemTrace | None" = None):
        if name not in PHASES:
            raise ValueError(f"unknown phase {name!r}")
        ctx = trace.phase(name) if trace is not None else contextlib.nullcontext()
        if not self.enabled:
            with ctx:
                yield
            return
        import time

        self._device_sync()
        t0 = time.perf_counter()
        try:
            with ctx:
                yield
        finally:
            self._device_sync()
            self.ms[name] = self.ms.get(name, 0.0) + (time.perf_counter() - t0) * 1e3

    def take(self) -> dict[str, float]:
        out, self.ms = {k: round(v, 3) for k, v in self.ms.items()}, {}
        return out
