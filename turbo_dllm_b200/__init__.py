"""turbo_dllm_b200: a B200-native (sm_100a) training framework for block-diffusion language
models and diffusion speculative drafters.

Public surface mirrors the reference package export list
(dllm_parallel/__init__.py:12-50): RunSpec, load_run_spec, train, the parallel specs and the
objective descriptors. Heavy modules are imported lazily so `import turbo_dllm_b200` stays cheap.
"""
from __future__ import annotations

__version__ = "0.2.0"

_LAZY = {
    "RunSpec": ("turbo_dllm_b200.config.run_spec", "RunSpec"),
    "load_run_spec": ("turbo_dllm_b200.config.run_spec", "load_run_spec"),
    "train": ("turbo_dllm_b200.training.trainer", "train"),
    "CPBPPolicy": ("turbo_dllm_b200.parallel.specs", "CPBPPolicy"),
    "ParallelSpec": ("turbo_dllm_b200.parallel.specs", "ParallelSpec"),
    "BlockDiffusionObjective": ("turbo_dllm_b200.parallel.specs", "BlockDiffusionObjective"),
    "DiffusionSchedule": ("turbo_dllm_b200.parallel.specs", "DiffusionSchedule"),
    "AttentionPlan": ("turbo_dllm_b200.parallel.specs", "AttentionPlan"),
    "LossRegion": ("turbo_dllm_b200.parallel.specs", "LossRegion"),
    "SequenceRegion": ("turbo_dllm_b200.parallel.specs", "SequenceRegion"),
    "build_parallel_plan": ("turbo_dllm_b200.parallel.topology", "build_parallel_plan"),
    "build_block_schedule": ("turbo_dllm_b200.parallel.schedule", "build_block_schedule"),
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'turbo_dllm_b200' has no attribute {name!r}")


__all__ = sorted(_LAZY) + ["__version__"]
