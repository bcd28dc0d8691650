"""Model families, the objectives each supports, and optimizer backends.

Counterparts: dllm_parallel/core/models/registry.py:18-58 (families, optimizer backends), :123-156
(executor_for_family / infer_family) and dllm_parallel/core/models/compatibility.py:9-41
(family × objective allow-list).
"""
from __future__ import annotations

from ..config.schema import FAMILIES, OPTIMIZER_BACKENDS

FAMILY_OBJECTIVES: dict[str, tuple[str, ...]] = {
    "causal_lm": ("fast_dllm_v2", "standard_block_diffusion"),
    "dflash": ("dflash_distillation",),
    "diffusion_gemma": ("diffusiongemma_native_sft", "standard_block_diffusion"),
    "nemotron_labs_diffusion": ("standard_block_diffusion",),
    "qwen3_8": ("fast_dllm_v2",),
}


def supported_families() -> tuple[str, ...]:
    return FAMILIES


def objectives_for_family(family: str) -> tuple[str, ...]:
    if family not in FAMILY_OBJECTIVES:
        raise ValueError(f"unknown model family {family!r}; known: {', '.join(FAMILIES)}")
    return FAMILY_OBJECTIVES[family]


def infer_family(model_id: str, objective: str | None = None, architectures: tuple[str, ...] = ()) -> str:
    """Family from a preset id, HF architecture names, or the objective as a last resort."""
    mid = model_id.lower()
    archs = " ".join(architectures).lower()
    if "dflash" in mid or "dflash" in archs or objective == "dflash_distillation":
        return "dflash"
    if "gemma" in mid or "moe" in mid or "gemma" in archs:
        return "diffusion_gemma"
    if "nemotron" in mid or "nemotron" in archs:
        return "nemotron_labs_diffusion"
    if "qwen3.8" in mid or "qwen3_8" in mid or "deltanet" in archs:
        return "qwen3_8"
    return "causal_lm"


def describe_supported_configs() -> dict:
    return {"families": {f: {"objectives": list(o)} for f, o in FAMILY_OBJECTIVES.items()},
            "optimizer_backends": list(OPTIMIZER_BACKENDS),
            "dtypes": ["bf16", "fp16", "fp32"],
            "parallel_axes": ["data", "context", "block", "tensor", "expert", "pipeline (size 1 only)"]}
