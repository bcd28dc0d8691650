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


_DESCRIPTIONS = {
    "causal_lm": "dense causal LMs (Qwen3 and alike) converted to block diffusion",
    "dflash": "DFlash / DFlash2 speculative drafters distilled from a frozen verifier",
    "diffusion_gemma": "DiffusionGemma-style decoders, dense or with routed experts",
    "nemotron_labs_diffusion": "Nemotron-Labs-Diffusion block-diffusion decoders",
    "qwen3_8": "hybrid Gated DeltaNet + gated softmax attention decoders",
}
_EXECUTORS: dict[str, object] = {}


def register_executor(family: str, executor) -> None:
    """Adds (or replaces) the executor of a family: the extension point for new model families."""
    _EXECUTORS[family] = executor
    if family not in FAMILY_OBJECTIVES:
        FAMILY_OBJECTIVES[family] = tuple(executor.family.objectives)


def executor_for_family(family: str):
    """The `BackboneExecutor` that builds, validates and describes models of `family`."""
    if family not in _EXECUTORS:
        from . import contracts as c

        if family not in FAMILY_OBJECTIVES:
            raise ValueError(f"unknown model family {family!r}; known: {', '.join(FAMILY_OBJECTIVES)}")
        spec = c.ModelFamilySpec(family, FAMILY_OBJECTIVES[family], _DESCRIPTIONS.get(family, ""))
        cls = {"causal_lm": c.DenseExecutor, "nemotron_labs_diffusion": c.DenseExecutor,
               "diffusion_gemma": c.MoEExecutor, "qwen3_8": c.HybridExecutor, "dflash": c.DFlashExecutor}[family]
        _EXECUTORS[family] = cls(spec)
    return _EXECUTORS[family]


def family_of_config(cfg, spec) -> str:
    """Family of a resolved model config: the spec's explicit family, else what the config and objective imply."""
    fam = spec.model.family
    if fam not in ("auto", "hf"):
        return fam
    if spec.objective.name == "dflash_distillation":
        return "dflash"
    if getattr(cfg, "is_hybrid", False):
        return "qwen3_8"
    if getattr(cfg, "is_moe", False):
        return "diffusion_gemma"
    return getattr(cfg, "family", None) or infer_family(spec.model.id, spec.objective.name)


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
    """Families with their objectives and what each family's executor can run (parallel axes, parameter sharding,
    adapters, attention head widths): what `dllm-train --print-supported-configs` prints."""
    from dataclasses import asdict

    fams = {}
    for f, o in FAMILY_OBJECTIVES.items():
        caps = asdict(executor_for_family(f).capabilities)
        caps["head_dims"] = list(caps.get("head_dims", ()))
        fams[f] = {"objectives": list(o), "capabilities": caps}
    return {"families": fams,
            "optimizer_backends": list(OPTIMIZER_BACKENDS),
            "dtypes": ["bf16", "fp16", "fp32"],
            "parallel_axes": ["data", "context", "block", "tensor", "expert", "pipeline (size 1 only)"]}
