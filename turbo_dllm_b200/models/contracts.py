"""What a model family has to provide to be trained by this framework.

`TrainingSession` and the trainer never branch on a family name: they ask the family's `BackboneExecutor`
(found through `registry.executor_for_family`) for its capabilities, let it validate the run spec, build the
model, name the units its parameters may be sharded by, pick the data runtime and report the work units the
parallel planner balances. Adding a family means adding an executor and registering it.

Counterpart of the reference's contracts (dllm_parallel/core/models/contracts.py:20-219: ModelFamilySpec,
BackboneCapabilities, BackboneKernelPolicy, BackboneExecutor).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol, runtime_checkable

import torch


@dataclass(frozen=True)
class ModelFamilySpec:
    name: str
    objectives: tuple[str, ...]
    description: str = ""
    hf_architectures: tuple[str, ...] = ()


@dataclass(frozen=True)
class BackboneCapabilities:
    tensor_parallel: bool = False
    sequence_parallel: bool = False
    expert_parallel: bool = False
    context_parallel: bool = True
    block_parallel: bool = True
    parameter_sharding: bool = False       # optimizer.backend: fsdp
    lora: bool = False
    activation_offload: bool = True
    # head sizes the sm_100a attention covers for this family: 128 in one kernel; 64, 256 and 512 as tensor-core
    # products around the masked-softmax kernels (ops/wide_attention.py)
    head_dims: tuple[int, ...] = (64, 128, 256, 512)


@dataclass(frozen=True)
class BackboneKernelPolicy:
    """Which native kernels the family's hot path needs on a CUDA device (checked by `verify_native_kernels`)."""
    required_symbols: tuple[str, ...] = ("tdllm_gemm_bf16", "tdllm_attn_fwd", "tdllm_attn_bwd_fused",
                                         "tdllm_rmsnorm_fwd", "tdllm_adamw")
    optional_symbols: tuple[str, ...] = ()


@dataclass
class BuildContext:
    """Everything an executor may need to build its model for one rank."""
    spec: Any
    cfg: Any
    device: torch.device
    dtype: torch.dtype
    runtime: Any = None
    seed: int = 0
    activation_offload: bool = False
    extras: dict = field(default_factory=dict)


@runtime_checkable
class BackboneExecutor(Protocol):
    family: ModelFamilySpec
    capabilities: BackboneCapabilities
    kernel_policy: BackboneKernelPolicy

    def validate_run_spec(self, spec, world_size: int | None = None) -> list[str]: ...
    def build_model(self, ctx: BuildContext): ...
    def parameter_shard_units(self, model) -> list[str]: ...
    def build_data_runtime(self, spec, cfg, device, dp_rank: int, dp_size: int, host_staged: bool = False): ...
    def parallel_work_units(self, spec) -> int: ...
    def verify_native_kernels(self) -> list[str]: ...
    def checkpoint_state(self, model) -> dict: ...


class _ExecutorBase:
    family: ModelFamilySpec
    capabilities = BackboneCapabilities()
    kernel_policy = BackboneKernelPolicy()

    # ---- validation -------------------------------------------------------------------------------------
    def validate_run_spec(self, spec, world_size: int | None = None) -> list[str]:
        """Family-specific problems with a run spec (empty = fine); generic rules live in `RunSpec.validate`."""
        t, caps, out = spec.topology, self.capabilities, []
        if spec.objective.name not in self.family.objectives:
            out.append(f"objective {spec.objective.name} is not supported by family {self.family.name} "
                       f"(supported: {', '.join(self.family.objectives)})")
        if t.tensor_parallel_size > 1 and not caps.tensor_parallel:
            out.append(f"family {self.family.name} does not run tensor-parallel")
        if t.sequence_parallel and not caps.sequence_parallel:
            out.append(f"family {self.family.name} does not run sequence-parallel")
        if t.expert_parallel_size > 1 and not caps.expert_parallel:
            out.append(f"family {self.family.name} has no experts to distribute")
        if spec.optimizer.backend in ("fsdp", "fsdp2") and not caps.parameter_sharding:
            out.append(f"optimizer.backend={spec.optimizer.backend} is not built for family {self.family.name}")
        if spec.adapter.type == "lora" and not caps.lora:
            out.append(f"LoRA adapters are not built for family {self.family.name}")
        return out

    # ---- data ---------------------------------------------------------------------------------------------
    def build_data_runtime(self, spec, cfg, device, dp_rank: int, dp_size: int, host_staged: bool = False):
        from ..data.runtimes import HostStagedRandomRuntime, RandomTokenDataRuntime

        kw = dict(batch_size=spec.training.batch_size, seq_len=spec.model.seq_len, vocab_size=cfg.vocab_size,
                  mask_token_id=cfg.mask_token_id, seed=spec.launch.seed + 104729 * (dp_rank + 1),
                  vocab_sample_size=spec.data.vocab_sample_size)
        if spec.data.input_mode == "random":
            return (HostStagedRandomRuntime if host_staged else RandomTokenDataRuntime)(device=device, **kw)
        from ..data.artifact_runtimes import build_artifact_runtime

        return build_artifact_runtime(spec, device=device, dp_rank=dp_rank, dp_size=dp_size)

    # ---- planner / kernels / checkpoints --------------------------------------------------------------------
    def parallel_work_units(self, spec) -> int:
        """Units the block-parallel schedule distributes: diffusion blocks of one sequence."""
        return spec.model.seq_len // spec.objective.block_size

    def parameter_shard_units(self, model) -> list[str]:
        from ..parallel.fsdp import plan_units

        return [u.name for u in plan_units(model.flat, 1)]

    def verify_native_kernels(self) -> list[str]:
        """Missing symbols of the native library (empty = ready). Only meaningful where the library is built."""
        from ..kernels import native

        try:
            lib = native.lib()
        except Exception as e:
            return [f"native library unavailable: {e}"]
        return [s for s in self.kernel_policy.required_symbols if not hasattr(lib, s)]

    def checkpoint_state(self, model) -> dict:
        return {"family": self.family.name}


class DenseExecutor(_ExecutorBase):
    """Qwen3-style dense decoders: generic causal LMs converted with Fast-dLLM v2 and Nemotron-style
    block-diffusion models (dllm_parallel/core/models/backbones/causal_lm/executor.py:76-249)."""

    capabilities = BackboneCapabilities(tensor_parallel=True, sequence_parallel=True, parameter_sharding=True,
                                        lora=True)

    def __init__(self, family: ModelFamilySpec):
        self.family = family

    def build_model(self, ctx: BuildContext):
        from ..parallel.tensor_parallel import TPContext
        from .dense import BlockDiffusionTransformer

        rt, spec = ctx.runtime, ctx.spec
        tp = None
        if rt is not None and rt.tensor_parallel_size > 1:
            tp = TPContext(rt.tensor_group, spec.topology.sequence_parallel)
            if not spec.topology.tensor_parallel_overlap:
                # projections and their collectives as separate steps (GEMM + NCCL) instead of the fused kernels
                tp.fused_allreduce_enabled = False
                tp.fused_sequence_parallel_enabled = False
        model = BlockDiffusionTransformer(ctx.cfg, dtype=ctx.dtype, device=ctx.device,
                                          activation_checkpointing=spec.training.activation_checkpointing,
                                          activation_offload=ctx.activation_offload, seed=ctx.seed, tp=tp)
        for layer in model.layers:
            layer.mlp_token_chunk = int(spec.kernel.mlp_token_chunk_size)
        model.checkpoint_scope = str(spec.training.activation_checkpointing_scope)
        return model


class MoEExecutor(_ExecutorBase):
    """DiffusionGemma-style routed experts (dllm_parallel/core/models/backbones/diffusiongemma/model.py:33-460)."""

    capabilities = BackboneCapabilities(expert_parallel=True, tensor_parallel=True, sequence_parallel=True, lora=True,
                                        parameter_sharding=True)
    kernel_policy = BackboneKernelPolicy(optional_symbols=("tdllm_gemm_grouped_bf16", "tdllm_ep_dispatch"))

    def __init__(self, family: ModelFamilySpec):
        self.family = family

    def build_model(self, ctx: BuildContext):
        from .dense import BlockDiffusionTransformer
        from .moe import MoEBlockDiffusionTransformer

        from ..parallel.tensor_parallel import TPContext

        rt, spec = ctx.runtime, ctx.spec
        tp = None
        if rt is not None and rt.tensor_parallel_size > 1:
            tp = TPContext(rt.tensor_group, spec.topology.sequence_parallel)
            if not spec.topology.tensor_parallel_overlap:
                tp.fused_allreduce_enabled = False
                tp.fused_sequence_parallel_enabled = False
        if not ctx.cfg.is_moe:     # the family's dense checkpoints use the dense decoder
            return BlockDiffusionTransformer(ctx.cfg, dtype=ctx.dtype, device=ctx.device,
                                             activation_checkpointing=spec.training.activation_checkpointing,
                                             activation_offload=ctx.activation_offload, seed=ctx.seed, tp=tp)
        ep = rt.expert_parallel_size if rt is not None else 1
        return MoEBlockDiffusionTransformer(ctx.cfg, ep_group=rt.group("expert") if ep > 1 else None,
                                            dtype=ctx.dtype, device=ctx.device,
                                            activation_checkpointing=spec.training.activation_checkpointing,
                                            activation_offload=ctx.activation_offload, seed=ctx.seed, tp=tp)


class HybridExecutor(_ExecutorBase):
    """Gated DeltaNet + gated softmax attention (dllm_parallel/core/models/backbones/qwen3_8/executor.py:192-413)."""

    capabilities = BackboneCapabilities(tensor_parallel=True, sequence_parallel=True, lora=True, parameter_sharding=True,
                                        head_dims=(128,))
    kernel_policy = BackboneKernelPolicy(optional_symbols=("tdllm_gdn_scan_fwd", "tdllm_gdn_scan_bwd"))

    def __init__(self, family: ModelFamilySpec):
        self.family = family

    def validate_run_spec(self, spec, world_size: int | None = None) -> list[str]:
        out = super().validate_run_spec(spec, world_size)
        return out

    def build_model(self, ctx: BuildContext):
        from ..parallel.tensor_parallel import TPContext
        from .hybrid import HybridBlockDiffusionTransformer

        rt = ctx.runtime
        tp = None
        if rt is not None and rt.tensor_parallel_size > 1:
            tp = TPContext(rt.tensor_group, ctx.spec.topology.sequence_parallel)
            if not ctx.spec.topology.tensor_parallel_overlap:
                tp.fused_allreduce_enabled = False
                tp.fused_sequence_parallel_enabled = False
        return HybridBlockDiffusionTransformer(ctx.cfg, dtype=ctx.dtype, device=ctx.device,
                                               activation_checkpointing=ctx.spec.training.activation_checkpointing,
                                               activation_offload=ctx.activation_offload, seed=ctx.seed, tp=tp)


class DFlashExecutor(_ExecutorBase):
    """Diffusion speculative drafters trained against a frozen verifier
    (dllm_parallel/core/models/backbones/dflash/executor.py:36-408). The model comes with its task: the session
    builds `training.dflash_task.DFlashTask`, which owns the drafter, the verifier and the objective."""

    # (context / block parallelism here means one drafter replica over several ranks: context rows and anchors divided)
    capabilities = BackboneCapabilities(context_parallel=True, block_parallel=True)

    def __init__(self, family: ModelFamilySpec):
        self.family = family

    def build_model(self, ctx: BuildContext):
        from ..training.dflash_task import DFlashTask

        dp_rank = ctx.extras.get("dp_rank", 0)
        return DFlashTask(ctx.spec, ctx.cfg, dtype=ctx.dtype, device=ctx.device, seed=ctx.seed, dp_rank=dp_rank)

    def parallel_work_units(self, spec) -> int:
        return max(int(spec.objective.max_anchors or 1), 1)
