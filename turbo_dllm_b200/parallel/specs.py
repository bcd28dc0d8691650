"""Frozen descriptors of the parallel / objective contract shared by planner, runtime and models.

Names and meanings follow dllm_parallel/core/specs.py:54-176 (CPBPPolicy, ParallelSpec,
BlockDiffusionObjective, DiffusionSchedule, AttentionPlan, LossRegion, SequenceRegion).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class CPBPPolicy:
    """How clean K/V are laid out over context-parallel ranks and how they travel.

    clean_kv_layout: "zigzag" (dual-chunk: rank r owns chunks r and 2P-1-r) or "contiguous".
    clean_kv_transport: "collective" (all-gather / reduce-scatter), "streaming" (step-wise
    exchange with online-softmax merge) or "peer_pull" (kernels read peers' K/V over NVLink).
    """

    clean_kv_layout: str = "zigzag"
    clean_kv_transport: str = "collective"
    transport_dtype: str = "bf16"

    def __post_init__(self):
        if self.clean_kv_layout not in ("zigzag", "contiguous"):
            raise ValueError(f"unknown clean_kv_layout {self.clean_kv_layout!r}")
        if self.clean_kv_transport not in ("collective", "streaming", "peer_pull", "fused"):
            raise ValueError(f"unknown clean_kv_transport {self.clean_kv_transport!r}")


@dataclass(frozen=True)
class ParallelSpec:
    data_parallel_size: int = 1
    context_parallel_size: int = 1
    block_parallel_size: int = 1
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    sequence_parallel: bool = False
    replicate_clean_prefix: bool = False
    policy: CPBPPolicy = CPBPPolicy()

    def __post_init__(self):
        cp, bp = self.context_parallel_size, self.block_parallel_size
        for n in (self.data_parallel_size, cp, bp, self.tensor_parallel_size,
                  self.expert_parallel_size, self.pipeline_parallel_size):
            if n < 1:
                raise ValueError("parallel sizes must be >= 1")
        if cp > 1 and bp > 1 and (bp < cp or bp % cp):
            raise ValueError(f"fused CP+BP needs BP ({bp}) to be a multiple of CP ({cp})")

    @property
    def local_parallel_size(self) -> int:
        return max(self.context_parallel_size, self.block_parallel_size)

    @property
    def model_parallel_size(self) -> int:
        return (self.local_parallel_size * self.tensor_parallel_size * self.expert_parallel_size
                * self.pipeline_parallel_size)

    @property
    def world_size(self) -> int:
        return self.data_parallel_size * self.model_parallel_size

    @property
    def fused_cp_bp(self) -> bool:
        return self.context_parallel_size > 1 and self.block_parallel_size > 1


@dataclass(frozen=True)
class DiffusionSchedule:
    name: str = "loglinear"
    epsilon: float = 1e-3
    sampling_epsilon_min: float = 1e-3
    sampling_epsilon_max: float = 1.0
    antithetic: bool = True


@dataclass(frozen=True)
class BlockDiffusionObjective:
    name: str = "standard_block_diffusion"
    block_size: int = 32
    loss_weighting: str = "inverse_move_chance"
    schedule: DiffusionSchedule = DiffusionSchedule()

    @property
    def supports_fused_cp_bp(self) -> bool:
        # objectives whose noisy blocks only look at the clean prefix can hand whole blocks to ranks
        return self.name in ("standard_block_diffusion", "fast_dllm_v2", "diffusiongemma_native_sft",
                             "dflash_distillation")


@dataclass(frozen=True)
class SequenceRegion:
    """Half-open token range [start, stop) of the logical [noisy ; clean] 2L sequence."""

    start: int
    stop: int
    kind: str = "noisy"  # "noisy" | "clean"

    def __post_init__(self):
        if self.stop < self.start:
            raise ValueError("SequenceRegion stop < start")

    @property
    def length(self) -> int:
        return self.stop - self.start


@dataclass(frozen=True)
class LossRegion:
    """Rows that contribute to the loss and how they are normalised."""

    region: SequenceRegion
    reduction: str = "token_mean"
    scale: float = 1.0


@dataclass(frozen=True)
class AttentionPlan:
    kv_backend: str = "replicated"      # "replicated" | "ring" (context-sharded K/V)
    active_block_mode: str = "all_blocks"  # "all_blocks" | "dual_end"
    policy: CPBPPolicy = CPBPPolicy()
