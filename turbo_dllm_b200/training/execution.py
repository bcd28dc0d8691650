"""What the trainer needs to know about the distributed layout of a run, as one small protocol.

`execution_for(runtime, world)` adapts a `ParallelRuntime` (or its absence: single process / plain
data parallel) to that protocol, so that code which only needs ranks, group sizes and the active-block
mode does not reach into the runtime.

Counterpart of `DistributedExecution` (dllm_parallel/training/execution.py:13-52).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol


class DistributedExecution(Protocol):
    world_size: int
    data_parallel_size: int
    data_parallel_rank: int
    context_parallel_size: int
    block_parallel_size: int
    tensor_parallel_size: int
    expert_parallel_size: int

    @property
    def active_block_mode(self) -> str: ...


@dataclass(frozen=True)
class Execution:
    world_size: int = 1
    data_parallel_size: int = 1
    data_parallel_rank: int = 0
    context_parallel_size: int = 1
    block_parallel_size: int = 1
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1

    @property
    def active_block_mode(self) -> str:
        """Ranks of a block-parallel group train disjoint block sets chosen by the dual-end schedule;
        otherwise every rank trains all blocks of its sequences."""
        return "dual_end" if self.block_parallel_size > 1 else "all_blocks"


def execution_for(runtime, world_size: int = 1, rank: int = 0) -> Execution:
    if runtime is None:
        return Execution(world_size=world_size, data_parallel_size=world_size, data_parallel_rank=rank)
    return Execution(world_size=world_size,
                     data_parallel_size=runtime.data_parallel_size,
                     data_parallel_rank=getattr(runtime, "data_parallel_rank", 0),
                     context_parallel_size=runtime.context_parallel_size,
                     block_parallel_size=runtime.block_parallel_size,
                     tensor_parallel_size=runtime.tensor_parallel_size,
                     expert_parallel_size=getattr(runtime, "expert_parallel_size", 1))
