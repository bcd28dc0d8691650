"""Per-rank parallel runtime: sizes, ranks, groups and the helpers models use.

Built from the run spec and the world: plan (topology.py) → groups (groups.py) → runtime. Holds
the K/V backend choice (`ring` = context-sharded clean K/V, `replicated` otherwise), the active
block mode (`dual_end` when blocks are distributed), batch broadcast inside the model-input
group and the one-element warm-up collectives.

Counterpart of ParallelRuntime / build_parallel_runtime / warm_parallel_runtime_collectives
(dllm_parallel/core/parallel/runtime.py:72-247, :289-471, :474-519, :530-555).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .groups import ProcessGroupCollection, parse_group_timeouts
from .specs import CPBPPolicy
from .topology import ParallelPlan, RankAssignment, plan_from_run_spec


@dataclass
class ParallelRuntime:
    plan: ParallelPlan
    assignment: RankAssignment
    groups: ProcessGroupCollection
    policy: CPBPPolicy
    device: torch.device
    rank: int
    world_size: int
    share_clean_replicas: bool = True
    pure_cp_token_split: bool = True

    # sizes
    @property
    def data_parallel_size(self): return self.plan.data_parallel_size
    @property
    def context_parallel_size(self): return self.plan.context_parallel_size
    @property
    def block_parallel_size(self): return self.plan.block_parallel_size
    @property
    def tensor_parallel_size(self): return self.plan.tensor_parallel_size
    @property
    def expert_parallel_size(self): return self.plan.expert_parallel_size
    @property
    def local_parallel_size(self): return self.plan.local_parallel_size
    # ranks
    @property
    def data_parallel_rank(self): return self.assignment.data_parallel_rank
    @property
    def context_parallel_rank(self): return self.assignment.context_parallel_rank
    @property
    def block_parallel_rank(self): return self.assignment.block_parallel_rank
    @property
    def tensor_parallel_rank(self): return self.assignment.tensor_parallel_rank
    @property
    def expert_parallel_rank(self): return self.assignment.expert_parallel_rank
    @property
    def owned_blocks(self): return self.assignment.owned_blocks

    @property
    def sample_parallel_rank(self) -> int:
        """Index of the data shard this rank reads (EP ranks read different samples)."""
        return self.data_parallel_rank * self.expert_parallel_size + self.expert_parallel_rank

    @property
    def kv_backend(self) -> str:
        return "ring" if self.context_parallel_size > 1 else "replicated"

    @property
    def active_block_mode(self) -> str:
        return "dual_end" if self.block_parallel_size > 1 else "all_blocks"

    @property
    def uses_context_parallel_attention(self) -> bool:
        return self.context_parallel_size > 1

    @property
    def loss_scale(self) -> float:
        """Scale that makes a mean over ranks equal the global mean when each rank owns 1/BP of the
        blocks. This framework sums gradients and divides by the global denominator instead, so
        the value is informational (step events, checkpoints)."""
        return float(self.block_parallel_size) if self.active_block_mode == "dual_end" else 1.0

    # groups
    def group(self, axis: str):
        return self.groups.group(axis)

    @property
    def optimizer_group(self):
        return self.groups.group("optimizer_data_parallel")

    @property
    def splits_block_tokens(self) -> bool:
        """Context parallelism without block parallelism: the tokens INSIDE every noisy block are divided over the
        ranks (two-ended), noisy K/V travel with the clean K/V, and no noisy row is computed twice."""
        return self.pure_cp_token_split and self.context_parallel_size > 1 and self.block_parallel_size == 1

    @property
    def shares_clean_replicas(self) -> bool:
        """Blocks are spread over more ranks than the clean tokens (BP > CP > 1). The ranks that would hold a
        second copy of a clean shard hold no clean rows at all: every rank of the context/block axis pulls clean
        K/V from the CP shard owners and returns clean dK/dV to them, so the clean stream is computed once per
        shard. The reference computes it on the owner too and broadcasts tensors inside `clean_replica` groups
        (dllm_parallel/core/parallel/runtime.py:558-687); on NVSwitch any rank reaches any owner directly."""
        return (self.share_clean_replicas and self.context_parallel_size > 1
                and self.block_parallel_size > self.context_parallel_size)

    @property
    def owns_clean_shard(self) -> bool:
        return not self.shares_clean_replicas or self.assignment.local_parallel_rank < self.context_parallel_size

    @property
    def context_group(self):
        return self.groups.group("local_parallel" if self.shares_clean_replicas else "context_block_parallel")

    def context_members(self) -> list[tuple[int, int, bool]]:
        """(rank, clean shard index, owns that shard) of every member of `context_group`, in group order."""
        axis = "local_parallel" if self.shares_clean_replicas else "context_block_parallel"
        out = []
        for r in self.groups.ranks[axis]:
            a = self.plan.assignment(r)
            owns = not self.shares_clean_replicas or a.local_parallel_rank < self.context_parallel_size
            out.append((r, a.context_parallel_rank, owns))
        return out

    @property
    def tensor_group(self):
        return self.groups.group("tensor")

    def broadcast_batch(self, tensor: torch.Tensor) -> torch.Tensor:
        """All ranks of one model replica must see the same token batch."""
        ranks = self.groups.ranks["model_input"]
        if len(ranks) > 1:
            dist.broadcast(tensor, src=ranks[0], group=self.groups.group("model_input"))
        return tensor

    def warm_collectives(self) -> None:
        """One tiny all-reduce per group so communicator set-up is not billed to step 1."""
        if not dist.is_initialized():
            return
        t = torch.ones(1, device=self.device)
        for axis, g in self.groups.groups.items():
            if g is not None and len(self.groups.ranks[axis]) > 1:
                dist.all_reduce(t, group=g)

    def destroy(self) -> None:
        self.groups.destroy()


def detect_node_size(world_size: int) -> int | None:
    local = os.environ.get("LOCAL_WORLD_SIZE")
    if local and int(local) < world_size:
        return int(local)
    return None


def build_parallel_runtime(spec, *, device, rank: int | None = None, world_size: int | None = None,
                           node_size: int | None = None) -> ParallelRuntime:
    rank = dist.get_rank() if rank is None and dist.is_initialized() else (rank or 0)
    world_size = dist.get_world_size() if world_size is None and dist.is_initialized() else (world_size or 1)
    plan = plan_from_run_spec(spec, world_size, node_size if node_size is not None else detect_node_size(world_size))
    t = spec.topology
    timeouts = parse_group_timeouts(t.process_group_timeout, t.process_group_timeout_seconds)
    groups = ProcessGroupCollection.from_plan(plan, rank, timeouts)
    policy = CPBPPolicy(clean_kv_layout=spec.kernel.cp_bp_clean_kv_layout,
                        clean_kv_transport=spec.kernel.cp_bp_clean_kv_transport)
    return ParallelRuntime(plan=plan, assignment=plan.assignment(rank), groups=groups, policy=policy,
                           device=torch.device(device), rank=rank, world_size=world_size,
                           share_clean_replicas=bool(spec.kernel.cp_bp_share_clean_replicas),
                           pure_cp_token_split=bool(spec.kernel.pure_cp_token_split)
                           and (spec.objective.block_size or 0) % max(spec.topology.context_parallel_size, 1) == 0)
