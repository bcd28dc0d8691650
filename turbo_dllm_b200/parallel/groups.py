"""Process groups: one communicator per parallel axis, built from a ParallelPlan.

Every axis gets its own `dist.new_group`, also when it spans the whole world, so that each has
an independent ordering domain; every rank takes part in creating every group (a collective
requirement of `new_group`). Per-group timeouts come from `GROUP=SECONDS` settings. The
`optimizer_data_parallel_group` joins ranks that hold the same parameter shard coordinates
(equal PP/TP/EP rank), i.e. DP × CP/BP.

Counterpart of dllm_parallel/core/parallel/groups.py:21-45 (timeouts), :76-152 (from_plan),
:154-177 (destroy), :243-265 (optimizer group).
"""
from __future__ import annotations

import datetime as _dt
from dataclasses import dataclass, field

import torch.distributed as dist

from .topology import ParallelPlan, RankAssignment

AXES = ("data_parallel", "dense_data_parallel", "context_block_parallel", "local_parallel", "clean_replica",
        "tensor", "pipeline", "expert", "model_input", "model_parallel", "optimizer_data_parallel",
        "dense_optimizer")


def parse_group_timeouts(entries, default_seconds: float | None = None) -> dict[str, float]:
    out: dict[str, float] = {}
    if default_seconds:
        out["default"] = float(default_seconds)
    for item in entries or ():
        name, _, secs = item.partition("=")
        name = name.strip()
        if name not in AXES and name != "default":
            raise ValueError(f"unknown process group {name!r} in timeout setting; known: {AXES}")
        out[name] = float(secs)
    return out


def dense_optimizer_ranks(plan: ParallelPlan, a: RankAssignment) -> list[int]:
    """Ranks holding the same replicated (non-expert) parameter shard: equal PP and TP coordinates,
    any DP / CP-BP / EP coordinate."""
    return sorted(b.rank for b in plan.rank_assignments
                  if (b.pipeline_parallel_rank, b.tensor_parallel_rank)
                  == (a.pipeline_parallel_rank, a.tensor_parallel_rank))


def optimizer_data_parallel_ranks(plan: ParallelPlan, a: RankAssignment) -> list[int]:
    return sorted(b.rank for b in plan.rank_assignments
                  if (b.pipeline_parallel_rank, b.tensor_parallel_rank, b.expert_parallel_rank)
                  == (a.pipeline_parallel_rank, a.tensor_parallel_rank, a.expert_parallel_rank))


@dataclass
class ProcessGroupCollection:
    plan: ParallelPlan
    rank: int
    ranks: dict[str, list[int]] = field(default_factory=dict)
    groups: dict[str, object] = field(default_factory=dict)
    _created: list = field(default_factory=list)

    @classmethod
    def from_plan(cls, plan: ParallelPlan, rank: int, timeouts: dict[str, float] | None = None,
                  backend: str | None = None) -> "ProcessGroupCollection":
        timeouts = timeouts or {}
        self = cls(plan=plan, rank=rank)
        mine = plan.assignment(rank)
        field_of = {"data_parallel": "data_parallel_group", "dense_data_parallel": "dense_data_parallel_group",
                    "context_block_parallel": "context_block_parallel_group", "clean_replica": "clean_replica_group",
                    "local_parallel": "local_parallel_group",
                    "tensor": "tensor_parallel_group", "pipeline": "pipeline_parallel_group",
                    "expert": "expert_parallel_group", "model_input": "model_input_group",
                    "model_parallel": "model_parallel_group"}
        for axis in AXES:
            if axis in ("optimizer_data_parallel", "dense_optimizer"):
                fn = optimizer_data_parallel_ranks if axis == "optimizer_data_parallel" else dense_optimizer_ranks
                all_lists, seen = [], set()
                for a in plan.rank_assignments:
                    g = tuple(fn(plan, a))
                    if g not in seen:
                        seen.add(g)
                        all_lists.append(list(g))
                my_list = fn(plan, mine)
            else:
                all_lists = plan.groups(field_of[axis])
                my_list = list(getattr(mine, field_of[axis]))
            secs = timeouts.get(axis, timeouts.get("default"))
            kw = {}
            if secs:
                kw["timeout"] = _dt.timedelta(seconds=secs)
            if backend:
                kw["backend"] = backend
            for ranks in all_lists:  # every rank creates every group, in the same order
                g = dist.new_group(ranks=ranks, **kw) if dist.is_initialized() else None
                self._created.append(g)
                if ranks == my_list:
                    self.groups[axis] = g
            self.ranks[axis] = my_list
        return self

    def group(self, axis: str):
        return self.groups[axis]

    def size(self, axis: str) -> int:
        return len(self.ranks[axis])

    def rank_in(self, axis: str) -> int:
        return self.ranks[axis].index(self.rank)

    def destroy(self) -> None:
        for g in self._created:
            if g is not None:
                try:
                    dist.destroy_process_group(g)
                except Exception:
                    pass
        self._created.clear()
        self.groups.clear()
