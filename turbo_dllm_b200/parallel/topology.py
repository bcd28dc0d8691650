"""Topology planner: world ranks -> (DP, PP, local CP/BP, TP, EP) coordinates and groups.

Logical rank order is DP × PP × local × TP × EP with EP fastest, then TP, so tensor- and
expert-parallel peers are neighbours (same NVSwitch domain) and data-parallel replicas are the
outermost stride. Each rank gets a `RankAssignment` with nine groups. On multi-node jobs a
placement policy maps logical to physical ranks so that a model replica stays inside a node
when it fits (`auto`) or so that context-parallel peers span nodes (`inter_node_cp`).

Mirrors dllm_parallel/core/parallel/topology.py:71-224 (build_parallel_plan), :227-417
(rank assignment), :449-649 (physical maps), :675-728 (CP/BP rank, clean replicas), :731-785
(layout names).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass, field

from .schedule import BlockSchedule, build_block_schedule


@dataclass(frozen=True)
class RankAssignment:
    rank: int
    data_parallel_rank: int
    pipeline_parallel_rank: int
    local_parallel_rank: int
    context_parallel_rank: int
    block_parallel_rank: int
    tensor_parallel_rank: int
    expert_parallel_rank: int
    data_parallel_group: list[int]
    dense_data_parallel_group: list[int]
    context_block_parallel_group: list[int]
    clean_replica_group: list[int]
    tensor_parallel_group: list[int]
    pipeline_parallel_group: list[int]
    expert_parallel_group: list[int]
    model_input_group: list[int]
    model_parallel_group: list[int]
    owned_blocks: tuple[int, ...] = ()
    # all ranks of the context/block axis of one replica (the clean K/V of every shard owner is pulled by all of
    # them when blocks are spread over more ranks than the clean tokens)
    local_parallel_group: tuple[int, ...] = ()

    GROUP_FIELDS = ("data_parallel_group", "dense_data_parallel_group", "context_block_parallel_group",
                    "clean_replica_group", "tensor_parallel_group", "pipeline_parallel_group",
                    "expert_parallel_group", "model_input_group", "model_parallel_group")


@dataclass(frozen=True)
class ParallelPlan:
    world_size: int
    data_parallel_size: int
    pipeline_parallel_size: int
    context_parallel_size: int
    block_parallel_size: int
    tensor_parallel_size: int
    expert_parallel_size: int
    local_parallel_size: int
    model_parallel_size: int
    layout: str
    placement: str
    node_size: int | None
    block_schedule: BlockSchedule
    rank_assignments: list[RankAssignment] = field(default_factory=list)
    logical_to_physical: list[int] = field(default_factory=list)

    def assignment(self, rank: int) -> RankAssignment:
        return self.rank_assignments[rank]

    def groups(self, name: str) -> list[list[int]]:
        """Distinct rank lists of one group kind, in first-member order."""
        seen, out = set(), []
        for a in self.rank_assignments:
            g = tuple(getattr(a, name))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out


def layout_name(dp: int, cp: int, bp: int, tp: int, ep: int, pp: int, replicate_clean_prefix: bool) -> str:
    parts = ["dp"]
    if pp > 1:
        parts.append("pp")
    if cp > 1 and bp > 1:
        parts.append("fused_cp_bp")
    elif cp > 1:
        parts.append("cp")
    elif bp > 1:
        parts.append("replicated_prefix_bp" if replicate_clean_prefix else "bp")
    if tp > 1:
        parts.append("tp")
    if ep > 1:
        parts.append("ep")
    return "_x_".join(parts)


def _physical_map(world: int, model_parallel: int, tp_ep: int, local: int, node_size: int | None,
                  policy: str) -> tuple[list[int], str]:
    """Permutation logical rank -> physical rank, and the placement name."""
    ident = list(range(world))
    if not node_size or node_size >= world:
        return ident, "single_node" if not node_size or node_size >= world else "identity"
    if policy == "inter_node_cp":
        # put the `local` (CP/BP) axis across nodes: ranks with equal (dp, tp/ep) coordinates and
        # consecutive local coordinates land on different nodes
        nodes = world // node_size
        if nodes > 1 and local % nodes == 0:
            phys = [0] * world
            slot = [0] * nodes
            for lr in range(world):
                local_coord = (lr // tp_ep) % local
                node = local_coord % nodes
                phys[lr] = node * node_size + slot[node]
                slot[node] += 1
            if sorted(phys) == ident:
                return phys, "inter_node_context_parallel"
        return ident, "identity"
    if model_parallel <= node_size and node_size % model_parallel == 0:
        # replicas fit inside a node: logical order already keeps a replica contiguous, and
        # TP/EP (innermost) on neighbouring GPUs
        return ident, "node_local_model_parallel_tp_inner" if tp_ep > 1 else "node_local_model_parallel"
    if model_parallel % node_size == 0:
        return ident, "multi_node_model_parallel_tp_inner" if tp_ep > 1 else "multi_node_model_parallel"
    return ident, "identity"


def build_parallel_plan(*, num_blocks: int, world_size: int, data_parallel_size: int = 1,
                        context_parallel_size: int = 1, block_parallel_size: int = 1,
                        tensor_parallel_size: int = 1, expert_parallel_size: int = 1,
                        pipeline_parallel_size: int = 1, replicate_clean_prefix: bool = False,
                        node_size: int | None = None, placement_policy: str = "auto",
                        block_schedule_policy: str | None = None) -> ParallelPlan:
    dp, pp, cp, bp = data_parallel_size, pipeline_parallel_size, context_parallel_size, block_parallel_size
    tp, ep = tensor_parallel_size, expert_parallel_size
    if min(dp, pp, cp, bp, tp, ep) < 1:
        raise ValueError("parallel sizes must be >= 1")
    if cp > 1 and bp > 1 and (bp < cp or bp % cp):
        raise ValueError(f"fused CP+BP needs block_parallel_size ({bp}) to be a multiple of "
                         f"context_parallel_size ({cp})")
    local = max(cp, bp)
    model_parallel = pp * local * tp * ep
    if dp * model_parallel != world_size:
        raise ValueError(f"world_size {world_size} != dp {dp} × pp {pp} × local {local} × tp {tp} × ep {ep}")
    if placement_policy not in ("auto", "inter_node_cp"):
        raise ValueError(f"unknown placement policy {placement_policy!r}")
    schedule = build_block_schedule(num_blocks, bp, block_schedule_policy)
    l2p, placement = _physical_map(world_size, model_parallel, tp * ep, local, node_size, placement_policy)

    def coords(lr: int):
        e = lr % ep
        t = (lr // ep) % tp
        l = (lr // (ep * tp)) % local
        p = (lr // (ep * tp * local)) % pp
        d = lr // (ep * tp * local * pp)
        return d, p, l, t, e

    def logical(d, p, l, t, e):
        return (((d * pp + p) * local + l) * tp + t) * ep + e

    def phys(lrs):
        return sorted(l2p[x] for x in lrs)

    assignments: dict[int, RankAssignment] = {}
    for lr in range(world_size):
        d, p, l, t, e = coords(lr)
        cp_rank = l % cp
        bp_rank = l if bp > 1 else 0
        cp_chunk = (l // cp) * cp
        a = RankAssignment(
            rank=l2p[lr], data_parallel_rank=d, pipeline_parallel_rank=p, local_parallel_rank=l,
            context_parallel_rank=cp_rank, block_parallel_rank=bp_rank, tensor_parallel_rank=t,
            expert_parallel_rank=e,
            data_parallel_group=phys(logical(x, p, l, t, e) for x in range(dp)),
            dense_data_parallel_group=phys(logical(x, p, l, t, y) for x in range(dp) for y in range(ep)),
            context_block_parallel_group=phys(logical(d, p, cp_chunk + x, t, e) for x in range(cp)),
            clean_replica_group=phys(logical(d, p, x, t, e) for x in range(local) if x % cp == cp_rank),
            tensor_parallel_group=phys(logical(d, p, l, x, e) for x in range(tp)),
            pipeline_parallel_group=phys(logical(d, x, l, t, e) for x in range(pp)),
            expert_parallel_group=phys(logical(d, p, l, t, x) for x in range(ep)),
            model_input_group=phys(logical(d, x, y, z, e) for x in range(pp) for y in range(local)
                                   for z in range(tp)),
            model_parallel_group=phys(logical(d, x, y, z, w) for x in range(pp) for y in range(local)
                                      for z in range(tp) for w in range(ep)),
            owned_blocks=schedule.blocks_by_worker[bp_rank] if bp > 1 else tuple(range(num_blocks)),
            local_parallel_group=tuple(phys(logical(d, p, x, t, e) for x in range(local))),
        )
        assignments[a.rank] = a
    return ParallelPlan(
        world_size=world_size, data_parallel_size=dp, pipeline_parallel_size=pp,
        context_parallel_size=cp, block_parallel_size=bp, tensor_parallel_size=tp,
        expert_parallel_size=ep, local_parallel_size=local, model_parallel_size=model_parallel,
        layout=layout_name(dp, cp, bp, tp, ep, pp, replicate_clean_prefix), placement=placement,
        node_size=node_size, block_schedule=schedule,
        rank_assignments=[assignments[r] for r in range(world_size)], logical_to_physical=l2p)


def infer_data_parallel_size(world_size: int, spec) -> int:
    """DP is whatever the model-parallel axes leave of the world (run-spec topology section).
    Expert parallelism reuses data-parallel ranks for dense parameters, so EP divides DP×EP."""
    mp = spec.model_parallel_size()
    if world_size % mp:
        t = spec.topology
        raise ValueError(
            f"world size {world_size} is not a multiple of the model-parallel size {mp} "
            f"(local {spec.local_parallel_size} × tp {t.tensor_parallel_size} × ep {t.expert_parallel_size}"
            f" × pp {t.pipeline_parallel_size})")
    return world_size // mp


def plan_from_run_spec(spec, world_size: int, node_size: int | None = None) -> ParallelPlan:
    t = spec.topology
    bs = spec.objective.block_size or spec.model.seq_len
    return build_parallel_plan(
        num_blocks=max(spec.model.seq_len // bs, 1), world_size=world_size,
        data_parallel_size=infer_data_parallel_size(world_size, spec),
        context_parallel_size=t.context_parallel_size, block_parallel_size=t.block_parallel_size,
        tensor_parallel_size=t.tensor_parallel_size, expert_parallel_size=t.expert_parallel_size,
        pipeline_parallel_size=t.pipeline_parallel_size,
        replicate_clean_prefix=t.replicate_clean_prefix, node_size=node_size,
        placement_policy=t.placement_policy)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Print the parallel plan for a topology")
    ap.add_argument("--num-blocks", type=int, default=32)
    ap.add_argument("--world-size", type=int, required=True)
    for n in ("data", "context", "block", "tensor", "expert", "pipeline"):
        ap.add_argument(f"--{n}-parallel-size", type=int, default=1)
    ap.add_argument("--node-size", type=int)
    ap.add_argument("--placement-policy", default="auto")
    a = ap.parse_args(argv)
    plan = build_parallel_plan(
        num_blocks=a.num_blocks, world_size=a.world_size, data_parallel_size=a.data_parallel_size,
        context_parallel_size=a.context_parallel_size, block_parallel_size=a.block_parallel_size,
        tensor_parallel_size=a.tensor_parallel_size, expert_parallel_size=a.expert_parallel_size,
        pipeline_parallel_size=a.pipeline_parallel_size, node_size=a.node_size,
        placement_policy=a.placement_policy)
    print(json.dumps({"layout": plan.layout, "placement": plan.placement,
                      "prefix_cost_by_worker": plan.block_schedule.active_prefix_cost_by_worker,
                      "ranks": [{k: getattr(r, k) for k in ("rank", "data_parallel_rank", "local_parallel_rank",
                                                             "context_parallel_rank", "block_parallel_rank",
                                                             "tensor_parallel_rank", "expert_parallel_rank",
                                                             "context_block_parallel_group", "tensor_parallel_group",
                                                             "data_parallel_group")}
                                for r in plan.rank_assignments]}, indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
