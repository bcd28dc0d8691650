"""Assignment of whole noisy blocks to block-parallel workers.

Noisy block b attends to b clean blocks, so its cost grows linearly with b. The dual-end
schedule pairs block l with block B-1-l (constant pair cost) and deals pairs out contiguously,
which balances the prefix cost across workers; a `contiguous` policy exists for ablations.
Behaviour follows dllm_parallel/core/schedules/block.py:52-230 (pairs :52-65, schedule :68-120,
dual-end dealing :166-203, short case by greedy LPT :206-230, env override :149-163).
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass

POLICY_ENV = "DLLM_BLOCK_SCHEDULE_POLICY"
POLICIES = ("dual_end", "contiguous")


@dataclass(frozen=True)
class BlockSchedule:
    num_blocks: int
    num_workers: int
    policy: str
    blocks_by_worker: tuple[tuple[int, ...], ...]

    @property
    def active_prefix_cost_by_worker(self) -> list[int]:
        return [sum(b) for b in self.blocks_by_worker]

    @property
    def blocks_per_worker(self) -> list[int]:
        return [len(b) for b in self.blocks_by_worker]

    def worker_of_block(self, block: int) -> int:
        for w, blocks in enumerate(self.blocks_by_worker):
            if block in blocks:
                return w
        raise KeyError(block)

    def imbalance(self) -> float:
        costs = self.active_prefix_cost_by_worker
        mean = sum(costs) / max(len(costs), 1)
        return (max(costs) / mean) if mean > 0 else 1.0


def dual_end_pairs(num_blocks: int) -> list[tuple[int, ...]]:
    """[(0, B-1), (1, B-2), ...] plus the lone middle block when B is odd."""
    pairs: list[tuple[int, ...]] = [(l, num_blocks - 1 - l) for l in range(num_blocks // 2)]
    if num_blocks % 2:
        pairs.append((num_blocks // 2,))
    return pairs


def resolve_policy(policy: str | None = None) -> str:
    chosen = policy or os.environ.get(POLICY_ENV) or "dual_end"
    if chosen not in POLICIES:
        raise ValueError(f"unknown block schedule policy {chosen!r}; choose from {POLICIES}")
    return chosen


def _balanced_bounds(n: int, parts: int, i: int) -> tuple[int, int]:
    base, rem = divmod(n, parts)
    start = i * base + min(i, rem)
    return start, start + base + (1 if i < rem else 0)


def _dual_end(num_blocks: int, workers: int) -> list[list[int]]:
    full_pairs = [p for p in dual_end_pairs(num_blocks) if len(p) == 2]
    if len(full_pairs) < workers:
        # fewer pairs than workers: greedy longest-processing-time over single blocks,
        # heaviest (last) block first, ties to the lowest worker index
        owned: list[list[int]] = [[] for _ in range(workers)]
        load = [0] * workers
        count = [0] * workers
        for b in range(num_blocks - 1, -1, -1):
            w = min(range(workers), key=lambda i: (load[i], count[i], i))
            owned[w].append(b)
            load[w] += b
            count[w] += 1
        return owned
    owned = [[] for _ in range(workers)]
    for w in range(workers):
        lo, hi = _balanced_bounds(len(full_pairs), workers, w)
        for p in full_pairs[lo:hi]:
            owned[w].extend(p)
    if num_blocks % 2:
        mid = num_blocks // 2
        w = min(range(workers), key=lambda i: (sum(owned[i]), i))
        owned[w].append(mid)
    return owned


def build_block_schedule(num_blocks: int, num_workers: int, policy: str | None = None) -> BlockSchedule:
    if num_workers < 1:
        raise ValueError("num_workers must be >= 1")
    if num_blocks < num_workers:
        raise ValueError(f"cannot give {num_workers} block-parallel workers at least one of "
                         f"{num_blocks} blocks")
    pol = resolve_policy(policy)
    if pol == "contiguous":
        owned = [list(range(*_balanced_bounds(num_blocks, num_workers, w))) for w in range(num_workers)]
    else:
        owned = _dual_end(num_blocks, num_workers)
    sched = BlockSchedule(num_blocks, num_workers, pol, tuple(tuple(sorted(b)) for b in owned))
    validate_block_schedule(sched)
    return sched


def validate_block_schedule(s: BlockSchedule) -> None:
    seen = sorted(b for blocks in s.blocks_by_worker for b in blocks)
    if seen != list(range(s.num_blocks)):
        raise ValueError("block schedule must own every block exactly once")
    if any(len(b) == 0 for b in s.blocks_by_worker):
        raise ValueError("every block-parallel worker needs at least one block")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Print the block schedule for a (blocks, workers) pair")
    ap.add_argument("--num-blocks", type=int, required=True)
    ap.add_argument("--num-workers", type=int, required=True)
    ap.add_argument("--policy", choices=POLICIES)
    a = ap.parse_args(argv)
    s = build_block_schedule(a.num_blocks, a.num_workers, a.policy)
    print(json.dumps({"policy": s.policy, "blocks_by_worker": s.blocks_by_worker,
                      "prefix_cost_by_worker": s.active_prefix_cost_by_worker,
                      "imbalance": round(s.imbalance(), 4)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
