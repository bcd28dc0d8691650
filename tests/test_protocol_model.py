"""Exhaustive interleaving check of the cross-rank flag protocols the peer-memory kernels use.

Each rank is modelled as the sequence of globally visible steps its stream performs (stores to peers' memory, flag
stores with release order, bounded flag waits with acquire order, loads from peers). A depth-first search visits every
interleaving of the ranks' steps (states are memoised), and at every load the model checks which value is visible.
The flag steps are those of `csrc/comm.cu` (`barrier_kernel`: rank r stores the epoch into slot r of every peer's flag
array, then waits until every slot of its own array has reached the epoch; epochs only grow) and of the fused
context-parallel attention forward (`csrc/peer_pull.cuh`: puller warps claim pieces from an atomic counter, copy them,
and add to a per-tile counter that the consumer waits on).

What is checked:
  * the fused optimizer step (barrier, pull-reduce, barrier, update + push, barrier) never reads a peer's gradient
    before the peer finished writing it, never overwrites parameters a peer still reads, over several steps that reuse
    the same buffers and flag slots;
  * leaving out the middle or the closing barrier IS caught (the model is not vacuous);
  * the ranks' shares of the gradient norm are read only after every rank wrote its share of the same step;
  * a rank that never arrives leaves the others waiting at the barrier and nowhere else (that wait is the bounded one
    that raises on the device);
  * the pull protocol hands a tile to the consumer only after every piece of it was copied, for any number of pullers.
"""
from __future__ import annotations

import pytest

# ------------------------------------------------------------------------------------------------ the explorer


class Violation(Exception):
    pass


def explore(programs, init_memory, max_states=2_000_000):
    """programs[r]: list of steps; a step is a function (mem, r) -> None | "blocked" that mutates `mem` (a dict).
    Explores every interleaving. Returns (#states, set of tuples of program counters at which the system was stuck)."""
    seen = set()
    stuck = set()
    stack = [(tuple(0 for _ in programs), tuple(sorted(init_memory.items(), key=repr)))]
    while stack:
        state = stack.pop()
        if state in seen:
            continue
        seen.add(state)
        if len(seen) > max_states:
            raise RuntimeError("state space larger than expected")
        pcs, mem_items = state
        progressed = False
        for r, prog in enumerate(programs):
            if pcs[r] >= len(prog):
                continue
            mem = dict(mem_items)
            if prog[pcs[r]](mem, r) == "blocked":
                continue
            progressed = True
            nxt = tuple(p + (i == r) for i, p in enumerate(pcs))
            stack.append((nxt, tuple(sorted(mem.items(), key=repr))))
        if not progressed and any(pcs[r] < len(p) for r, p in enumerate(programs)):
            stuck.add(pcs)
    return len(seen), stuck


# ----------------------------------------------------------------------------------- steps of the barrier kernel
def arrive(epoch, world):
    """flag_store_release(flags[peer] + rank, epoch) for every peer: one step per peer (the stores are independent)."""
    def step_for(peer):
        def step(mem, r):
            if mem[("flag", peer, r)] > epoch:
                raise Violation("epochs must grow")
            mem[("flag", peer, r)] = epoch
        return step
    return [step_for(p) for p in range(world)]


def wait_all(epoch, world):
    """flag_wait_geq(flags[rank] + peer, epoch) for every peer."""
    def step_for(peer):
        def step(mem, r):
            return None if mem[("flag", r, peer)] >= epoch else "blocked"
        return step
    return [step_for(p) for p in range(world)]


def barrier(epoch, world):
    return arrive(epoch, world) + wait_all(epoch, world)


def flags(world):
    return {("flag", a, b): 0 for a in range(world) for b in range(world)}


# ------------------------------------------------------------------------------------------ fused optimizer step
def optimizer_step_program(world, steps, *, middle_barrier=True, closing_barrier=True):
    """One rank's stream over `steps` optimizer steps. Memory: ("grad", owner) = step whose gradient the owner's buffer
    holds; ("param", holder, shard) = step whose parameters of `shard` the holder's buffer holds; ("reading", owner, reader).
    Per step t (epochs 3t+1 .. 3t+3): the backward pass writes this rank's gradient buffer; barrier; pull-reduce reads every
    peer's gradient (must be step t's); barrier; update pushes the new parameters of this rank's shard into every peer;
    barrier; the next forward reads every shard's parameters from the rank's own buffer (must be step t's)."""
    prog = []
    for t in range(1, steps + 1):
        e = 3 * (t - 1)

        def write_grad(mem, r, t=t):
            for reader in range(world):
                if mem[("reading", r, reader)]:
                    raise Violation(f"rank {r} overwrites its gradients while rank {reader} still reads them")
            mem[("grad", r)] = t
        prog.append(write_grad)
        prog += barrier(e + 1, world)
        for peer in range(world):
            def begin_read(mem, r, peer=peer, t=t):
                if mem[("grad", peer)] != t:
                    raise Violation(f"rank {r} reads gradients of step {mem[('grad', peer)]} from rank {peer} in step {t}")
                mem[("reading", peer, r)] = 1

            def end_read(mem, r, peer=peer):
                mem[("reading", peer, r)] = 0
            prog += [begin_read, end_read]

        def write_sumsq(mem, r, t=t):          # this rank's share of the squared gradient norm, read by every peer
            mem[("sumsq", r)] = t
        prog.append(write_sumsq)
        if middle_barrier:
            prog += barrier(e + 2, world)
        for peer in range(world):
            def read_sumsq(mem, r, peer=peer, t=t):
                if mem[("sumsq", peer)] != t:
                    raise Violation(f"rank {r} clips step {t} with rank {peer}'s norm share of step {mem[('sumsq', peer)]}")
            prog.append(read_sumsq)
        for peer in range(world):
            def push(mem, r, peer=peer, t=t):
                mem[("param", peer, r)] = t
            prog.append(push)
        if closing_barrier:
            prog += barrier(e + 3, world)

        def forward(mem, r, t=t):
            for shard in range(world):
                if mem[("param", r, shard)] != t:
                    raise Violation(f"rank {r} runs step {t + 1} with parameters of step {mem[('param', r, shard)]} in shard {shard}")
        prog.append(forward)
    return prog


def optimizer_memory(world):
    mem = flags(world)
    mem.update({("grad", r): 0 for r in range(world)})
    mem.update({("sumsq", r): 0 for r in range(world)})
    mem.update({("param", h, s): 0 for h in range(world) for s in range(world)})
    mem.update({("reading", o, r): 0 for o in range(world) for r in range(world)})
    return mem


@pytest.mark.parametrize("world,steps", [(2, 3), (3, 2)])
def test_fused_optimizer_step_orders_every_interleaving(world, steps):
    programs = [optimizer_step_program(world, steps) for _ in range(world)]
    states, stuck = explore(programs, optimizer_memory(world))
    assert states > 500 and not stuck


def test_the_model_catches_a_missing_barrier():
    # without the closing barrier a fast rank starts the next forward before a slow peer pushed its shard
    with pytest.raises(Violation, match="parameters of step"):
        explore([optimizer_step_program(2, 2, closing_barrier=False) for _ in range(2)], optimizer_memory(2))
    # without the middle barrier a rank clips with a peer's norm share of the previous step
    with pytest.raises(Violation, match="norm share"):
        explore([optimizer_step_program(2, 2, middle_barrier=False) for _ in range(2)], optimizer_memory(2))


def test_a_missing_rank_blocks_the_others_only_inside_the_barrier_wait():
    world = 3
    programs = [optimizer_step_program(world, 1) for _ in range(world)]
    programs[2] = programs[2][:1]                 # rank 2 writes its gradients and never arrives
    _, stuck = explore(programs, optimizer_memory(world))
    first_wait = 1 + world                        # gradient write, `world` arrival stores, then the waits
    assert stuck
    for pcs in stuck:
        for r in (0, 1):
            # the wait on rank 2's slot of the FIRST barrier: the bounded wait that sets the device error record
            assert pcs[r] == first_wait + 2


# ----------------------------------------------------------------- pull protocol of the fused attention forward
def pull_programs(pullers, tiles, pieces_per_tile):
    """Pullers: claim a piece from the shared counter (atomicAdd), copy it (remote load, local store), add one to its
    tile's ready counter (release). Consumer: per tile, wait until the counter equals pieces_per_tile (acquire), then
    read every piece of the tile from local memory."""
    total = tiles * pieces_per_tile

    def claim(mem, r):
        mem[("mine", r)] = mem["next"]
        mem["next"] += 1

    def copy(mem, r):
        p = mem[("mine", r)]
        if p < total:
            mem[("copied", p)] = 1

    def publish(mem, r):
        p = mem[("mine", r)]
        if p < total:
            mem[("ready", p // pieces_per_tile)] += 1

    # every puller loops until the counter runs out: at most `total` rounds each, plus the one that finds nothing
    puller = [claim, copy, publish] * (total + 1)
    consumer = []
    for t in range(tiles):
        def wait(mem, r, t=t):
            return None if mem[("ready", t)] == pieces_per_tile else "blocked"

        def read(mem, r, t=t):
            for p in range(t * pieces_per_tile, (t + 1) * pieces_per_tile):
                if not mem[("copied", p)]:
                    raise Violation(f"tile {t} was handed over before piece {p} arrived")
        consumer += [wait, read]
    mem = {"next": 0}
    mem.update({("mine", r): 0 for r in range(pullers)})
    mem.update({("copied", p): 0 for p in range(total)})
    mem.update({("ready", t): 0 for t in range(tiles)})
    return [list(puller) for _ in range(pullers)] + [consumer], mem


@pytest.mark.parametrize("pullers", [1, 2])
def test_pulled_tiles_are_complete_when_the_consumer_sees_them(pullers):
    programs, mem = pull_programs(pullers, tiles=2, pieces_per_tile=2)
    states, stuck = explore(programs, mem)
    assert states > 30 and not stuck


def test_publishing_before_the_copy_is_caught():
    programs, mem = pull_programs(2, tiles=1, pieces_per_tile=2)
    for prog in programs[:2]:                      # swap copy and publish in every round
        for i in range(0, len(prog), 3):
            prog[i + 1], prog[i + 2] = prog[i + 2], prog[i + 1]
    with pytest.raises(Violation, match="before piece"):
        explore(programs, mem)
