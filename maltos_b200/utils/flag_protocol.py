"""Host-side model of the flag protocols of the one-sided kernels, checked over EVERY interleaving.

The kernels that move data between GPUs without a collective library (``csrc/tp_pull.cu``, the push roles of
``csrc/gemm.cu``, ``csrc/moe_dispatch.cu``, ``ops/peer_ring.py``) are safe only if their flags order every remote write
before the read that needs it and every read before the write that recycles the buffer. A race in such a protocol does
not show up in a numerics test that happens to run the ranks in lock step, so the protocols are written down here as
small programs over shared cells and flags and explored exhaustively: every reachable state of every interleaving of
the agents (a rank, or a role inside a rank's kernel) is visited once.

Checked: a read sees exactly the version it expects (not a stale one, not one recycled too early) and never overlaps a
write of the same cell; two writes of a cell never overlap; no state is reached in which unfinished agents all wait.
The reference has no counterpart (its transfers are NCCL calls); this is the check that replaces a race detector for
hand-written signalling.

Step vocabulary (tuples):
    ("write", cell, version)      split into begin / end so that overlap with a read or another write is visible
    ("read", cell, version)       the cell must hold ``version`` and must not be in the middle of a write
    ("set", flag, value)          plain store of a flag word
    ("wait", flag, at_least)      blocks until ``flag >= at_least`` (flags start at 0; the kernels compare wrap-safe)
    ("barrier", name, members)    all ``members`` (agent names) leave together (a group all-reduce, or a kernel boundary)
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass


class ProtocolViolation(AssertionError):
    """A read saw the wrong version / an overlapping write, or two writes overlapped."""


class ProtocolDeadlock(AssertionError):
    """Unfinished agents exist and none can take a step."""


@dataclass
class Exploration:
    states: int
    transitions: int


def _expand(program):
    out = []
    for step in program:
        if step[0] == "write":
            out.append(("write_begin", step[1], step[2]))
            out.append(("write_end", step[1], step[2]))
        else:
            out.append(step)
    return tuple(out)


def explore(programs: dict, *, max_states: int = 2_000_000) -> Exploration:
    """``programs``: agent name -> list of steps. Explores all interleavings; raises on the first violation / deadlock."""
    names = sorted(programs)
    progs = {n: _expand(programs[n]) for n in names}
    index = {n: i for i, n in enumerate(names)}
    start = (tuple(0 for _ in names), frozenset(), frozenset())      # pcs, cells {(cell, version, writers)}, flags {(flag, value)}
    seen = {start}
    queue = deque([start])
    transitions = 0
    while queue:
        pcs, cells_f, flags_f = queue.popleft()
        cells, flags = dict((c, (v, w)) for c, v, w in cells_f), dict(flags_f)
        moved = False
        done_barriers = set()
        for i, name in enumerate(names):
            prog = progs[name]
            if pcs[i] >= len(prog):
                continue
            step = prog[pcs[i]]
            kind = step[0]
            new_pcs, new_cells, new_flags = list(pcs), cells, flags
            if kind == "wait":
                if flags.get(step[1], 0) < step[2]:
                    continue
            elif kind == "set":
                new_flags = dict(flags)
                new_flags[step[1]] = step[2]
            elif kind == "write_begin":
                version, writers = cells.get(step[1], (0, 0))
                if writers:
                    raise ProtocolViolation(f"{name}: write of {step[1]} (version {step[2]}) overlaps another write")
                new_cells = dict(cells)
                new_cells[step[1]] = (version, 1)
            elif kind == "write_end":
                new_cells = dict(cells)
                new_cells[step[1]] = (step[2], 0)
            elif kind == "read":
                version, writers = cells.get(step[1], (0, 0))
                if writers:
                    raise ProtocolViolation(f"{name}: read of {step[1]} (expects version {step[2]}) overlaps a write")
                if version != step[2]:
                    raise ProtocolViolation(f"{name}: read of {step[1]} expects version {step[2]}, holds {version}")
            elif kind == "barrier":
                key = (step[1], tuple(step[2]))
                if key in done_barriers:
                    continue
                members = step[2]
                if not all(pcs[index[m]] < len(progs[m]) and progs[m][pcs[index[m]]][:2] == ("barrier", step[1]) for m in members):
                    continue
                done_barriers.add(key)
                for m in members:
                    new_pcs[index[m]] += 1
                new_pcs[i] -= 1          # the common increment below
            else:
                raise ValueError(f"unknown step {step!r}")
            new_pcs[i] += 1
            moved = True
            transitions += 1
            state = (tuple(new_pcs), frozenset((c, v, w) for c, (v, w) in new_cells.items()), frozenset(new_flags.items()))
            if state not in seen:
                if len(seen) >= max_states:
                    raise RuntimeError(f"state space larger than {max_states}")
                seen.add(state)
                queue.append(state)
        if not moved and any(pcs[i] < len(progs[n]) for i, n in enumerate(names)):
            stuck = {n: progs[n][pcs[i]] for i, n in enumerate(names) if pcs[i] < len(progs[n])}
            raise ProtocolDeadlock(f"no agent can move: {stuck}")
    return Exploration(len(seen), transitions)


# ------------------------------------------------------------------------------------------------ the protocols
def pull_collective(world: int, calls: int, *, double_buffered: bool = True, publish_before_write: bool = False) -> dict:
    """``pull_reduce_scatter_kernel`` / ``pull_all_gather_kernel``: every rank writes its buffer of parity ``n & 1``,
    stores ``n`` into every peer's flag word, waits for every peer's word, then reads the peers' buffers. No second flag:
    passing the wait of call ``n + 1`` implies that every peer has left call ``n``. ``double_buffered=False`` and
    ``publish_before_write=True`` are broken variants the checker must reject."""
    programs = {}
    for me in range(world):
        prog = []
        for n in range(1, calls + 1):
            b = (n & 1) if double_buffered else 0
            write = [("write", ("data", me, b), n)]
            publish = [("set", ("ready", peer, b, me), n) for peer in range(world) if peer != me]
            prog += (publish + write) if publish_before_write else (write + publish)
            prog += [("wait", ("ready", me, b, peer), n) for peer in range(world) if peer != me]
            prog += [("read", ("data", peer, b), n) for peer in range(world) if peer != me]
        programs[f"rank{me}"] = prog
    return programs


def push_with_back_pressure(world: int, calls: int, *, back_pressure: bool = True, double_buffered: bool = True) -> dict:
    """The push inside the GEMM (all-gather; the reduce-scatter's staging slots have the same shape): the push role of rank
    ``s`` waits until destination ``d`` has consumed its buffer of two calls ago, writes slot ``s`` of ``d``'s buffer of
    parity ``n & 1`` and stores ``n`` into ``d``'s "arrived" word; the consumer role of ``d`` (the GEMM producer warp of
    the SAME kernel) waits per source, reads, and at the end stores ``n`` into every rank's "consumed" word. The two roles
    of a rank meet at the kernel boundary. What the exploration shows: with two buffers the "consumed" wait is redundant
    (a rank reaches call ``n + 2`` only after every peer has started call ``n + 1``, i.e. left call ``n``) - it is kept in
    the kernels as a second line of defence; with ONE buffer it is what makes the protocol safe (``back_pressure=False,
    double_buffered=False`` is the broken variant)."""
    programs = {}
    for me in range(world):
        push, consume = [], []
        for n in range(1, calls + 1):
            b = (n & 1) if double_buffered else 0
            lag = 2 if double_buffered else 1
            for step in range(world):
                dst = (me - step) % world
                if back_pressure and n > lag:
                    push.append(("wait", ("consumed", me, b, dst), n - lag))
                push.append(("write", ("slot", dst, b, me), n))
                push.append(("set", ("arrived", dst, b, me), n))
            for step in range(world):
                src = (me + step) % world
                consume.append(("wait", ("arrived", me, b, src), n))
                consume.append(("read", ("slot", me, b, src), n))
            consume += [("set", ("consumed", r, b, me), n) for r in range(world)]
            boundary = ("barrier", f"kernel{me}.{n}", (f"rank{me}.push", f"rank{me}.gemm"))
            push.append(boundary)
            consume.append(boundary)
        programs[f"rank{me}.push"], programs[f"rank{me}.gemm"] = push, consume
    return programs


def alternating_buffers_with_barrier(world: int, transfers: int, *, buffers: int = 2) -> dict:
    """Expert-parallel dispatch / combine: every rank pushes rows into every peer's buffer ``n % 2``, one group barrier,
    every rank reads its own buffer. The next transfer uses the other buffer; a buffer is written again only after the
    barrier of the transfer in between, which a rank enters after it has read. ``buffers=1`` is the broken variant."""
    members = tuple(f"rank{r}" for r in range(world))
    programs = {}
    for me in range(world):
        prog = []
        for n in range(1, transfers + 1):
            b = n % buffers
            prog += [("write", ("rows", dst, b, me), n) for dst in range(world)]
            prog.append(("barrier", f"transfer{n}", members))
            prog += [("read", ("rows", me, b, src), n) for src in range(world)]
        programs[f"rank{me}"] = prog
    return programs


def ring_publish(world: int, calls: int, *, barrier_before_overwrite: bool = True, backward: bool = True, buffers: int = 1) -> dict:
    """Ring attention over peer memory: publish the own block into buffer ``n % buffers``, barrier B, pull the peers'
    blocks; in backward push one gradient contribution into every owner's slot for this rank, barrier C, sum the own slots.
    With ONE published buffer a barrier A is needed in front (all pulls of the previous call are done) -
    ``barrier_before_overwrite=False`` with one buffer is the broken variant. With TWO buffers alternating by call A is
    redundant: a rank reaches the publish of call ``n + 2`` only after barrier B of call ``n + 1``, which every rank enters
    after its pulls of call ``n``. The gradient slots need neither: they are recycled only after barrier C."""
    members = tuple(f"rank{r}" for r in range(world))
    programs = {}
    for me in range(world):
        prog = []
        for n in range(1, calls + 1):
            b = n % buffers
            if barrier_before_overwrite:
                prog.append(("barrier", f"A{n}", members))
            prog.append(("write", ("kv", me, b), n))
            if backward:
                prog += [("write", ("grad", me, src), -n) for src in range(world)]       # the owner zeroes its slots
            prog.append(("barrier", f"B{n}", members))
            prog += [("read", ("kv", (me - s) % world, b), n) for s in range(1, world)]
            if backward:
                prog += [("write", ("grad", owner, me), n) for owner in range(world)]
                prog.append(("barrier", f"C{n}", members))
                prog += [("read", ("grad", me, src), n) for src in range(world)]
        programs[f"rank{me}"] = prog
    return programs


def owner_reduce_and_push(world: int, steps: int, *, barrier_after_reduce: bool = True, barrier_after_push: bool = True) -> dict:
    """Peer-memory mode of the sharded optimizers (``runtime/plugins/zero1.py``, ``csrc/zero_fused.cu``): backward fills the
    rank's flat gradient bucket; barrier G1; the owner of shard ``r`` reads slice ``r`` of every rank's bucket
    (``peer_reduce_shard``); barrier G2; AdamW on the own shard stores the new slice into every rank's parameter buffer
    (``adamw_push``); barrier G3; the next forward / backward reads all slices of the own parameter buffer and overwrites the
    gradient bucket. Without G3 a rank reads a parameter slice that a peer has not stored yet; without G2 AND G3 a fast rank's
    next backward also overwrites a bucket that a peer still reads (both rejected by the exploration). G2 alone is redundant
    while G3 (or the all-gather that replaces the push) follows: every rank enters it after its reads. The plugin keeps G2:
    one more one-element all-reduce per step, and the reduction stays safe whatever follows it."""
    members = tuple(f"rank{r}" for r in range(world))
    programs = {}
    for me in range(world):
        prog = []
        for n in range(1, steps + 1):
            prog += [("read", ("param", me, owner), n - 1) for owner in range(world)]          # forward + backward of step n
            prog += [("write", ("grad", me, shard), n) for shard in range(world)]
            prog.append(("barrier", f"G1.{n}", members))
            prog += [("read", ("grad", src, me), n) for src in range(world)]
            if barrier_after_reduce:
                prog.append(("barrier", f"G2.{n}", members))
            prog += [("write", ("param", dst, me), n) for dst in range(world)]
            if barrier_after_push:
                prog.append(("barrier", f"G3.{n}", members))
        prog += [("read", ("param", me, owner), steps) for owner in range(world)]
        programs[f"rank{me}"] = prog
    return programs


__all__ = ["Exploration", "ProtocolDeadlock", "ProtocolViolation", "alternating_buffers_with_barrier", "explore", "owner_reduce_and_push",
           "pull_collective",
           "push_with_back_pressure", "ring_publish"]
