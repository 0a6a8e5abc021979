"""CPU model of the buffer-reuse protocols of the NVLink data plane.

Ranks are interleaved at random at the granularity of their stream operations; a barrier lets a rank continue
only when every rank has arrived. The model checks the two invariants the kernels rely on:

* pull all-gather / reduce-scatter staging with two alternating buffers: a rank overwrites buffer ``k % 2`` for
  use ``k`` only after passing the barrier of use ``k - 1``, and no peer still reads use ``k - 2`` then;
* push all-gather into one persistent buffer per call site: peers store the slices of use ``k`` only after the
  barrier of use ``k``, which the owner reaches after its last read of use ``k - 1``.
"""

import random

import pytest


class Sim:
    def __init__(self, world: int, programs: list[list[tuple]], seed: int):
        self.world, self.programs = world, programs
        self.pc = [0] * world
        self.arrived: dict[int, set[int]] = {}
        self.rng = random.Random(seed)

    def runnable(self, r: int) -> bool:
        if self.pc[r] >= len(self.programs[r]):
            return False
        op = self.programs[r][self.pc[r]]
        if op[0] == "barrier":
            self.arrived.setdefault(op[1], set()).add(r)
            return len(self.arrived[op[1]]) == self.world
        return True

    def run(self, execute) -> None:
        while True:
            ready = [r for r in range(self.world) if self.runnable(r)]
            if not ready:
                assert all(self.pc[r] >= len(self.programs[r]) for r in range(self.world)), "deadlock"
                return
            r = self.rng.choice(ready)
            op = self.programs[r][self.pc[r]]
            if op[0] != "barrier":
                execute(r, op)
            self.pc[r] += 1


@pytest.mark.parametrize("world,seed", [(2, 0), (4, 1), (8, 2), (4, 3)])
def test_pull_gather_with_two_buffers(world, seed):
    uses = 7
    src = [[None, None] for _ in range(world)]          # src[rank][buffer] = (use, rank) tag of the slice held
    programs = []
    for r in range(world):
        prog = []
        for k in range(uses):
            prog.append(("publish", k))                 # write own slice into buffer k % 2
            prog.append(("barrier", k))
            for step in range(1, world):                # the copy CTAs of the fused kernel, peer by peer
                prog.append(("pull", k, (r + step) % world))
        programs.append(prog)

    def execute(r, op):
        if op[0] == "publish":
            src[r][op[1] % 2] = (op[1], r)
        else:
            _, k, peer = op
            assert src[peer][k % 2] == (k, peer), f"rank {r} read a slice of use {src[peer][k % 2]} while gathering use {k}"

    Sim(world, programs, seed).run(execute)


@pytest.mark.parametrize("world,seed", [(2, 0), (4, 1), (8, 2)])
def test_push_gather_into_persistent_site(world, seed):
    uses = 6
    site = [[None] * world for _ in range(world)]       # site[owner][slice] = use tag
    flags = [[-1] * world for _ in range(world)]
    programs = []
    for r in range(world):
        prog = []
        for k in range(uses):
            prog.append(("local", k))                   # own slice + own flag, before the barrier
            prog.append(("barrier", k))
            for step in range(1, world):
                prog.append(("push", k, (r - step) % world))
            for s in range(world):                      # the GEMM consumes the slices in ring order
                prog.append(("consume", k, (r + s) % world))
            prog.append(("backward_read", k))           # later reader of the same contents (weight gradient)
        programs.append(prog)

    def execute(r, op):
        if op[0] == "local":
            site[r][r] = op[1]
            flags[r][r] = op[1]
        elif op[0] == "push":
            _, k, peer = op
            site[peer][r] = k
            flags[peer][r] = k
        elif op[0] == "consume":
            _, k, s = op
            if flags[r][s] < k:                         # flag not yet raised: the tile waits; model it as a retry
                sim.pc[r] -= 1
                return
            assert site[r][s] == k, f"rank {r} consumed slice {s} of use {site[r][s]} for use {k}"
        else:
            assert all(v == op[1] for v in site[r]), f"rank {r}: site changed before its backward read of use {op[1]}"

    sim = Sim(world, programs, seed)
    sim.run(execute)


def test_reduce_scatter_staging_two_buffers():
    world, uses = 4, 6
    stage = [[[None] * world for _ in range(2)] for _ in range(world)]   # stage[owner][buffer][source] = use
    programs = []
    for r in range(world):
        prog = []
        for k in range(uses):
            for step in range(world):
                prog.append(("send", k, (r + 1 + step) % world))          # epilogue stores, own rows last
            prog.append(("barrier", k))
            prog.append(("sum", k))
        programs.append(prog)

    def execute(r, op):
        if op[0] == "send":
            stage[op[2]][op[1] % 2][r] = op[1]
        else:
            assert all(v == op[1] for v in stage[r][op[1] % 2]), f"rank {r} summed stale slots for use {op[1]}"

    Sim(world, programs, 5).run(execute)
