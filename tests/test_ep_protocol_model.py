"""The flag protocol of the expert-parallel exchange over peer memory (csrc/ep.cu: ep_push_kernel,
ep_return_kernel, ep_signal_and_wait), checked as a small state machine over every interleaving.

Per block call e a rank (1) stores its rows into slot `rank` of every rank's gather buffer, (2) writes e
into its flag word at every rank, (3) waits until its own flag words of all ranks have reached e,
(4) reads the gather buffer, (5) stores expert outputs into every home rank's output buffer, (6) writes
e into its return flag at every rank, (7) waits for the return flags, (8) reads its output buffer.
Buffers are single (no double buffering): the claim is that the two hand-shakes alone keep a fast rank
from overwriting what a slow rank still reads, and that nobody reads a slot before it is written.
The model explores all interleavings of the ranks' steps (each store, flag write and read is one
atomic step; a rank's stores precede its flag writes, as the fence in the kernel guarantees) and checks
that every read sees exactly the value of the current call."""
import itertools
from collections import deque

import pytest


def program(W, rank, calls):
    """The rank's steps in program order: (op, call, peer)."""
    steps = []
    for e in range(1, calls + 1):
        steps += [("store_x", e, d) for d in range(W)]
        steps += [("flag_g", e, d) for d in range(W)]
        steps += [("wait_g", e, None)]
        steps += [("read_x", e, s) for s in range(W)]
        steps += [("store_y", e, d) for d in range(W)]
        steps += [("flag_r", e, d) for d in range(W)]
        steps += [("wait_r", e, None)]
        steps += [("read_y", e, s) for s in range(W)]
    return steps


def explore(W, calls):
    progs = [program(W, r, calls) for r in range(W)]
    # state: pcs, X[d][r], GF[d][r], Y[d][r], RF[d][r]  (d = the rank that holds the memory, r = the writer)
    zero = tuple(tuple(0 for _ in range(W)) for _ in range(W))
    start = (tuple(0 for _ in range(W)), zero, zero, zero, zero)
    seen = {start}
    todo = deque([start])
    finished = False

    def put(m, d, r, v):
        return tuple(tuple(v if (i == d and j == r) else m[i][j] for j in range(W)) for i in range(W))

    while todo:
        pcs, X, GF, Y, RF = todo.popleft()
        if all(pcs[r] == len(progs[r]) for r in range(W)):
            finished = True
            continue
        moved = False
        for r in range(W):
            if pcs[r] == len(progs[r]):
                continue
            op, e, p = progs[r][pcs[r]]
            nX, nGF, nY, nRF = X, GF, Y, RF
            if op == "store_x":
                nX = put(X, p, r, e)
            elif op == "flag_g":
                nGF = put(GF, p, r, e)
            elif op == "wait_g":
                if any(GF[r][s] < e for s in range(W)):
                    continue
            elif op == "read_x":
                assert X[r][p] == e, ("gather buffer", r, p, e, X[r][p])
            elif op == "store_y":
                nY = put(Y, p, r, e)
            elif op == "flag_r":
                nRF = put(RF, p, r, e)
            elif op == "wait_r":
                if any(RF[r][s] < e for s in range(W)):
                    continue
            elif op == "read_y":
                assert Y[r][p] == e, ("output buffer", r, p, e, Y[r][p])
            moved = True
            npcs = tuple(pcs[i] + 1 if i == r else pcs[i] for i in range(W))
            st = (npcs, nX, nGF, nY, nRF)
            if st not in seen:
                seen.add(st)
                todo.append(st)
        assert moved, "deadlock"
    assert finished
    return len(seen)


@pytest.mark.parametrize("W,calls", [(2, 5), (3, 3), (4, 2)])
def test_every_interleaving_reads_the_current_call(W, calls):
    assert explore(W, calls) > 100


def test_the_model_catches_a_missing_handshake():
    """Without the return phase (steps 5-8) a fast rank's next stores overwrite rows a slow rank has not
    read yet: the model has to find that, or it proves nothing."""
    def broken(W, rank, calls):
        steps = []
        for e in range(1, calls + 1):
            steps += [("store_x", e, d) for d in range(W)]
            steps += [("flag_g", e, d) for d in range(W)]
            steps += [("wait_g", e, None)]
            steps += [("read_x", e, s) for s in range(W)]
        return steps
    global program
    good = program
    program = broken
    try:
        with pytest.raises(AssertionError, match="gather buffer"):
            explore(2, 2)
    finally:
        program = good
