"""The flag protocol of the symmetric-memory exchange (muse_moe_w4a16/ep.py, SymmExchange.step),
replayed on the CPU as a discrete-event model: every rank has its main stream and its copy
stream, each a FIFO of the operations step() enqueues (flag writes and waits, event records and
waits, peer copies, the expert chunks, the combine). A random scheduler runs whichever stream
heads are runnable, so ranks drift apart as far as the protocol lets them. Checked for several
(ranks, chunks): nothing deadlocks, every copy and every kernel reads rows of the step it belongs
to, and no buffer is overwritten while a copy or a kernel that started on it is still running.
"""
import random

import pytest


def build_rank_program(r, n, chunks, steps):
    """The two operation lists of rank r for `steps` steps, in the order step() enqueues them.
    chunks: None (the default layout), a number of equal chunks, or the chunk sizes (chunk_sizes)."""
    from muse_moe_w4a16.ep import chunk_sizes

    sizes = chunk_sizes(n, chunks)
    bounds = [0]
    for m in sizes:
        bounds.append(bounds[-1] + m)
    s0, s1 = [], []
    for e in range(1, steps + 1):
        b = e & 1
        ev = lambda name: (r, e, name)

        def run_chunk(c):
            reads = [("gx", r, b, j) for j in range(bounds[c], bounds[c + 1])]
            writes = [("part", r, b, j) for j in range(bounds[c], bounds[c + 1])]
            s0.append(("kernel", reads, writes, e))
            for j in range(max(bounds[c], 1), bounds[c + 1]):
                s0.append(("flag_write", (r + j) % n, 2 * n + 2 * r + b, e))

        # main stream: inputs into slot 0, tell the peers
        s0.append(("produce", ("gx", r, b, 0), e))
        s0.append(("record", ev("in")))
        for j in range(1, n):
            s0.append(("flag_write", (r + j) % n, 2 * r + b, e))
        # a first chunk of the own rows alone is issued before the copy stream's calls
        own_first = sizes[0] == 1
        if own_first:
            run_chunk(0)
        # copy stream: pull the other ranks' rows
        s1.append(("wait_event", ev("in")))
        ready = {}
        for j in range(1, n):
            p = (r + j) % n
            s1.append(("flag_wait", 2 * p + b, e))
            s1.append(("copy", ("gx", p, b, 0), ("gx", r, b, j), e))
            if j + 1 in bounds:
                c = bounds.index(j + 1) - 1
                ready[c] = ev(("ready", c))
                s1.append(("record", ready[c]))
        # main stream: the other expert chunks
        for c in range(1 if own_first else 0, len(sizes)):
            if c in ready:
                s0.append(("wait_event", ready[c]))
            run_chunk(c)
        # copy stream: pull this rank's partial rows back
        for j in range(1, n):
            q = (r - j) % n
            s1.append(("flag_wait", 2 * n + 2 * q + b, e))
            s1.append(("copy", ("part", q, b, j), ("back", r, 0, q), e))
        s1.append(("record", ev("back")))
        s0.append(("wait_event", ev("back")))
        s0.append(("kernel", [("back", r, 0, q) for q in range(n) if q != r] + [("part", r, b, 0)], [], e))
    return s0, s1


def simulate(n, chunks, steps, seed):
    rng = random.Random(seed)
    queues = {}
    for r in range(n):
        s0, s1 = build_rank_program(r, n, chunks, steps)
        queues[(r, 0)], queues[(r, 1)] = list(s0), list(s1)
    flags = [[0] * (4 * n) for _ in range(n)]
    events = set()
    content = {}      # buffer -> step whose rows it holds
    readers = {}      # buffer -> number of running copies / kernels reading it
    writers = {}      # buffer -> number of running copies / kernels writing it
    running = {}      # stream -> (op, remaining ticks)

    def start(key, op):
        kind = op[0]
        if kind in ("produce",):
            reads, writes, e = [], [op[1]], op[2]
        elif kind == "copy":
            reads, writes, e = [op[1]], [op[2]], op[3]
        else:
            reads, writes, e = op[1], op[2], op[3]
        for buf in reads:
            assert content.get(buf) == e, f"{key} {kind} of step {e} reads {buf} holding step {content.get(buf)}"
            assert writers.get(buf, 0) == 0, f"{key} reads {buf} while it is being written"
            readers[buf] = readers.get(buf, 0) + 1
        for buf in writes:
            assert readers.get(buf, 0) == 0, f"{key} overwrites {buf} of step {content.get(buf)} while it is being read"
            assert writers.get(buf, 0) == 0
            writers[buf] = writers.get(buf, 0) + 1
        running[key] = (reads, writes, e, rng.randint(1, 6))

    def finish(key):
        reads, writes, e, _ = running.pop(key)
        for buf in reads:
            readers[buf] -= 1
        for buf in writes:
            writers[buf] -= 1
            content[buf] = e

    while any(queues.values()) or running:
        progressed = False
        keys = list(queues.keys())
        rng.shuffle(keys)
        for key in keys:
            if key in running:
                reads, writes, e, left = running[key]
                if left > 1 and rng.random() < 0.7:
                    running[key] = (reads, writes, e, left - 1)
                else:
                    finish(key)
                progressed = True
                continue
            if not queues[key]:
                continue
            op = queues[key][0]
            kind = op[0]
            if kind == "flag_wait" and flags[key[0]][op[1]] < op[2]:
                continue
            if kind == "wait_event" and op[1] not in events:
                continue
            if rng.random() < 0.35:      # this stream idles a tick: lets the ranks drift apart
                progressed = True
                continue
            queues[key].pop(0)
            progressed = True
            if kind == "flag_write":
                flags[op[1]][op[2]] = max(flags[op[1]][op[2]], op[3])
            elif kind == "record":
                events.add(op[1])
            elif kind in ("produce", "copy", "kernel"):
                start(key, op)
        assert progressed, "deadlock: " + str({k: q[0] for k, q in queues.items() if q})


@pytest.mark.parametrize("n,chunks", [(2, 1), (2, 2), (4, 1), (4, 2), (4, 4), (8, 2), (8, 4), (8, 8), (6, 3),
                                      (3, None), (4, None), (5, None), (8, None), (8, (1, 3, 3, 1)), (8, (3, 4, 1))])
def test_exchange_protocol_neither_deadlocks_nor_mixes_steps(n, chunks):
    for seed in range(6):
        simulate(n, chunks, steps=4, seed=seed)


def test_simulator_catches_a_protocol_without_the_partial_ready_flags():
    """The model is not vacuous: without the waits on the "partial rows written" flags a rank pulls
    rows its peer has not produced yet, and the simulator says so."""
    scope = simulate.__globals__
    original = scope["build_rank_program"]

    def no_back_waits(r, n, chunks, steps):
        s0, s1 = original(r, n, chunks, steps)
        return s0, [op for op in s1 if not (op[0] == "flag_wait" and op[1] >= 2 * n)]

    scope["build_rank_program"] = no_back_waits
    try:
        failures = 0
        for seed in range(20):
            try:
                simulate(4, 2, steps=4, seed=seed)
            except AssertionError:
                failures += 1
        assert failures > 0
    finally:
        scope["build_rank_program"] = original
