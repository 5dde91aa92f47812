"""A randomised model of the partial-tile hand-off of the stream-K GEMM (no GPU), after csrc/kernels/gemm_fp4.cu.

Unit u + 1 leaves the FP32 partial of a tile it shares with unit u in ITS slot and sets the slot's flag with a
release store; unit u waits for the flag (acquire), adds the partial, and resets the flag with a release store once
every lane has the data in registers.  Slots and flags belong to the device, not to a launch, so launch L + 1 reuses
them; its producer first waits until the flag is 0.  Launches on one stream follow one another, but with programmatic
dependent launch (or two streams) units of launch L + 1 can run while units of launch L are still at work, which is
what the model lets happen: every unit of every launch is its own thread of control and a random scheduler
interleaves them, subject only to "a unit of launch L + 1 starts after the SAME unit index of launch L has finished"
(an SM holds one CTA of this kernel at a time).

Checked on every schedule: a producer never overwrites a partial that has not been consumed; a consumer only ever
reads the partial of its own launch, complete; every flag is 0 at the end; nobody waits forever.  `variant` removes
one rule to show that the checker can fail: "no_free_wait" (the producer does not wait for flag == 0) and
"early_reset" (the consumer resets the flag before it has read the data) must both produce violations.
"""
from __future__ import annotations

import random


class Violation(AssertionError):
    pass


def run(units: int, launches: int, seed: int, variant: str = "product", words: int = 3, max_steps: int = 200000) -> None:
    rng = random.Random(seed)
    flag = [0] * units                       # flag of slot s (slot s is written by unit s, read by unit s - 1)
    slot = [[None] * words for _ in range(units)]
    # which units share a tile: in a launch unit u consumes from u + 1 iff shared[L][u]; random per launch
    shared = [[rng.random() < 0.7 for _ in range(units - 1)] + [False] for _ in range(launches)]
    # program of (launch, unit): produce (if unit u - 1 consumes from u) FIRST, then consume (if shared) LAST
    pc = {}
    for L in range(launches):
        for u in range(units):
            ops = []
            if u > 0 and shared[L][u - 1]:
                if variant != "no_free_wait":
                    ops.append(("wait_free", u))
                ops += [("write", u, w) for w in range(words)] + [("set", u)]
            ops.append(("work",))
            if shared[L][u]:
                ops.append(("wait_full", u + 1))
                if variant == "early_reset":
                    ops.append(("reset", u + 1))
                ops += [("read", u + 1, w) for w in range(words)]
                if variant != "early_reset":
                    ops.append(("reset", u + 1))
            pc[(L, u)] = [ops, 0]
    done = set()
    steps = 0
    while len(done) < launches * units:
        steps += 1
        if steps > max_steps:
            raise Violation("no progress: a wait never ends")
        ready = [(L, u) for (L, u), (ops, i) in pc.items() if (L, u) not in done and (L == 0 or (L - 1, u) in done)]
        L, u = rng.choice(ready)
        ops, i = pc[(L, u)]
        op = ops[i]
        advance = True
        if op[0] == "wait_free":
            advance = flag[op[1]] == 0
        elif op[0] == "write":
            s, w = op[1], op[2]
            if flag[s] != 0:
                raise Violation(f"launch {L} unit {u} overwrites slot {s} whose partial has not been consumed")
            slot[s][w] = (L, w)
        elif op[0] == "set":
            flag[op[1]] = 1
        elif op[0] == "wait_full":
            advance = flag[op[1]] == 1
        elif op[0] == "read":
            s, w = op[1], op[2]
            if slot[s][w] != (L, w):
                raise Violation(f"launch {L} unit {u} read {slot[s][w]} from slot {s} word {w}")
        elif op[0] == "reset":
            flag[op[1]] = 0
        if advance:
            pc[(L, u)][1] = i + 1
            if i + 1 == len(ops):
                done.add((L, u))
    if any(flag):
        raise Violation("a flag is still set at the end")


def check(units: int, launches: int, seeds: int = 200, variant: str = "product") -> int:
    """Number of seeds (out of `seeds`) on which the model found a violation."""
    bad = 0
    for seed in range(seeds):
        try:
            run(units, launches, seed, variant)
        except Violation:
            bad += 1
    return bad
