"""A small randomised model checker for the window hand-off protocol of the fused AllReduce (no GPU).

What is modelled, after csrc/kernels/ar_kernel.cuh and csrc/runtime/runtime.cu:

  * every rank owns a window of `nbuf` buffers (2 in the product) of slots that hold either SENTINEL or one record;
  * call c uses buffer c % nbuf; a rank walks its rows as the kernel's software pipeline does (step k: two-shot owner
    step of row k - lag_o, push of row k, finish of row k - lag_f; one-shot: push row k, finish row k - 1);
  * every store (a push into a peer's slot, the consumer's sentinel re-arm of its own slot) is ASYNCHRONOUS: it lands
    at an arbitrary later moment, in any order relative to other stores, but before the issuing rank's call ends (the
    kernel waits for its bulk stores before it exits);
  * a consumer polls a slot until it is not SENTINEL, uses it, and re-arms it;
  * ranks run at arbitrary relative speeds (a random scheduler, optionally starving one rank for long stretches).

What is checked on every schedule:

  * a record that lands finds its slot armed (SENTINEL): nothing unconsumed is ever overwritten;
  * a re-arm that lands finds the very record its issuer consumed: it never erases newer data;
  * every record a consumer accepts is the one it waits for (same call, source, row): nothing stale is consumed;
  * the system never deadlocks, and at the end every slot of every window is SENTINEL again.

`variant` switches one protocol rule off to show that the checker can fail: "one_buffer" (no call parity) and
"no_drain" (a call may end before its own stores have landed) must both produce violations.  So must
"empty_call_bumps": a call that exchanges nothing (zero rows) but still advances the call counter lets a fast rank
reach the buffer parity that a slow rank is still consuming; the runtime therefore launches nothing for a zero-row
call ("empty_call_skipped", safe), and loop-back (compute-mode) calls, which do advance the counter, need a barrier
before the next fused call.

The reference project argues the same properties on paper (docs/DESIGN.md:122-128) and probes them with rotating
input sets and skewed ranks on GPUs; this is the exhaustive-in-spirit counterpart that needs no GPU and is where a
"rank that stops pushing" is exercised (`dead_rank`): the others' bounded waits give up and report, nobody hangs.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Callable, Optional

SENT = None


class Violation(AssertionError):
    pass


@dataclass
class Store:
    issuer: int
    dst: int
    buf: int
    slot: tuple
    value: Optional[tuple]          # a record (call, kind, src, row) or SENT for a re-arm
    expect: Optional[tuple] = None  # for a re-arm: the record that was consumed


@dataclass
class Model:
    P: int
    rows: int
    calls: int
    two_shot: bool = False
    lag_o: int = 1
    lag_f: int = 2
    nbuf: int = 2
    drain: bool = True
    seed: int = 0
    starve: bool = False
    dead_rank: int = -1             # this rank stops before pushing anything in call `dead_call`
    dead_call: int = 0
    wait_limit: int = 2000          # scheduler steps a blocked wait may last when a rank is dead
    empty_calls: tuple = ()         # program positions at which every rank issues a call that exchanges nothing
    empty_bumps: bool = False       # whether such a call advances the device call counter (the buffer parity)
    rng: random.Random = field(init=False)
    win: list = field(init=False)
    inflight: list = field(init=False)
    gave_up: list = field(init=False)
    clock: int = 0

    def __post_init__(self):
        self.rng = random.Random(self.seed)
        self.win = [[dict() for _ in range(self.nbuf)] for _ in range(self.P)]
        self.inflight = []
        self.gave_up = []

    # ------------------------------------------------------------------ stores
    def issue(self, st: Store):
        self.inflight.append(st)

    def land(self, st: Store):
        cur = self.win[st.dst][st.buf].get(st.slot, SENT)
        if st.value is SENT:
            if cur != st.expect:
                raise Violation(f"re-arm by rank {st.issuer} of slot {st.slot} (buffer {st.buf}) found {cur}, consumed {st.expect}")
            self.win[st.dst][st.buf].pop(st.slot, None)
        else:
            if cur is not SENT:
                raise Violation(f"record {st.value} from rank {st.issuer} landed on unconsumed {cur} in slot {st.slot} of rank {st.dst}")
            self.win[st.dst][st.buf][st.slot] = st.value

    # ------------------------------------------------------------------ one rank
    def rank_program(self, me: int):
        P, R = self.P, self.rows
        counter = 0                      # the device call counter of this rank
        for pos in range(self.calls):
            if me == self.dead_rank and pos >= self.dead_call:
                return
            if pos in self.empty_calls:
                # a call with nothing to exchange (zero rows; or a loop-back call, which only touches the own window)
                if self.empty_bumps:
                    counter += 1
                yield None
                continue
            c = counter
            counter += 1
            buf = c % self.nbuf

            def push(dst, slot, rec):
                self.issue(Store(me, dst, buf, slot, rec))

            def consume(slot, want):
                """Generator: wait for `want` in the own slot, check it, issue the re-arm."""
                t0 = self.clock
                while self.win[me][buf].get(slot, SENT) is SENT:
                    if self.dead_rank >= 0 and self.clock - t0 > self.wait_limit:
                        self.gave_up.append((me, c, slot))
                        return False
                    yield lambda: self.win[me][buf].get(slot, SENT) is not SENT or (
                        self.dead_rank >= 0 and self.clock - t0 > self.wait_limit)
                got = self.win[me][buf].get(slot, SENT)
                if got is SENT:
                    self.gave_up.append((me, c, slot))
                    return False
                if got != want:
                    raise Violation(f"rank {me} call {c} consumed {got} while waiting for {want}")
                self.issue(Store(me, me, buf, slot, SENT, expect=got))
                return True

            lag_o = self.lag_o if self.two_shot else 0
            lag_f = self.lag_f if self.two_shot else 1
            for k in range(R + lag_f):
                yield None
                if self.two_shot:
                    ko = k - lag_o
                    if 0 <= ko < R and ko % P == me:                      # owner step
                        ok = True
                        for s in range(P):
                            if s != me:
                                ok = (yield from consume(("rs", s, ko), (c, "rs", s, ko))) and ok
                        if ok:
                            for d in range(P):
                                if d != me:
                                    push(d, ("ag", me, ko), (c, "ag", me, ko))
                    if k < R and k % P != me:                             # push row k to its owner
                        push(k % P, ("rs", me, k), (c, "rs", me, k))
                    kf = k - lag_f
                    if 0 <= kf < R and kf % P != me:                      # finish a row owned by a peer
                        yield from consume(("ag", kf % P, kf), (c, "ag", kf % P, kf))
                else:
                    if k < R:
                        for d in range(P):
                            if d != me:
                                push(d, ("os", me, k), (c, "os", me, k))
                    kf = k - 1
                    if 0 <= kf < R:
                        for s in range(P):
                            if s != me:
                                yield from consume(("os", s, kf), (c, "os", s, kf))
            if self.drain:                                                 # the kernel waits for its stores before it ends
                while any(st.issuer == me for st in self.inflight):
                    yield lambda: not any(st.issuer == me for st in self.inflight)

    # ------------------------------------------------------------------ scheduler
    def run(self, max_steps: int = 2_000_000) -> dict:
        progs = [self.rank_program(r) for r in range(self.P)]
        cond: list[Optional[Callable[[], bool]]] = [None] * self.P
        alive = [True] * self.P
        starved, starve_left = -1, 0
        for _ in range(max_steps):
            self.clock += 1
            runnable = [r for r in range(self.P) if alive[r] and (cond[r] is None or cond[r]())]
            if self.starve:
                if starve_left == 0 and self.rng.random() < 0.02:
                    starved, starve_left = self.rng.randrange(self.P), self.rng.randrange(50, 400)
                if starve_left > 0:
                    starve_left -= 1
                    others = [r for r in runnable if r != starved]
                    if others or self.inflight:
                        runnable = others
            choices = len(runnable) + len(self.inflight)
            if choices == 0:
                if not any(alive):
                    break
                if self.dead_rank >= 0:
                    continue                       # only the clock moves: blocked waits run into their limit
                raise Violation(f"deadlock: ranks {[r for r in range(self.P) if alive[r]]} blocked, nothing in flight")
            pick = self.rng.randrange(choices)
            if pick < len(runnable):
                r = runnable[pick]
                try:
                    cond[r] = next(progs[r])
                except StopIteration:
                    alive[r] = False
            else:
                self.land(self.inflight.pop(pick - len(runnable)))
        else:
            raise Violation("step limit reached")
        while self.inflight and not self.drain:    # stores of a variant without the drain rule still land eventually
            self.land(self.inflight.pop(self.rng.randrange(len(self.inflight))))
        leftovers = sum(len(b) for w in self.win for b in w)
        if leftovers and self.dead_rank < 0:
            raise Violation(f"{leftovers} slots are not re-armed at the end")
        return {"steps": self.clock, "gave_up": len(self.gave_up), "leftover_slots": leftovers}


def check(P: int, rows: int, calls: int, *, two_shot: bool, lag_o: int = 1, lag_f: int = 2, seeds: int = 200,
          variant: str = "product", starve: bool = True) -> dict:
    """Run `seeds` random schedules; returns {'schedules', 'violations', 'first'}."""
    nbuf = 1 if variant == "one_buffer" else 2
    drain = variant != "no_drain"
    empty = tuple(range(1, calls, 2)) if variant.startswith("empty_call") else ()
    bad, first = 0, None
    for s in range(seeds):
        m = Model(P, rows, calls, two_shot=two_shot, lag_o=lag_o, lag_f=lag_f, nbuf=nbuf, drain=drain, seed=s,
                  starve=starve and s % 2 == 1, empty_calls=empty, empty_bumps=variant == "empty_call_bumps")
        try:
            m.run()
        except Violation as e:
            bad += 1
            first = first or f"seed {s}: {e}"
    return {"schedules": seeds, "violations": bad, "first": first}


def main(argv=None) -> int:
    import argparse
    import json

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ranks", default="2,4,8")
    ap.add_argument("--calls", type=int, default=6)
    ap.add_argument("--seeds", type=int, default=100)
    ns = ap.parse_args(argv)
    rc = 0
    for P in (int(p) for p in ns.ranks.split(",")):
        for two_shot, lags in ((False, [(0, 1)]), (True, [(1, 2), (2, 3), (2, 4), (3, 4)])):
            for lo, lf in lags:
                for variant in ("product", "one_buffer", "no_drain"):
                    # the product must be safe for every row count; a broken rule shows with few rows per team, where
                    # the pipeline order alone no longer keeps a fast rank behind a slow one
                    total = {"schedules": 0, "violations": 0, "first": None}
                    for rows in ((1, 2, 3, 7) if variant == "product" else (1, 2)):
                        r = check(P, rows, ns.calls, two_shot=two_shot, lag_o=lo, lag_f=lf, seeds=ns.seeds, variant=variant)
                        total["schedules"] += r["schedules"]
                        total["violations"] += r["violations"]
                        total["first"] = total["first"] or r["first"]
                    expect_bad = variant != "product"
                    ok = (total["violations"] > 0) == expect_bad
                    rc |= 0 if ok else 1
                    print(json.dumps({"kind": "protocol_model", "ranks": P, "two_shot": two_shot, "lags": [lo, lf],
                                      "variant": variant, **total, "as_expected": ok}), flush=True)
    return rc


if __name__ == "__main__":
    import sys

    sys.exit(main())
