"""Worker of tests/test_host_group_cpu.py: one gloo rank of the host AllReduce (started by torch.distributed.run)."""
import argparse
import datetime
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fp4_all_reduce_b200 import _native as N  # noqa: E402
from fp4_all_reduce_b200 import oracle as O  # noqa: E402
from fp4_all_reduce_b200.parallel.host_group import HostAllReduce, PeerTimeout  # noqa: E402
from fp4_all_reduce_b200.utils import data as D  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=37)
    ap.add_argument("--leaves", type=int, default=-1, help="this rank exits after the first call (host-made failure)")
    ns = ap.parse_args()
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
    rank, world = dist.get_rank(), dist.get_world_size()
    ar = HostAllReduce()
    xs = [D.partial(ns.rows, r) for r in range(world)]
    bits = [O.bf16_bits(x) for x in xs]
    out = {"rank": rank, "world": world, "mismatches": {}}
    for name, algo in (("oneshot", N.ALGO_ONESHOT), ("twoshot", N.ALGO_TWOSHOT)):
        got = O.bf16_bits(ar.all_reduce(xs[rank], algo=algo))
        want = O.allreduce(bits, algo=1 if algo == N.ALGO_TWOSHOT and world > 1 else 0, input_kind=0)["out"]
        out["mismatches"][name] = int(np.count_nonzero(got != want))
    # NVFP4 input with static per-rank scales
    gs = [float(np.float32(np.abs(O.bf16_bits_to_f32(b)).max()) / np.float32(2688.0)) for b in bits]
    q = [O.encode_static(b, g) for b, g in zip(bits, gs)]
    algo = N.ALGO_ONESHOT if world <= 2 else N.ALGO_TWOSHOT
    got = O.bf16_bits(ar.all_reduce(torch.from_numpy(q[rank]), algo=algo, gs=gs))
    want = O.allreduce(q, algo=0 if world <= 2 else 1, input_kind=1, gs=gs)["out"]
    out["mismatches"]["nvfp4_in"] = int(np.count_nonzero(got != want))
    if ns.leaves >= 0:
        if rank == ns.leaves:
            print(json.dumps({"rank": rank, "left": True}), flush=True)
            os._exit(0)                      # leaves between steps, nothing in flight
        try:
            ar.all_reduce(xs[rank])
            out["peer_timeout"] = False
        except PeerTimeout:
            out["peer_timeout"] = True
        print(json.dumps(out), flush=True)
        os._exit(0)                          # the group is broken: skip the collective teardown
    print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if not any(out["mismatches"].values()) else 3


if __name__ == "__main__":
    sys.exit(main())
