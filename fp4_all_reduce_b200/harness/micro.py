"""NVLink micro-benchmarks, one process per GPU (2 or more ranks):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port X \
        -m fp4_all_reduce_b200.harness.micro [--mb 256] [--out micro.jsonl]

* bandwidth: every rank pushes (or pulls) `--mb` MiB to (from) its next neighbour, all ranks at once
  ("bidir": both directions of every link busy, which is what an AllReduce does) and rank 0 alone ("uni");
  methods: bulk store with several chunk sizes, st.v4, bulk load (pull), multimem.st when the fabric offers a
  multicast mapping; CTA counts 16 / 32 / 148.
* latency: ping-pong between rank 0 and rank 1 through polled slots; one-way = round trip / 2.

One JSON line per configuration (GB/s of payload per direction per GPU; time = CUDA events, max over ranks).
The reference's equivalents: bench/micro/bw.cu, lat.cu and their README tables (bench/micro/README.md:48-59).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import _native as N
from ..parallel.symmetric import allocate_symmetric, multicast_pointer


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default=None)
    ns = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = N.cuda()
    lib.fp4ar_micro_bandwidth.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.fp4ar_micro_latency.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    total = ns.mb << 20
    buf, ptrs, handle = allocate_symmetric(total + 4096, dev, dist.group.WORLD)
    mc = multicast_pointer(handle)
    nxt = (rank + 1) % world
    stream = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    records = []

    def emit(r):
        records.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    def run(method, chunk, ctas, inflight, active):
        """active: 'bidir' every rank runs, 'uni' only rank 0."""
        times = []
        for it in range(ns.iters + 2):
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if active == "bidir" or rank == 0:
                target = mc if method == 3 else ptrs[nxt]
                N.check(lib.fp4ar_micro_bandwidth(target, total, chunk, method, ctas, inflight, stream()), "micro_bw")
            b.record()
            b.synchronize()
            if it >= 2:
                times.append(a.elapsed_time(b))
        t = torch.tensor([min(times)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    names = {0: "bulk_store", 1: "st_v4", 2: "bulk_load_pull", 3: "multimem_st"}
    for active in ("bidir", "uni"):
        for method, chunk, ctas, inflight in ((0, 3472, 148, 4), (0, 3584, 148, 4), (0, 4096, 148, 4), (0, 4096, 32, 4),
                                              (0, 4096, 16, 4), (0, 16384, 148, 2), (0, 1024, 148, 8), (0, 256, 148, 16),
                                              (1, 4096, 148, 1), (1, 4096, 32, 1), (2, 4096, 148, 1), (2, 16384, 148, 1),
                                              (3, 4096, 148, 1)):
            if method == 3 and (not mc or active == "uni"):
                continue
            ms = run(method, chunk, ctas, inflight, active)
            moved = (total // chunk) * chunk
            emit({"kind": "bw", "method": names[method], "chunk": chunk, "ctas": ctas, "inflight": inflight, "active": active,
                  "tp": world, "mb": ns.mb, "ms": round(ms, 4), "gbs_per_dir": round(moved / ms / 1e6, 1)})
    # latency between rank 0 and rank 1
    slots = buf[total:total + 4096]
    slots.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    out2 = torch.zeros(2, dtype=torch.int64, device=dev)
    iters = 2000
    if rank < 2:
        my_slot = ptrs[rank] + total
        peer_slot = ptrs[1 - rank] + total      # each rank polls a slot in its own buffer and writes the peer's
        N.check(lib.fp4ar_micro_latency(my_slot, peer_slot, iters, 1 if rank == 0 else 0, 2000, out2.data_ptr(), stream()),
                "micro_latency")
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        ns_total, gave_up = int(out2[0].item()), int(out2[1].item())
        emit({"kind": "latency", "method": "polled_slot_st_volatile", "iters": iters, "one_way_us": round(ns_total / iters / 2 / 1e3, 3),
              "gave_up": gave_up})
    if rank == 0 and ns.out:
        with open(ns.out, "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
