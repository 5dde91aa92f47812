"""NVLink micro-benchmarks, one process per GPU (2 or more ranks):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port X \
        -m fp4_all_reduce_b200.harness.micro [--mb 256] [--out micro.jsonl]

* bandwidth: every rank pushes (or pulls) `--mb` MiB to (from) its next neighbour, all ranks at once
  ("bidir": both directions of every link busy, which is what an AllReduce does) and rank 0 alone ("uni");
  methods: bulk store with several chunk sizes, st.v4, bulk load (pull), multimem.st when the fabric offers a
  multicast mapping; CTA counts 16 / 32 / 148.
* latency: ping-pong between rank 0 and rank 1; one-way = round trip / 2.  Three hand-offs: the data is the signal
  (st.volatile into the peer, poll the own memory), payload + st.release.sys flag polled with ld.acquire.sys, and
  a pull (write the own slot, poll the peer's across the link).
* publish: tiles written into the peer and published per tile (nothing / fence.acq_rel.sys + flag / st.release.sys
  flag) -> GB/s versus tile size; and nanoseconds per (remote 16-byte store + fence.acq_rel.sys) from one thread.
* tear: are 16-byte stores into a peer seen whole?  Rank 0 rewrites 4096 slots of rank 1 with {i,i,i,i} while rank 1
  polls them; counts loads whose words differ, for 16-byte and (the control) 2 x 8-byte accesses.
* copy engine: a peer copy issued by the runtime (cudaMemcpyAsync) against the SM kernels.
* link counters: `nvidia-smi nvlink -gt d` read before and after a run of bulk stores and of st.v4 stores: counted
  bytes over payload bytes (read-only; skipped with a record when the counters are not exposed).

One JSON line per configuration (GB/s of payload per direction per GPU; time = CUDA events, max over ranks).
The reference's equivalents: bench/micro/bw.cu, lat.cu, fence.cu, tear.cu, bench/link/ce.cu and their README
tables (bench/micro/README.md:48-59).
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


def nvlink_data_kib(index: int):
    """(tx KiB, rx KiB) summed over the links of GPU `index`, read from `nvidia-smi nvlink -gt d`; None when the
    tool or the counters are not available.  Reading counters changes nothing on the GPU.  (The reference brackets its
    runs the same way: bench/link/common.sh:5-6, cnt.py.)"""
    import re
    import shutil
    import subprocess

    exe = shutil.which("nvidia-smi")
    if exe is None:
        return None
    try:
        out = subprocess.run([exe, "nvlink", "-gt", "d", "-i", str(index)], capture_output=True, text=True, timeout=20).stdout
    except Exception:
        return None
    tx = [int(v) for v in re.findall(r"Data Tx:\s*(\d+)\s*KiB", out)]
    rx = [int(v) for v in re.findall(r"Data Rx:\s*(\d+)\s*KiB", out)]
    if not tx or not rx:
        return None
    return sum(tx), sum(rx)


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
    lib.fp4ar_micro_latency.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.fp4ar_micro_copy_engine.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.fp4ar_micro_publish.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.fp4ar_micro_fence_cost.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.fp4ar_micro_tear_writer.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.fp4ar_micro_tear_reader.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    total = ns.mb << 20
    buf, ptrs, handle = allocate_symmetric(total + (1 << 17), dev, dist.group.WORLD)
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
    # wire bytes against payload bytes from the link counters (256-byte bulk-store packets against 128-byte st.v4 ones)
    for method, chunk in ((0, 4096), (1, 4096)):
        torch.cuda.synchronize()
        dist.barrier()
        before = nvlink_data_kib(local) if rank == 0 else None
        reps = 8
        for _ in range(reps):
            N.check(lib.fp4ar_micro_bandwidth(ptrs[nxt], total, chunk, method, 148, 4 if method == 0 else 1, stream()), "micro_bw")
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            after = nvlink_data_kib(local)
            if before is None or after is None:
                emit({"kind": "nvlink_counters", "method": names[method], "skipped": "nvidia-smi nvlink counters not available"})
            else:
                payload = reps * (total // chunk) * chunk
                tx = (after[0] - before[0]) * 1024
                rx = (after[1] - before[1]) * 1024
                emit({"kind": "nvlink_counters", "method": names[method], "chunk": chunk, "payload_bytes_sent": payload,
                      "counter_tx_bytes": tx, "counter_rx_bytes": rx, "tx_over_payload": round(tx / payload, 4) if payload else None})

    def timed(launch, active):
        """min over iterations of the CUDA-event time of `launch`, max over ranks."""
        times = []
        for it in range(ns.iters + 2):
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if active == "bidir" or rank == 0:
                launch()
            b.record()
            b.synchronize()
            if it >= 2:
                times.append(a.elapsed_time(b))
        t = torch.tensor([min(times)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # copy engine: a peer copy issued by the runtime (cudaMemcpyAsync) instead of an SM kernel
    src = torch.empty(total, dtype=torch.uint8, device=dev)
    for active in ("bidir", "uni"):
        for name, d, s_ in (("copy_engine_push", ptrs[nxt], src.data_ptr()), ("copy_engine_pull", src.data_ptr(), ptrs[nxt])):
            ms = timed(lambda: N.check(lib.fp4ar_micro_copy_engine(d, s_, total, stream()), "copy_engine"), active)
            emit({"kind": "bw", "method": name, "chunk": total, "ctas": 0, "inflight": 1, "active": active,
                  "tp": world, "mb": ns.mb, "ms": round(ms, 4), "gbs_per_dir": round(total / ms / 1e6, 1)})
    del src

    # publication cost per tile
    flags_off = total
    for tile in (1024, 4096, 16384, 65536):
        base = None
        for mode, mname in ((0, "none"), (1, "fence_acq_rel_sys+flag"), (2, "st_release_sys_flag")):
            ms = timed(lambda: N.check(lib.fp4ar_micro_publish(ptrs[nxt], ptrs[nxt] + flags_off, total, tile, mode, 148,
                                                               stream()), "micro_publish"), "bidir")
            base = ms if mode == 0 else base
            emit({"kind": "publish", "publish": mname, "tile": tile, "ctas": 148, "tp": world, "ms": round(ms, 4),
                  "gbs_per_dir": round(total / ms / 1e6, 1), "vs_unpublished": round(ms / base, 3)})
    out1 = torch.zeros(1, dtype=torch.int64, device=dev)
    fence_ns = {}
    for wf in (0, 1):
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            N.check(lib.fp4ar_micro_fence_cost(ptrs[nxt], 4000, wf, out1.data_ptr(), stream()), "micro_fence_cost")
            torch.cuda.synchronize()
            fence_ns[wf] = int(out1.item()) / 4000
    if rank == 0:
        emit({"kind": "fence", "ns_per_remote_store": round(fence_ns[0], 1),
              "ns_per_remote_store_plus_fence_acq_rel_sys": round(fence_ns[1], 1)})

    # latency between rank 0 and rank 1
    slots = buf[total:total + (1 << 17)]
    iters = 2000
    out3 = torch.zeros(3, dtype=torch.int64, device=dev)
    for method, mname in ((0, "data_is_signal_st_volatile"), (1, "payload+st_release_sys_flag"), (2, "pull_poll_peer")):
        slots.zero_()
        out3.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        if rank < 2:
            my_slot = ptrs[rank] + total
            peer_slot = ptrs[1 - rank] + total
            N.check(lib.fp4ar_micro_latency(my_slot, peer_slot, iters, 1 if rank == 0 else 0, method, 1000, out3.data_ptr(),
                                            stream()), "micro_latency")
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            ns_total, gave_up = int(out3[0].item()), int(out3[1].item())
            emit({"kind": "latency", "method": mname, "iters": iters, "one_way_us": round(ns_total / iters / 2 / 1e3, 3),
                  "gave_up": gave_up})

    # tear: rank 0 writes into rank 1, rank 1 polls its own memory; neither waits for the other
    nslots = 4096
    out2 = torch.zeros(2, dtype=torch.int64, device=dev)
    for how, hname in ((0, "16B_store_16B_load"), (1, "2x8B_store_2x8B_load")):
        slots.zero_()
        out2.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            N.check(lib.fp4ar_micro_tear_writer(ptrs[1] + total, nslots, 3000, how, stream()), "tear_writer")
        elif rank == 1:
            N.check(lib.fp4ar_micro_tear_reader(ptrs[1] + total, nslots, 3000, how, out2.data_ptr(), stream()), "tear_reader")
        torch.cuda.synchronize()
        res = out2.clone()
        dist.broadcast(res, src=1)
        if rank == 0:
            emit({"kind": "tear", "access": hname, "slots": nslots, "polls_per_slot": 3000, "torn_loads": int(res[0].item()),
                  "value_changes_seen": int(res[1].item())})
    if rank == 0 and ns.out:
        with open(ns.out, "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
