"""Worker of tests/test_custom_ops_gpu.py::test_linear_all_reduce_norm_op_on_two_gpus (run under torch.distributed.run,
one process per GPU).  Calls the custom ops on a real tensor-parallel group and prints one JSON line per op with the
number of output elements that differ from the host model (summed over the ranks)."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fp4_all_reduce_b200 import _native as N          # noqa: E402
from fp4_all_reduce_b200 import oracle as O           # noqa: E402
from fp4_all_reduce_b200.ops import allreduce as A    # noqa: E402
from fp4_all_reduce_b200.ops import gemm as G         # noqa: E402
from fp4_all_reduce_b200.parallel.context import Fp4ArContext  # noqa: E402
from fp4_all_reduce_b200.utils import data as D       # noqa: E402


def main() -> int:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    rows = 320
    ctx = Fp4ArContext(rows, device=dev)
    cid = A.register_context(ctx)
    algo = 0 if world <= 2 else 1

    def total(v):
        t = torch.tensor([v], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        return int(t.item())

    def diff(t, want):
        got = O.bf16_bits(t) if t.dtype == torch.bfloat16 else t.cpu().numpy()
        return int(np.count_nonzero(got != want))

    def report(op, mism):
        m = total(mism)
        if rank == 0:
            print(json.dumps({"op": op, "tp": world, "rows": rows, "mismatches": m, "status": ctx.status().describe()}), flush=True)

    xs = [D.partial(rows, r) for r in range(world)]
    bits = [O.bf16_bits(x) for x in xs]
    res = D.residual(rows).to(dev)
    w = D.norm_weight().to(dev)
    rb, wb = O.bf16_bits(res), O.bf16_bits(w)
    x = xs[rank].to(dev)

    y = torch.ops.fp4ar.all_reduce(x, cid)
    torch.cuda.synchronize()
    report("all_reduce", diff(y, O.allreduce(bits, algo=algo)["out"]))

    r1 = res.clone()
    y = torch.ops.fp4ar.all_reduce_add_rms_norm(x, r1, w, 1e-6, 1.0, cid)
    torch.cuda.synchronize()
    want = O.allreduce(bits, algo=algo, epi=1, res_in=rb, weight=wb, eps=1e-6, wbias=1.0)
    report("all_reduce_add_rms_norm", diff(y, want["out"]) + diff(r1, want["res_out"]))

    # row-parallel linear: X [rows, K] @ Wt [6144, K]^T on every rank, partial quantised with a static scale in the
    # GEMM's epilogue and pushed into the peers' windows, then AllReduce + residual + norm
    K = 1024
    g = torch.Generator().manual_seed(300 + rank)
    xk = torch.randn(rows, K, generator=g).to(torch.bfloat16).to(dev)
    wt = (torch.randn(N.HIDDEN, K, generator=g) / (K * world) ** 0.5).to(torch.bfloat16).to(dev)
    mine = torch.tensor([G.calibrate_gs(xk, wt)], device=dev)
    alls = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(alls, mine)
    gs = [float(a.item()) for a in alls]
    lq = torch.ops.fp4ar.linear_nvfp4(xk, wt, gs[rank])          # this rank's NVFP4 partial, for the host model
    allq = [torch.empty_like(lq) for _ in range(world)]
    dist.all_gather(allq, lq)
    r2 = res.clone()
    y = torch.ops.fp4ar.linear_all_reduce_add_rms_norm(xk, wt, gs, r2, w, 1e-6, 1.0, cid)
    torch.cuda.synchronize()
    want = O.allreduce([q.cpu().numpy() for q in allq], algo=algo, input_kind=1, gs=gs, epi=1, res_in=rb, weight=wb,
                       eps=1e-6, wbias=1.0)
    report("linear_all_reduce_add_rms_norm", diff(y, want["out"]) + diff(r2, want["res_out"]) + int(G.gemm_status().code != 0))

    ok = ctx.status().ok
    A.unregister_context(cid)
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 4


if __name__ == "__main__":
    sys.exit(main())
