"""Failure detection without faulting a GPU: a rank whose peer never pushes must give up after the
configured limit, report where it waited, finish the kernel and leave the CUDA context usable.

The "missing peer" is made on the host: a two-rank context is created on one GPU and only rank 0 is ever
launched, so the slots it polls simply stay sentinels (a flag that nothing sets)."""
import ctypes as C
import time

import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200.harness.gate import CellConfig, gate_cell_emulated
from fp4_all_reduce_b200.parallel.context import make_args
from fp4_all_reduce_b200.utils import data as D

pytestmark = pytest.mark.gpu


def _lonely_rank0(nranks, rows):
    lib = N.cuda()
    nbytes = int(lib.fp4ar_window_bytes(rows, N.HIDDEN, nranks))
    wins = [torch.empty(nbytes, dtype=torch.uint8, device="cuda:0") for _ in range(nranks)]
    for w in wins[1:]:
        w.zero_()
    ptrs = (C.c_void_p * nranks)(*[w.data_ptr() for w in wins])
    ctx = C.c_void_p()
    N.check(lib.fp4ar_create(C.byref(ctx), 0, nranks, 0, rows, N.HIDDEN, ptrs, nbytes), "create")
    return lib, ctx, wins


@pytest.mark.parametrize("nranks", [2, 4])
def test_missing_peer_times_out_with_a_status(nranks):
    rows = 64
    lib, ctx, wins = _lonely_rank0(nranks, rows)
    N.check(lib.fp4ar_set_timeout_ms(ctx, 50), "timeout")
    x = D.partial(rows, 0).cuda()
    out = torch.zeros_like(x)
    args = (N.Args * 1)(make_args(x=x, out=out, rows=rows))
    t0 = time.time()
    N.check(lib.fp4ar_launch(ctx, args, None), "launch")
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert dt < 5.0, f"the kernel took {dt:.2f} s; waits must give up after about the 50 ms limit"
    st = N.StatusWords()
    N.check(lib.fp4ar_status(ctx, 0, C.byref(st)), "status")
    assert st.code == 1 and st.count >= 1
    assert st.source != 0 and st.source < nranks
    assert st.detail in (1, 2, 3)
    # the CUDA context is alive and other work is still correct
    y = (torch.ones(1024, device="cuda:0") * 2).sum().item()
    assert y == 2048.0
    # the context refuses further calls (its window is no longer consistent) until it is reset
    assert lib.fp4ar_launch(ctx, args, None) == 4
    with pytest.raises(N.ContextPoisoned):
        N.check(lib.fp4ar_launch(ctx, args, None), "launch")
    N.check(lib.fp4ar_reset(ctx), "reset")
    N.check(lib.fp4ar_status(ctx, 0, C.byref(st)), "status")
    assert st.code == 0
    # after the reset a launch is accepted again (zero rows: accepted without a kernel, the peer is still absent)
    zero = (N.Args * 1)(make_args(x=x, out=out, rows=0))
    assert lib.fp4ar_launch(ctx, zero, None) == 0
    lib.fp4ar_destroy(ctx)
    rec = gate_cell_emulated(CellConfig(nranks=2, rows=64), reps=3, graph_calls=0)
    assert rec["pass"], rec


def test_oversized_call_is_rejected_on_the_host():
    lib, ctx, wins = _lonely_rank0(2, 64)
    x = D.partial(128, 0).cuda()
    out = torch.zeros_like(x)
    args = (N.Args * 1)(make_args(x=x, out=out, rows=128))
    assert lib.fp4ar_launch(ctx, args, None) == 1      # rows > max_rows
    args = (N.Args * 1)(make_args(x=x, out=None, rows=64))
    assert lib.fp4ar_launch(ctx, args, None) == 1      # missing output
    a = make_args(x=x, out=out, rows=64)
    a.hidden = 4096
    assert lib.fp4ar_launch(ctx, (N.Args * 1)(a), None) == 1
    lib.fp4ar_destroy(ctx)
