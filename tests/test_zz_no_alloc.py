"""fp4ar_reduce_reencode_noalloc, called through its exported C symbol.

Some users of this library cannot allocate device memory at the point where they call it (a plugin inside
another framework's memory plan, code running under a frozen allocator).  For them the library keeps the
owner step's record buffer in a fixed device array.  This test loads the shared library directly, calls the
symbol twice in a row and requires the BF16 output to equal, bit for bit, what the regular entry point
(`fp4ar_reduce_reencode`, caller-provided record buffer) produces; it also checks that a call beyond the
built-in capacity is refused with a message.  The file is named so that pytest collects it last."""
import ctypes as C

import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200.ops import codec
from fp4_all_reduce_b200.utils import data as D

pytestmark = pytest.mark.gpu
MAX_ROWS = 1024   # FP4AR_NOALLOC_MAX_ROWS in csrc/include/fp4ar_noalloc.h


def _symbol():
    lib = C.CDLL(str(N.cuda_library_path()))
    fn = lib.fp4ar_reduce_reencode_noalloc
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.c_long, C.POINTER(C.c_void_p), C.POINTER(C.c_float), C.c_int,
                   C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    lib.fp4ar_noalloc_last_error.restype = C.c_char_p
    return lib, fn


def _call(fn, qs, rss, rows, out):
    n = len(qs)
    src = (C.c_void_p * n)(*[q.data_ptr() for q in qs])
    rsp = (C.c_void_p * n)(*[r.data_ptr() for r in rss])
    gs = (C.c_float * N.MAX_RANKS)()
    return fn(n, src, N.QROW_BYTES, rsp, gs, rows, out.data_ptr(), C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_two_calls_in_a_row_match_the_regular_entry_point():
    torch.cuda.set_device(0)
    lib, fn = _symbol()
    for rows, seed in ((MAX_ROWS, 0), (301, 1)):          # the second call reuses the array the first one filled
        xs = [D.gaussian_mags(rows, s, seed).cuda() for s in range(4)]
        enc = [codec.encode(x) for x in xs]
        qs, rss = [e[0] for e in enc], [e[1] for e in enc]
        _, want = codec.reduce_reencode(qs, rss)
        out = torch.zeros(rows, N.HIDDEN, dtype=torch.bfloat16, device="cuda:0")
        rc = _call(fn, qs, rss, rows, out)
        assert rc == 0, lib.fp4ar_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), want.view(torch.int16))


def test_a_call_beyond_the_capacity_is_refused():
    torch.cuda.set_device(0)
    lib, fn = _symbol()
    rows = MAX_ROWS + 1
    q = torch.zeros(rows, N.QROW_BYTES, dtype=torch.uint8, device="cuda:0")
    rs = torch.ones(rows, dtype=torch.float32, device="cuda:0")
    out = torch.full((rows, N.HIDDEN), 3.0, dtype=torch.bfloat16, device="cuda:0")
    rc = _call(fn, [q], [rs], rows, out)
    assert rc == 1
    msg = lib.fp4ar_noalloc_last_error().decode()
    assert "exceed" in msg and str(MAX_ROWS) in msg
    torch.cuda.synchronize()
    assert bool((out == 3.0).all())     # nothing was launched
