"""A bounded device-side wait that runs out: the exchange kernel of the sequence-parallel attention merge
is launched as rank 0 of 2 on ONE GPU, with the second rank's receive buffer being ordinary local memory
that no kernel ever writes. The flag of rank 1 therefore never arrives. With the wait limit set to two
milliseconds the kernel must return by itself, leave the output untouched and record the "peer time-out"
status; the context stays usable. Nothing faults and nothing spins without a limit: the same path with
the default limit gives up after one second."""
import ctypes as C

import numpy as np
import pytest

from fast_llm_b200 import capi

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ST_PEER_TIMEOUT = 2


def test_peer_wait_runs_out_and_is_reported():
    ctx = capi.Context(0)
    lib = ctx.lib
    n, max_records = 8, 64
    h = C.c_void_p()
    capi._ck(lib.fl_b200_seqpar_create(ctx._h, C.c_uint32(0), C.c_uint32(2), C.c_uint32(max_records), C.byref(h)))
    buf, nbytes = C.c_void_p(), C.c_size_t()
    capi._ck(lib.fl_b200_seqpar_comm(h, C.byref(buf), C.byref(nbytes)))
    absent = torch.zeros(nbytes.value, dtype=torch.uint8, device="cuda")   # stands for rank 1's buffer; nobody answers
    ptrs = (C.c_void_p * 2)(buf.value, absent.data_ptr())
    capi._ck(lib.fl_b200_seqpar_set_peers(h, ptrs, C.c_uint32(2)))
    out_local = torch.randn((n, 128), device="cuda")
    lse = torch.ones((n, 2), device="cuda")
    out = torch.full((n, 128), 7.0, device="cuda")
    torch.cuda.synchronize()
    ctx.set_wait_limit(2_000_000)          # 2 ms
    ctx.timer_start()
    capi._ck(lib.fl_b200_seqpar_combine(h, capi._p(out_local), capi._p(lse), C.c_uint32(n), capi._p(out)))
    ms = ctx.timer_stop()
    assert ms < 500.0, ms                   # returned by itself, long before the default limit
    assert ms >= 1.5, ms                    # and it did wait
    assert ctx.status() == ST_PEER_TIMEOUT
    assert ctx.status() == 0                # reading clears the word
    assert bool(torch.all(out == 7.0))      # the output was not written
    # rank 0's own records did land in the stand-in buffer (the push half ran)
    assert bool(torch.any(absent != 0))
    # the context is still usable: an ordinary kernel runs and reports nothing
    x = torch.randn(4096, device="cuda"); w = torch.ones(4096, device="cuda"); y = torch.zeros(4096, device="cuda")
    torch.cuda.synchronize()
    ctx.rmsnorm(x, w, y, 1e-5, 4096)
    ctx.sync()
    assert ctx.status() == 0
    ref = x / torch.sqrt(torch.mean(x * x) + 1e-5)
    assert float(torch.max(torch.abs(y - ref))) < 1e-5
    ctx.set_wait_limit(0)
    lib.fl_b200_seqpar_destroy(h)
    ctx.close()
