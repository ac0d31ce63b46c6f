"""The allocation-free reduction entry point, acro_b200_reduce_batch_noalloc.

It exists for callers that are handed device pointers but cannot allocate device memory
themselves (applications that own the whole memory pool, components with a memory budget
fixed at start-up, host libraries that must not call cudaMalloc because an allocation can
synchronise the device): its scratch is a static device array inside the library.  The test calls it
through the C ABI twice in a row and compares each result with the ordinary entry point
(caller-provided scratch) on the same inputs.  This file is named so that pytest collects
it last."""
import ctypes

import numpy as np
import pytest

from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib

pytestmark = pytest.mark.gpu
TOL = 1e-12


def test_noalloc_reduction_matches_the_ordinary_entry_point_twice_in_a_row():
    import torch
    assert torch.cuda.is_available()
    rows, F = 200003, 9          # ragged tail: not a multiple of the 112-row tile
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)
    a = torch.rand(rows, F, generator=gen, device="cuda", dtype=torch.float64) * 2 - 1
    w = torch.rand(rows, generator=gen, device="cuda", dtype=torch.float64) + 0.5
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())

    nbytes = lib().acro_b200_reduce_batch_scratch_bytes(F)
    scratch = torch.empty(nbytes // 8 + 1, dtype=torch.float64, device="cuda")
    expect = torch.zeros(F, dtype=torch.float64, device="cuda")
    check(lib().acro_b200_reduce_batch(ptr(a), ptr(w), ptr(expect), rows, F, _lib.OP_ASSIGN, ptr(scratch), nbytes, None))
    scale = (a.abs() * w.view(-1, 1)).sum(dim=0)      # sum |terms| per output entry

    out = torch.full((F,), -7.0, dtype=torch.float64, device="cuda")
    for call in range(2):        # the second call finds the first call's leftovers in the shared scratch
        if call == 1:
            a.mul_(0.5)          # different data, so a stale result cannot pass
            check(lib().acro_b200_reduce_batch(ptr(a), ptr(w), ptr(expect), rows, F, _lib.OP_ASSIGN, ptr(scratch), nbytes, None))
            scale = scale * 0.5
        check(lib().acro_b200_reduce_batch_noalloc(ptr(a), ptr(w), ptr(out), rows, F, _lib.OP_ASSIGN, None))
        torch.cuda.synchronize()
        err = ((out - expect).abs() / scale).max().item()
        assert err <= TOL, (call, err)

    # accumulate form, and the size limit
    out.fill_(1.0)
    check(lib().acro_b200_reduce_batch_noalloc(ptr(a), None, ptr(out), rows, F, _lib.OP_ADD, None))
    plain = torch.zeros(F, dtype=torch.float64, device="cuda")
    check(lib().acro_b200_reduce_batch(ptr(a), None, ptr(plain), rows, F, _lib.OP_ASSIGN, ptr(scratch), nbytes, None))
    torch.cuda.synchronize()
    assert ((out - (1.0 + plain)).abs() / (1.0 + a.abs().sum(dim=0))).max().item() <= TOL
    max_f = lib().acro_b200_reduce_batch_noalloc_max_f()
    assert max_f == 32
    status = lib().acro_b200_reduce_batch_noalloc(ptr(a), None, ptr(out), 10, max_f + 1, _lib.OP_ASSIGN, None)
    assert status == _lib.EUNSUPPORTED
    assert b"built-in scratch" in lib().acro_b200_last_error()
