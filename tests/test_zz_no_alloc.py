"""The allocation-free reduction entry point, acro_b200_reduce_batch_noalloc.

It exists for callers that are handed device pointers but cannot allocate device memory
themselves (applications that own the whole memory pool, components with a memory budget
fixed at start-up, host libraries that must not call cudaMalloc because an allocation can
synchronise the device): its scratch is a static device array inside the library.  The test calls it
through the C ABI twice in a row and compares each result with the ordinary entry point
(caller-provided scratch) on the same inputs.  This file is named so that pytest collects
it last."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import acrotensor_b200 as ab
from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-12
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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


@pytest.mark.parametrize("F,offset", [(1, 0), (9, 0), (9, 1), (32, 0), (32, 1)])
def test_noalloc_reduction_matches_the_reference_executor(F, offset):
    """Against the CPU restatement of the reference executor (an independent check: the ordinary entry point
    runs the same kernel), for the shortest and the longest row the built-in scratch takes, and with the row
    operand starting 8 bytes off a 16-byte boundary (the kernel then reads it with 8-byte loads)."""
    import torch
    rows = 50021
    rng = np.random.default_rng(100 + F + offset)
    a, w = rng.random((rows, F)) * 2 - 1, rng.random(rows) + 0.5
    ref, mags = np.zeros(F), np.zeros(F)
    oracle.contract("port", "S_f = A_n_f W_n", ref, a, w)
    oracle.contract("port", "S_f = A_n_f W_n", mags, np.abs(a), w)
    room = torch.zeros(rows * F + 2, dtype=torch.float64, device="cuda")
    da = room[offset:offset + rows * F]
    da.copy_(torch.from_numpy(a.reshape(-1)))
    assert da.data_ptr() % 16 == 8 * offset
    dw = torch.from_numpy(w).cuda()
    out = torch.full((F,), 3.0, dtype=torch.float64, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    for call in range(2):
        check(lib().acro_b200_reduce_batch_noalloc(ptr(da), ptr(dw), ptr(out), rows, F, _lib.OP_ASSIGN, None))
        torch.cuda.synchronize()
        assert oracle.parity_error(out.cpu().numpy(), ref, mags) <= TOL


def test_noalloc_survives_a_context_switch_notice():
    """acro_b200_set_context tells the library that another CUDA context may be current: the array's address, which
    belongs to one context, is looked up again.  Here the context handed over is the one already current, so the
    result must simply stay right."""
    import torch
    torch.cuda.init()
    driver = ctypes.CDLL("libcuda.so.1")
    current = ctypes.c_void_p()
    assert driver.cuCtxGetCurrent(ctypes.byref(current)) == 0 and current.value
    rows, F = 30011, 9
    a = torch.rand(rows, F, device="cuda", dtype=torch.float64)
    out = torch.zeros(F, dtype=torch.float64, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    check(lib().acro_b200_reduce_batch_noalloc(ptr(a), None, ptr(out), rows, F, _lib.OP_ASSIGN, None))
    before = out.clone()
    check(lib().acro_b200_set_context(current))
    out.zero_()
    check(lib().acro_b200_reduce_batch_noalloc(ptr(a), None, ptr(out), rows, F, _lib.OP_ASSIGN, None))
    torch.cuda.synchronize()
    assert torch.equal(out, before)
    assert ((out - a.sum(dim=0)).abs() / a.sum(dim=0)).max().item() <= TOL
    assert lib().acro_b200_device_status() == _lib.OK


def test_noalloc_in_a_second_context_of_the_same_device(tmp_path):
    """A separate program (tests/cpp/noalloc_contexts.cpp) runs the entry point in the primary context, in a context
    created through the driver API, and in the primary context again, on memory of each, against a host sum."""
    exe = str(tmp_path / "noalloc_contexts")
    libdir = os.path.dirname(ab.LIB_PATH)
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"),
                            os.path.join(ROOT, "tests", "cpp", "noalloc_contexts.cpp"), "-L" + libdir, "-lacrotensor",
                            "-Wl,-rpath," + libdir, "-ldl", "-o", exe], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    if run.stdout.startswith("SKIP"):
        pytest.skip(run.stdout.strip())
    assert run.stdout.strip().endswith("OK")
