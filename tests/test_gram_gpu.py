"""GPU parity of the Gram form S_a_b (op)= X_n_a Y_n_b (two row operands contracted over their common
leading index), through the kernel layer of the C ABI and through the engine.  Rows are summed per
thread and per CTA (up to 16 x 16: streaming kernel with fused multiply-add; above: slabs of rows on
the fp64 tensor cores), so the order differs from the reference's sequential sum:
|gpu - ref| <= 1e-12 * sum|terms|; two runs give the same bits."""
import ctypes

import numpy as np
import pytest

import cases
import gpu_util as gu
from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-12


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def to_dev(torch, arr, offset=0):
    flat = torch.zeros(arr.size + offset, dtype=torch.float64, device="cuda")
    flat[offset:] = torch.from_numpy(np.ascontiguousarray(arr).reshape(-1)).cuda()
    return flat, ctypes.c_void_p(flat.data_ptr() + 8 * offset)


@pytest.mark.parametrize("rows,a,b,op,offset", [
    (64 * 500, 64, 64, 0, 0), (64 * 500 + 37, 64, 64, 1, 0), (70001, 40, 64, 2, 0), (9999, 33, 7, 0, 1), (50, 64, 64, 0, 0),
    (32 * 3000, 8, 8, 0, 0), (100003, 8, 8, 1, 0), (100000, 5, 9, 2, 0), (77777, 27, 27, 0, 1), (31, 8, 8, 0, 0), (32, 16, 3, 0, 0),
    (77777, 16, 16, 0, 1), (50001, 6, 10, 0, 0), (70000, 13, 4, 1, 0), (2049, 16, 16, 2, 0), (600000, 2, 1, 0, 0),
    (200001, 1, 1, 0, 0), (150000, 32, 1, 1, 0), (150000, 2, 32, 0, 1), (1, 3, 3, 0, 0), (400000, 3, 3, 0, 0),
    # odd row lengths on aligned operands: pairs of 32-row slabs by bulk copy, the rest through the ring
    (77777, 27, 27, 0, 0), (64 * 700, 27, 27, 1, 0), (64 * 300 + 33, 25, 31, 2, 0), (130, 17, 19, 0, 0), (64, 27, 27, 0, 0), (63, 27, 27, 0, 0),
    # full 64 x 64 slabs on the accumulating two-group kernel
    (64 * 1000, 64, 64, 0, 0), (64 * 3 + 5, 64, 64, 1, 0), (64 * 149, 64, 64, 2, 0)])
def test_gram_kernel(torch, rows, a, b, op, offset):
    rng = np.random.default_rng(rows + a + 3 * b)
    x, y = rng.standard_normal((rows, a)), rng.standard_normal((rows, b))
    s0 = rng.random((a, b))
    kx, px = to_dev(torch, x, offset)
    ky, py = to_dev(torch, y)
    ks, ps = to_dev(torch, s0, offset)
    assert lib().acro_b200_gram_supported(a, b) == 1
    nbytes = lib().acro_b200_gram_scratch_bytes(a, b)
    assert nbytes >= a * b * 8
    scratch = torch.full((nbytes // 8,), float("nan"), dtype=torch.float64, device="cuda")
    pscratch = ctypes.c_void_p(scratch.data_ptr())
    check(lib().acro_b200_gram(px, py, ps, rows, a, b, op, pscratch, nbytes, None))
    assert lib().acro_b200_device_status() == _lib.OK
    got = ks[offset:].cpu().numpy().reshape(a, b)
    prod, mags = np.zeros((a, b)), np.zeros((a, b))
    oracle.contract("port", "S_a_b = X_n_a Y_n_b", prod, x, y)
    oracle.contract("port", "S_a_b = X_n_a Y_n_b", mags, np.abs(x), np.abs(y))
    expect = [prod, s0 + prod, s0 - prod][op]
    assert oracle.parity_error(got, expect, mags + np.abs(s0)) <= TOL

    # the same call again: identical bits (fixed summation order, no floating-point atomics)
    ks2, ps2 = to_dev(torch, s0, offset)
    check(lib().acro_b200_gram(px, py, ps2, rows, a, b, op, pscratch, nbytes, None))
    assert np.array_equal(ks2[offset:].cpu().numpy().reshape(a, b), got)


def test_gram_limits(torch):
    assert lib().acro_b200_gram_supported(65, 3) == 0 and lib().acro_b200_gram_supported(3, 0) == 0
    assert lib().acro_b200_gram_scratch_bytes(65, 3) == 0
    x = torch.zeros(64, dtype=torch.float64, device="cuda")
    p = ctypes.c_void_p(x.data_ptr())
    assert lib().acro_b200_gram(p, p, p, 8, 2, 2, 0, p, 8, None) == _lib.EINVAL          # scratch too small
    assert lib().acro_b200_gram(p, p, p, 8, 65, 2, 0, p, 1 << 20, None) == _lib.EUNSUPPORTED


ENGINE = [
    ("gram64", [("S_a_b = X_n_a Y_n_b", "S", ["X", "Y"])], {"S": (64, 64), "X": (30011, 64), "Y": (30011, 64)}, False),
    ("normal_equations", [("S_a_b = X_n_a X_n_b", "S", ["X", "X"])], {"S": (27, 27), "X": (50000, 27)}, False),
    ("swapped_accumulate", [("S_a_b += Y_n_b X_n_a", "S", ["Y", "X"])], {"S": (5, 9), "Y": (120000, 9), "X": (120000, 5)}, False),
    ("subtract", [("S_a_b -= X_n_a Y_n_b", "S", ["X", "Y"])], {"S": (8, 8), "X": (65536, 8), "Y": (65536, 8)}, False),
]


@pytest.mark.parametrize("case", ENGINE, ids=lambda c: c[0])
def test_gram_strings_through_the_engine(case):
    start = cases.make_tensors(case)
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["gram"], plan
    kernel, out, ins = case[1][0]
    plain = kernel.replace("-=", "=").replace("+=", "=")
    prod = gu.oracle_case((case[0], [(plain, out, ins)], case[2], False))[out]
    mags = gu.oracle_case((case[0], [(plain, out, ins)], case[2], False), absolute=True)[out]
    ref = start[out] - prod if "-=" in kernel else (start[out] + prod if "+=" in kernel else prod)
    assert oracle.parity_error(got[out], ref, mags + np.abs(start[out])) <= TOL, plan
    assert lib().acro_b200_device_status() == _lib.OK


def test_short_contractions_stay_on_the_generic_kernel():
    case = ("short", [("S_a_b = X_n_a Y_n_b", "S", ["X", "Y"])], {"S": (8, 8), "X": (1000, 8), "Y": (1000, 8)}, False)
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["generic"]
