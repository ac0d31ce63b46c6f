"""GPU parity of batched products with an operand stored transposed ("C_e_i_j = A_e_k_i B_e_k_j",
"C_e_i_j = A_e_i_k B_e_j_k", both), through the kernel layer of the C ABI and through the engine.
Up to 16 x 16 x 16 the streaming kernel keeps the reference's operation order: bit-identical.
Above that the fp64 tensor-core kernels reorder the sum: |gpu - ref| <= 1e-12 * sum|terms|."""
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


def kernel_string(ta, tb, op="="):
    return "C_e_i_j %s %s %s" % (op, "A_e_k_i" if ta else "A_e_i_k", "B_e_j_k" if tb else "B_e_k_j")


def operands(rng, batch, m, n, k, ta, tb):
    a = rng.standard_normal((batch, k, m) if ta else (batch, m, k))
    b = rng.standard_normal((batch, n, k) if tb else (batch, k, n))
    return a, b


CASES = [
    # streaming kernel (bit-identical)
    (1000, 3, 3, 3, 1, 0, 0, 0), (1000, 3, 3, 3, 0, 1, 0, 0), (4097, 4, 4, 4, 1, 1, 1, 0), (513, 8, 8, 8, 0, 1, 2, 0),
    (2050, 16, 16, 16, 1, 0, 0, 0), (777, 16, 16, 16, 1, 1, 1, 1), (300, 5, 7, 3, 1, 1, 0, 0), (64, 2, 16, 9, 0, 1, 2, 1), (33, 16, 15, 16, 1, 0, 0, 1),
    # zero-padded into 32-wide slots
    (500, 27, 27, 27, 1, 0, 0, 0), (301, 27, 27, 27, 0, 1, 1, 1), (1000, 27, 27, 27, 1, 1, 2, 0), (222, 25, 31, 19, 1, 0, 0, 0), (223, 21, 17, 29, 0, 1, 1, 0),
    (90, 27, 23, 32, 1, 1, 0, 0), (64, 20, 24, 30, 1, 1, 0, 0), (55, 18, 24, 31, 1, 0, 2, 0), (90, 17, 32, 5, 0, 1, 0, 0),
    # the full 32-wide and 64-wide slots
    (200, 32, 32, 32, 1, 0, 0, 0), (201, 32, 32, 32, 1, 1, 1, 0), (150, 64, 64, 64, 0, 1, 0, 0), (149, 64, 64, 64, 1, 0, 2, 0), (33, 64, 64, 64, 1, 1, 0, 1),
    # zero-padded into 64-wide slots
    (40, 64, 64, 48, 1, 0, 0, 0), (64, 20, 33, 17, 1, 1, 0, 0), (130, 48, 48, 48, 0, 1, 1, 0), (20, 63, 63, 63, 1, 1, 0, 1), (75, 40, 24, 30, 1, 0, 0, 0),
    # one row or one column: the matrix-vector kernel with the two forms swapped
    (501, 27, 1, 27, 1, 0, 0, 1), (333, 1, 40, 33, 0, 1, 1, 0), (1000, 64, 1, 64, 1, 1, 2, 0),
]


@pytest.mark.parametrize("batch,m,n,k,ta,tb,op,offset", CASES)
def test_transposed_batched_gemm_kernel(torch, batch, m, n, k, ta, tb, op, offset):
    rng = np.random.default_rng(batch + 3 * m + 5 * k + ta + 2 * tb)
    a, b = operands(rng, batch, m, n, k, ta, tb)
    c0 = rng.random((batch, m, n))
    ka, pa = to_dev(torch, a, offset)
    kb, pb = to_dev(torch, b)
    kc, pc = to_dev(torch, c0, offset)
    assert lib().acro_b200_batched_gemm_t_supported(m, n, k, ta, tb) == 1
    check(lib().acro_b200_batched_gemm_t(pa, pb, pc, batch, m, n, k, ta, tb, op, None))
    assert lib().acro_b200_device_status() == _lib.OK
    got = kc[offset:].cpu().numpy().reshape(c0.shape)
    prod, mags = np.zeros_like(c0), np.zeros_like(c0)
    oracle.contract("port", kernel_string(ta, tb), prod, a, b)
    oracle.contract("port", kernel_string(ta, tb), mags, np.abs(a), np.abs(b))
    if max(m, n, k) <= 16 and m > 1 and n > 1:
        if op == 1:
            expect = c0.copy()
            oracle.contract("port", kernel_string(ta, tb, "+="), expect, a, b)
        else:
            expect = [prod, None, c0 - prod][op]
        assert np.array_equal(got, expect)
    else:
        expect = [prod, c0 + prod, c0 - prod][op]
        assert oracle.parity_error(got, expect, mags + np.abs(c0)) <= TOL


def test_transposed_limits():
    assert lib().acro_b200_batched_gemm_t_supported(65, 8, 8, 1, 0) == 0
    assert lib().acro_b200_batched_gemm_t_supported(8, 8, 65, 0, 1) == 0
    assert lib().acro_b200_batched_gemm_t_supported(65, 8, 8, 0, 0) == 1
    assert lib().acro_b200_batched_gemm_t_supported(64, 64, 64, 1, 1) == 1


ENGINE = [
    # the same tensor twice, transposed on the left
    (("metric_t", [("G_e_m_n = J_e_l_m J_e_l_n", "G", ["J", "J"])], {"G": (5000, 3, 3), "J": (5000, 3, 3)}, False), True),
    # both roles swapped: the first input is the right factor
    (("swapped", [("C_e_i_j = A_e_j_k B_e_k_i", "C", ["A", "B"])], {"C": (700, 9, 6), "A": (700, 6, 7), "B": (700, 7, 9)}, False), True),
    (("accumulate", [("C_e_i_j += A_e_k_i B_e_j_k", "C", ["A", "B"])], {"C": (90, 20, 24), "A": (90, 30, 20), "B": (90, 24, 30)}, False), False),
    (("matvec_t", [("Y_e_i = M_e_k_i X_e_k", "Y", ["M", "X"])], {"Y": (3000, 27), "M": (3000, 30, 27), "X": (3000, 30)}, False), False),
    (("cube64", [("C_e_i_j = A_e_i_k B_e_j_k", "C", ["A", "B"])], {"C": (300, 64, 64), "A": (300, 64, 64), "B": (300, 64, 64)}, False), False),
]


@pytest.mark.parametrize("case,exact", ENGINE, ids=lambda c: c[0] if isinstance(c, tuple) else None)
def test_transposed_products_through_the_engine(case, exact):
    start = cases.make_tensors(case)
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["batched_gemm"], plan
    out = cases.written(case)[0]
    kernel, _, ins = case[1][0]
    ref = gu.oracle_case(case)[out]
    if exact:
        assert np.array_equal(got[out], ref)
    else:
        mags = gu.oracle_case((case[0], [(kernel.replace("+=", "="), out, ins)], case[2], False), absolute=True)[out]
        assert oracle.parity_error(got[out], ref, mags + np.abs(start[out])) <= TOL, plan
    assert lib().acro_b200_device_status() == _lib.OK
