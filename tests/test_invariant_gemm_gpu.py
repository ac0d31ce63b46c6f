"""Assembly strings (one batched input whose indices are all contracted, times batch-invariant
inputs) planned as "multiply the invariant inputs out, then one tensor-core GEMM", and the GEMM
entry point itself.  Tolerance 1e-12 * sum|terms| against the CPU restatement of the reference's
interpreted executor (exec/CPUInterpretedExecutor.cpp:59-444): summation order and fused
multiply-add differ."""
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

ASSEMBLY = [
    # the reference's own assembly strings (unittest/kernel/test_TensorEngine.cpp:232-309,437-496) at scale
    ("mass2d_assembly", [("M_e_i1_i2_j1_j2=B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2", "M", ["B", "B", "B", "B", "D"])],
     {"M": (4100, 4, 4, 4, 4), "B": (4, 4), "D": (4100, 4, 4)}, False),
    ("stiff3d_assembly", [("S_e_i1_i2_i3_j1_j2_j3 = Bt1_i1_j1_k1_m_n Bt2_i2_j2_k2_m_n Bt3_i3_j3_k3_m_n D_e_k1_k2_k3_m_n",
                           "S", ["Bt1", "Bt2", "Bt3", "D"])],
     {"S": (70, 3, 3, 3, 3, 3, 3), "Bt1": (3, 3, 3, 3, 3), "Bt2": (3, 3, 3, 3, 3), "Bt3": (3, 3, 3, 3, 3), "D": (70, 3, 3, 3, 3, 3)}, False),
    # element mass matrices with more quadrature points than the rank1_gemm family takes; odd sizes, batched input first
    ("mass_q125", [("M_e_i_j = W_e_q B_q_i B_q_j", "M", ["W", "B", "B"])], {"M": (700, 9, 9), "W": (700, 125), "B": (125, 9)}, False),
    ("accumulate", [("M_e_i_j += W_e_q B_q_i C_q_j", "M", ["W", "B", "C"])], {"M": (1025, 7, 11), "W": (1025, 70), "B": (70, 7), "C": (70, 11)}, False),
    ("subtract", [("M_e_i_j -= B_q_i W_e_q C_q_j", "M", ["B", "W", "C"])], {"M": (1229, 8, 8), "B": (66, 8), "W": (1229, 66), "C": (66, 8)}, False),
]


@pytest.mark.parametrize("case", ASSEMBLY, ids=lambda c: c[0])
def test_assembly_strings_run_as_one_gemm(case):
    start = cases.make_tensors(case)
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["invariant_gemm"], plan
    out = cases.written(case)[0]
    kernel, _, ins = case[1][0]
    if "-=" in kernel:
        prod = gu.oracle_case((case[0], [(kernel.replace("-=", "="), out, ins)], case[2], False))
        ref = start[out] - prod[out]
    else:
        ref = gu.oracle_case(case)[out]
    mags = gu.oracle_case((case[0], [(kernel.replace("-=", "=").replace("+=", "="), out, ins)], case[2], False), absolute=True)[out]
    if "=" in kernel and "+=" not in kernel and "-=" not in kernel:
        scale = mags
    else:
        scale = mags + np.abs(start[out])
    assert oracle.parity_error(got[out], ref, scale) <= TOL, plan
    assert lib().acro_b200_device_status() == _lib.OK


def test_small_batches_stay_on_the_generic_kernel():
    case = ("small", [("M_e_i1_i2_j1_j2=B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2", "M", ["B", "B", "B", "B", "D"])],
            {"M": (10, 4, 4, 4, 4), "B": (4, 4), "D": (10, 4, 4)}, False)
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["generic"]
    assert np.array_equal(got["M"], gu.oracle_case(case)["M"])


@pytest.mark.parametrize("m,n,k,lda,ldp,ldc,op,offset", [
    (64, 64, 64, 64, 64, 64, 0, 0), (1, 1, 1, 1, 1, 1, 0, 0), (1000, 256, 16, 16, 256, 256, 0, 0), (333, 77, 129, 129, 77, 77, 0, 0),
    (130, 65, 63, 70, 66, 68, 1, 0), (200, 40, 200, 200, 40, 40, 2, 0), (97, 130, 5, 5, 130, 130, 0, 1), (4097, 17, 66, 66, 18, 17, 1, 1),
    (70, 729, 243, 243, 729, 729, 0, 0), (65, 3, 300, 300, 3, 3, 0, 0)])
def test_gemm_entry_point(m, n, k, lda, ldp, ldc, op, offset):
    import torch
    rng = np.random.default_rng(m + n + k)
    a, p, c0 = rng.standard_normal((m, lda)), rng.standard_normal((k, ldp)), rng.random((m, ldc))

    def dev(arr):
        flat = torch.zeros(arr.size + offset, dtype=torch.float64, device="cuda")
        flat[offset:] = torch.from_numpy(arr.reshape(-1)).cuda()
        return flat, ctypes.c_void_p(flat.data_ptr() + 8 * offset)

    (ka, pa), (kp, pp), (kc, pc) = dev(a), dev(p), dev(c0)
    check(lib().acro_b200_gemm(pa, pp, pc, m, n, k, lda, ldp, ldc, op, None))
    assert lib().acro_b200_device_status() == _lib.OK
    got = kc[offset:].cpu().numpy().reshape(m, ldc)
    prod = a[:, :k] @ p[:, :n]
    mags = np.abs(a[:, :k]) @ np.abs(p[:, :n])
    expect = [prod, c0[:, :n] + prod, c0[:, :n] - prod][op]
    assert np.max(np.abs(got[:, :n] - expect) / (mags + np.abs(c0[:, :n]))) <= 4e-15 * max(1.0, np.sqrt(k))
    assert np.array_equal(got[:, n:], c0[:, n:])                    # the gap between rows is not touched
    assert lib().acro_b200_gemm(pa, pp, pc, m, n, k, k - 1, ldp, ldc, op, None) == _lib.EINVAL
