"""GPU parity of the register-blocked variant of the generic kernel (a thread owns several
output entries along one outer loop and shares the loads that do not carry it).  Sizes are
chosen so that the launcher really picks that variant; results must be bit-identical to the
CPU restatement of the reference's interpreted executor (exec/CPUInterpretedExecutor.cpp:59-444),
because the operation order per entry is unchanged."""
import numpy as np
import pytest

import cases
import gpu_util as gu

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def only_the_generic_family(monkeypatch):
    # some of these strings would otherwise be planned on a specialised family (they are assembly strings)
    monkeypatch.setenv("ACRO_B200_ONLY_GENERIC", "1")

BLOCKED_CASES = [
    # the reference's 2D mass assembly string (unittest/kernel/test_TensorEngine.cpp:232-300) at scale:
    # two leading inputs are hoisted out of the k2 loop, four entries per thread
    ("mass2d_m_blocked", [("M_e_i1_i2_j1_j2=B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2", "M", ["B", "B", "B", "B", "D"])],
     {"M": (8192, 4, 4, 4, 4), "B": (4, 4), "D": (8192, 4, 4)}, False),
    # the reference's 3D stiffness string: five contracted indices (odometer over four of them), five entries per thread
    ("stiff3d_blocked", [("S_e_i1_i2_i3_j1_j2_j3 = Bt1_i1_j1_k1_m_n Bt2_i2_j2_k2_m_n Bt3_i3_j3_k3_m_n D_e_k1_k2_k3_m_n",
                          "S", ["Bt1", "Bt2", "Bt3", "D"])],
     {"S": (32, 5, 5, 5, 5, 5, 5), "Bt1": (5, 5, 5, 3, 3), "Bt2": (5, 5, 5, 3, 3), "Bt3": (5, 5, 5, 3, 3),
      "D": (32, 5, 5, 5, 3, 3)}, False),
    ("matmul_blocked", [("C_i_j = A_i_k B_k_j", "C", ["A", "B"])], {"C": (768, 512), "A": (768, 96), "B": (96, 512)}, False),
    # here the second input carries the blocked index (the first one above)
    ("matmul_first_input_blocked", [("C_i_j = A_k_j B_i_k", "C", ["A", "B"])],
     {"C": (768, 512), "A": (96, 512), "B": (768, 96)}, False),
    ("accumulate_blocked", [("A_m_n+=B_m_j C_n_j", "A", ["B", "C"])], {"A": (1024, 512), "B": (1024, 40), "C": (512, 40)}, False),
    ("subtract_blocked", [("A_m_n-=B_m_j C_n_j", "A", ["B", "C"])], {"A": (1024, 512), "B": (1024, 40), "C": (512, 40)}, False),
    # three entries per thread (3^11 rows), and two (2 * 100003 rows)
    ("three_per_thread", [("A_e_i = B_e_i_k C_k", "A", ["B", "C"])], {"A": (177147, 2), "B": (177147, 2, 7), "C": (7,)}, False),
    ("two_per_thread", [("A_e = B_e_k C_k D_k", "A", ["B", "C", "D"])], {"A": (200006,), "B": (200006, 5), "C": (5,), "D": (5,)}, False),
    # entry-wise products without any contraction (what builds the invariant factor of an assembly string)
    ("outer_product", [("P_a_b_c = X_a_c Y_b_c Z_c", "P", ["X", "Y", "Z"])], {"P": (300, 400, 6), "X": (300, 6), "Y": (400, 6), "Z": (6,)}, False),
    # a leading input without any contracted index, and a diagonal read
    ("hoisted_scale", [("A_i_j = S_i B_j_k C_k_k", "A", ["S", "B", "C"])], {"A": (640, 640), "S": (640,), "B": (640, 9), "C": (9, 9)}, False),
]


@pytest.mark.parametrize("case", BLOCKED_CASES, ids=lambda c: c[0])
def test_blocked_generic_kernel_is_bit_identical(case):
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["generic"], plan
    assert "output entries along" in plan, plan
    if case[0] == "three_per_thread":
        assert "thread per 3 output entries" in plan, plan
    if case[0] == "two_per_thread":
        assert "thread per 2 output entries" in plan, plan
    if case[0] == "subtract_blocked":
        # The reference's generated CUDA kernel subtracts for "-=" (exec/CudaExecutor.cpp:536) while its CPU executor
        # adds: compare with old value minus the "=" product, rounded once, which is what the kernel computes.
        start = cases.make_tensors(case)
        prod = gu.oracle_case((case[0], [(case[1][0][0].replace("-=", "="), "A", ["B", "C"])], case[2], False))
        assert np.array_equal(got["A"], start["A"] - prod["A"]), plan
        return
    ref = gu.oracle_case(case)
    for n in cases.written(case):
        assert np.array_equal(got[n], ref[n]), (n, plan)


def test_blocked_and_plain_variants_agree_bitwise():
    """The same string at a size below the blocking threshold (thread per entry) and above it."""
    small = ("s", [("A_m_n=B_m_j C_n_j", "A", ["B", "C"])], {"A": (64, 32), "B": (64, 40), "C": (32, 40)}, False)
    large = ("l", [("A_m_n=B_m_j C_n_j", "A", ["B", "C"])], {"A": (1024, 512), "B": (1024, 40), "C": (512, 40)}, False)
    tl = cases.make_tensors(large)
    got_l, plan_l = gu.run_case_on_gpu(large, tensors=tl)
    ts = {"A": np.zeros((64, 32)), "B": np.ascontiguousarray(tl["B"][:64]), "C": np.ascontiguousarray(tl["C"][:32])}
    got_s, plan_s = gu.run_case_on_gpu(small, tensors=ts)
    assert "thread per output entry" in plan_s and "output entries along" in plan_l
    assert np.array_equal(got_s["A"], got_l["A"][:64, :32])


@pytest.mark.parametrize("kernel,shape,offset", [("A_i = B_i", (100001,), 0), ("A_i_j += B_i_j", (333, 301), 0), ("A_i_j_k -= B_i_j_k", (50, 7, 11), 0),
                                                 ("A_i = B_i", (4099,), 1), ("A_i_j += B_i_j", (64, 65), 1)])
def test_same_layout_streams(kernel, shape, offset):
    """One input, nothing contracted, the same layout on both sides: the flat streaming path (pairs of entries
    when both device pointers are 16-byte aligned, single entries otherwise)."""
    import torch
    import acrotensor_b200 as ab
    rng = np.random.default_rng(int(np.prod(shape)))
    a0, b = rng.random(shape), rng.random(shape)
    host_a = a0.copy()
    n = a0.size
    bufs = [torch.zeros(n + offset, dtype=torch.float64, device="cuda") for _ in range(2)]
    bufs[0][offset:] = torch.from_numpy(a0.reshape(-1)).cuda()
    bufs[1][offset:] = torch.from_numpy(b.reshape(-1)).cuda()
    A = ab.Tensor(shape, hdata=host_a, ddata=bufs[0].data_ptr() + 8 * offset, ongpu=True)
    B = ab.Tensor(shape, hdata=b, ddata=bufs[1].data_ptr() + 8 * offset, ongpu=True)
    ab.TensorEngine("Cuda")(kernel, A, B)
    A.MoveFromGPU()
    expect = b if "+=" not in kernel and "-=" not in kernel else (a0 + b if "+=" in kernel else a0 - b)
    assert np.array_equal(host_a, expect)
