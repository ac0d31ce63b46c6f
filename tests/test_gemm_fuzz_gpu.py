"""Seeded random shapes through the engine for the families that tile matrices: batched products of any
m, n, k up to 64 (bit-identical up to 16, tolerance above) and assembly strings planned as one GEMM
(odd and even leading dimensions, ragged tiles, every operator).  The checker is the CPU restatement of
the reference's interpreted executor (exec/CPUInterpretedExecutor.cpp:59-444)."""
import numpy as np
import pytest

import acrotensor_b200 as ab
import gpu_util as gu
from acrotensor_b200 import _lib
from acrotensor_b200._lib import lib
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-12


def run(kernel, out0, *ins):
    got = out0.copy()
    te = ab.TensorEngine("Cuda")
    handles = {}
    operands = []
    for x in ins:
        if id(x) not in handles:
            handles[id(x)] = ab.Tensor(x.shape, hdata=x)
        operands.append(handles[id(x)])
    out = ab.Tensor(got.shape, hdata=got)
    plan = te.GetImplementation(kernel, out, *operands)
    te(kernel, out, *operands)
    out.MoveFromGPU()
    return got, gu.families(plan)[0]


def reference(kernel, out0, *ins):
    op = "-=" if "-=" in kernel else ("+=" if "+=" in kernel else "=")
    plain = kernel.replace("-=", "=").replace("+=", "=")
    prod, mags = np.zeros_like(out0), np.zeros_like(out0)
    oracle.contract("port", plain, prod, *ins)
    oracle.contract("port", plain, mags, *[np.abs(x) for x in ins])
    if op == "=":
        return prod, mags, prod
    exact = out0.copy()
    if op == "+=":
        oracle.contract("port", kernel, exact, *ins)           # term by term onto the old value
        return out0 + prod, mags + np.abs(out0), exact
    return out0 - prod, mags + np.abs(out0), out0 - prod


@pytest.mark.parametrize("seed", range(12))
def test_random_batched_products(seed):
    rng = np.random.default_rng(1000 + seed)
    m, n, k = (int(x) for x in rng.integers(1, 65, size=3))
    if seed % 3 == 0:
        m, n, k = (int(x) for x in rng.integers(1, 17, size=3))
    batch = int(rng.integers(1, 400))
    op = ["=", "+=", "-="][seed % 3]
    a, b, c0 = rng.standard_normal((batch, m, k)), rng.standard_normal((batch, k, n)), rng.random((batch, m, n))
    kernel = "C_e_i_j %s A_e_i_k B_e_k_j" % op
    got, family = run(kernel, c0, a, b)
    assert family == "batched_gemm"
    ref, mags, exact = reference(kernel, c0, a, b)
    if max(m, n, k) <= 16 and m > 1 and n > 1:
        assert np.array_equal(got, exact), (m, n, k, batch, op)
    else:
        assert oracle.parity_error(got, ref, mags) <= TOL, (m, n, k, batch, op)
    assert lib().acro_b200_device_status() == _lib.OK


@pytest.mark.parametrize("seed", range(10))
def test_random_assembly_strings(seed):
    rng = np.random.default_rng(2000 + seed)
    # Out_e_x1[_x2] = (one or two invariant factors) In_e_q1[_q2], factors in a random order
    q = [int(v) for v in rng.integers(2, 12, size=int(rng.integers(1, 3)))]
    x = [int(v) for v in rng.integers(3, 14, size=int(rng.integers(1, 3)))]
    while int(np.prod(x)) < 16:
        x[0] += 3
    while int(np.prod(q)) < 4:
        q[0] += 2
    # the planner takes this family from 64 elements and 2^22 terms on
    elements = int(rng.integers(64, 200)) + (1 << 22) // (int(np.prod(q)) * int(np.prod(x)))
    qn = ["q%d" % i for i in range(len(q))]
    xn = ["x%d" % i for i in range(len(x))]
    factors = []
    # factor 1 links the first q with the first x; factor 2 (if any q or x is left over) links the rest
    factors.append(("F", [qn[0], xn[0]], (q[0], x[0])))
    rest_q, rest_x = qn[1:], xn[1:]
    if rest_q or rest_x:
        idx = rest_x + rest_q
        shape = tuple([x[xn.index(i)] for i in rest_x] + [q[qn.index(i)] for i in rest_q])
        factors.append(("G", idx, shape))
    batched = ("D", ["e"] + qn, tuple([elements] + q))
    order = [batched] + factors
    order = [order[i] for i in rng.permutation(len(order))]
    op = ["=", "+=", "-="][seed % 3]
    kernel = "S_e_%s %s %s" % ("_".join(xn), op, " ".join("%s_%s" % (name, "_".join(idx)) for name, idx, _ in order))
    tensors = [rng.random(shape) * 2 - 1 for _, _, shape in order]
    out0 = rng.random(tuple([elements] + x))
    got, family = run(kernel, out0, *tensors)
    assert family == "invariant_gemm", kernel
    ref, mags, _ = reference(kernel, out0, *tensors)
    assert oracle.parity_error(got, ref, mags) <= TOL, kernel
    assert lib().acro_b200_device_status() == _lib.OK


@pytest.mark.parametrize("kernel,shapes", [
    ("Y_e_i = M_e_i_j X_e_j", [(3000, 27), (3000, 27, 27), (3000, 27)]),          # element matrices applied to element vectors
    ("Y_e_i += X_e_j M_e_i_j", [(1000, 8), (1000, 8), (1000, 8, 8)]),
    ("Y_e_j -= X_e_k M_e_k_j", [(777, 9), (777, 5), (777, 5, 9)]),                 # row vector times matrix
    ("Y_e_i = M_e_i_j X_e_j", [(500, 64), (500, 64, 64), (500, 64)]),
    ("Y_e_i = M_e_i_j X_e_j", [(1001, 3), (1001, 3, 3), (1001, 3)]),
    ("Y_e_j = X_e_k M_e_k_j", [(333, 64), (333, 33), (333, 33, 64)]),
    ("Y_e_i += M_e_i_j X_e_j", [(65, 17), (65, 17, 40), (65, 40)]),
])
def test_element_matrix_vector_products(kernel, shapes):
    rng = np.random.default_rng(len(kernel) + shapes[0][0])
    out0 = rng.random(shapes[0])
    ins = [rng.standard_normal(s) for s in shapes[1:]]
    got, family = run(kernel, out0, *ins)
    assert family == "batched_gemm"
    ref, mags, exact = reference(kernel, out0, *ins)
    assert oracle.parity_error(got, ref, mags) <= TOL, kernel       # rotated summation order, fused multiply-add
    assert lib().acro_b200_device_status() == _lib.OK
