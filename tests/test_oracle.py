"""The CPU checkers themselves: the C restatement against the committed golden vectors
(outputs of the unmodified reference) and, where the reference-backed library is present,
against that library directly.  No GPU involved."""
import os

import numpy as np
import pytest

import cases
from oracle import oracle

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


def run_case(kind, case):
    tensors = cases.make_tensors(case)
    names = sorted(tensors)
    oracle.run(kind, [tensors[n] for n in names], cases.as_oracle_program(case, names), multi=case[3])
    return tensors


@pytest.mark.parametrize("case", cases.all_cases(), ids=lambda c: c[0])
def test_restatement_matches_golden_bit_for_bit(case):
    fresh = cases.make_tensors(case)
    assert cases.digest(fresh) == str(GOLDEN[case[0] + "/inputs_sha256"]), "seeded inputs drifted from the fixtures"
    got = run_case("port", case)
    for n in cases.written(case):
        assert np.array_equal(got[n], GOLDEN["%s/out/%s" % (case[0], n)]), n


@pytest.mark.skipif(not oracle.have("ref"), reason="reference-backed checker not built")
@pytest.mark.parametrize("case", cases.all_cases(), ids=lambda c: c[0])
def test_reference_library_matches_golden(case):
    got = run_case("ref", case)
    for n in cases.written(case):
        assert np.array_equal(got[n], GOLDEN["%s/out/%s" % (case[0], n)]), n


def test_minus_equals_accumulates_like_the_reference_cpu_executor():
    # exec/CPUInterpretedExecutor.cpp:64-67,106: "-=" is executed as "+=".
    rng = np.random.default_rng(3)
    b, c = rng.random((3, 5)), rng.random((4, 5))
    a0 = rng.random((3, 4))
    plus, minus = a0.copy(), a0.copy()
    oracle.contract("port", "A_m_n+=B_m_j C_n_j", plus, b, c)
    oracle.contract("port", "A_m_n-=B_m_j C_n_j", minus, b, c)
    assert np.array_equal(plus, minus)


@pytest.mark.parametrize("text,ok", [
    ("Blah", False), ("Blah=", False), ("Blah=Alah", False), ("BLA1h=Alah", False), ("B_lah=A_lah", True),
    ("B_lah=A_lah_", False), ("B_lah_=A_lah", False), ("a_lah_=A_lah", False), ("BA_i=A_j", True),
    ("B1_i=CB_jBr_j", True), ("A_i += B_i", True), ("A_i -= B_i", True), ("A_i =+ B_i", False),
])
def test_restatement_grammar(text, ok):
    # accept / reject set of unittest/kernel/test_TensorKernel.cpp:15-25
    assert oracle.parses(text) == ok


def test_summation_order_is_sequential_from_zero():
    # 1 + 2^-53 + 2^-53 summed left to right stays 1.0; a pairwise sum would give 1 + 2^-52.
    a = np.array([1.0, 2.0 ** -53, 2.0 ** -53]).reshape(3, 1)
    s = np.zeros(1)
    oracle.contract("port", "S_i = A_n_i", s, a)
    assert s[0] == 1.0


def test_threaded_reference_driver_matches_single_thread():
    if not oracle.have("ref"):
        pytest.skip("reference-backed checker not built")
    rng = np.random.default_rng(5)
    n = 4096
    a, b = rng.random((n, 3, 3)), np.ones(n)
    s1, s4 = np.zeros((3, 3)), np.zeros((3, 3))
    prog = [("S_i_j = A_n_i_j B_n", 0, [1, 2])]
    oracle.run("ref", [s1, a, b], prog)
    oracle.run_ref_slabs([s4, a, b], prog, [0, 1, 1], n, 4)
    assert np.max(np.abs(s1 - s4) / s1) < 1e-13
    w, bb = rng.random((8, 64)), rng.random((64, 27)) - 0.5
    m1, m4 = np.zeros((8, 27, 27)), np.zeros((8, 27, 27))
    prog = [("M_e_i_j = W_e_q B_q_i B_q_j", 0, [1, 2, 2])]
    oracle.run("ref", [m1, w, bb], prog)
    oracle.run_ref_slabs([m4, w, bb], prog, [1, 1, 0], 8, 3)
    assert np.array_equal(m1, m4)


def test_fuzzed_strings_restatement_equals_reference_library():
    """Random strings (diagonals, broadcasts, +=, -=): the restatement and the reference's own
    code agree bit for bit, and the product's parser accepts every one of them."""
    import acrotensor_b200 as ab
    import fuzz
    if not oracle.have("ref"):
        pytest.skip("reference-backed checker not built")
    rng = np.random.default_rng(99)
    for text, shapes, in_names, op in fuzz.cases(2024, 150):
        tensors = {n: rng.random(s) * 2 - 1 for n, s in shapes.items()}
        a_port, a_ref = tensors["A"].copy(), tensors["A"].copy()
        oracle.contract("port", text, a_port, *[tensors[n] for n in in_names])
        oracle.contract("ref", text, a_ref, *[tensors[n] for n in in_names])
        assert np.array_equal(a_port, a_ref), text
        ab.describe_kernel(text)
