"""permute: index reorderings whose fastest index changes run as a tiled transpose; pure data movement,
so the result is bit-identical to the reference's interpreted executor (exec/CPUInterpretedExecutor.cpp:59-444)."""
import numpy as np
import pytest

import cases
import gpu_util as gu
from acrotensor_b200 import _lib
from acrotensor_b200._lib import lib

pytestmark = pytest.mark.gpu

PERMUTATIONS = [
    ("transpose", [("A_i_j=B_j_i", "A", ["B"])], {"A": (1000, 777), "B": (777, 1000)}, False),
    ("ragged_tiles", [("A_i_j=B_j_i", "A", ["B"])], {"A": (257, 263), "B": (263, 257)}, False),
    ("batched_transpose", [("A_e_i_j = B_e_j_i", "A", ["B"])], {"A": (3001, 27, 27), "B": (3001, 27, 27)}, False),
    ("rotate_three", [("A_i_j_k = B_k_i_j", "A", ["B"])], {"A": (40, 50, 64), "B": (64, 40, 50)}, False),
    ("reference_test_layout", [("Z_m_e_k = D_e_k_m", "Z", ["D"])], {"Z": (16, 700, 20), "D": (700, 20, 16)}, False),
    ("accumulate", [("A_i_j += B_j_i", "A", ["B"])], {"A": (300, 400), "B": (400, 300)}, False),
    ("subtract", [("A_i_j -= B_j_i", "A", ["B"])], {"A": (300, 400), "B": (400, 300)}, False),
]


@pytest.mark.parametrize("case", PERMUTATIONS, ids=lambda c: c[0])
def test_permutation_is_exact(case):
    start = cases.make_tensors(case)
    got, plan = gu.run_case_on_gpu(case)
    assert gu.families(plan) == ["permute"], plan
    kernel, out, ins = case[1][0]
    if "-=" in kernel:
        moved = gu.oracle_case((case[0], [(kernel.replace("-=", "="), out, ins)], case[2], False))[out]
        ref = start[out] - moved
    else:
        ref = gu.oracle_case(case)[out]
    assert np.array_equal(got[out], ref)
    assert lib().acro_b200_device_status() == _lib.OK


def test_same_fastest_index_or_short_runs_stay_on_the_generic_kernel():
    for case in [("s", [("A_i_j_k = B_j_i_k", "A", ["B"])], {"A": (100, 90, 64), "B": (90, 100, 64)}, False),
                 ("t", [("A_i_j = B_j_i", "A", ["B"])], {"A": (100000, 3), "B": (3, 100000)}, False)]:
        got, plan = gu.run_case_on_gpu(case)
        assert gu.families(plan) == ["generic"], plan
        assert np.array_equal(got["A"], gu.oracle_case(case)["A"])
