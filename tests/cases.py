"""Contraction cases shared by the golden-vector generator, the oracle tests and the GPU
parity tests.  Each case: (name, [(kernel, out, [ins])...], {tensor: shape}, multi?).
The strings of the first group are the ones the reference's own unit tests exercise
(unittest/kernel/test_TensorEngine.cpp:49-143, 211-228, 232-590, 632-687 of
LLNL/acrotensor); the second group is the five benchmark configurations at small batch."""
import numpy as np

from acrotensor_b200.workloads import WORKLOADS

REFERENCE_TEST_CASES = [
    ("copy", [("A_i=B_i", "A", ["B"])], {"A": (3,), "B": (3,)}, False),
    ("elementwise", [("A_i=B_iC_i", "A", ["B", "C"])], {"A": (3,), "B": (3,), "C": (3,)}, False),
    ("diagonal", [("A_i=B_i_i", "A", ["B"])], {"A": (3,), "B": (3, 3)}, False),
    ("contract_broadcast", [("A_i=B_j_j", "A", ["B"])], {"A": (3,), "B": (3, 3)}, False),
    ("matvec", [("A_i = C_i_j B_j", "A", ["C", "B"])], {"A": (3,), "C": (3, 3), "B": (3,)}, False),
    ("transpose", [("A_i_j=B_j_i", "A", ["B"])], {"A": (4, 5), "B": (5, 4)}, False),
    ("mmt", [("A_m_n=B_m_j B_n_j", "A", ["B", "B"])], {"A": (3, 3), "B": (3, 3)}, False),
    ("singleton", [("A_i=B_j_k_l_m_n", "A", ["B"])], {"A": (3,), "B": (1, 2, 3, 1, 5)}, False),
    ("multikernel_last_wins", [("A_i = B1_i", "A", ["B1"]), ("A_i = C_i_j B2_j", "A", ["C", "B2"])],
     {"A": (3,), "B1": (3,), "B2": (3,), "C": (3, 3)}, True),
    ("mass2d_d", [("D_e_k1_k2 = W_k1_k2 T_e_k1_k2", "D", ["W", "T"])],
     {"D": (10, 4, 4), "W": (4, 4), "T": (10, 4, 4)}, False),
    ("mass2d_m", [("M_e_i1_i2_j1_j2=B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2", "M", ["B", "B", "B", "B", "D"])],
     {"M": (10, 4, 4, 4, 4), "B": (4, 4), "D": (10, 4, 4)}, False),
    ("stiff2d_bx", [("BX_e_i1_k2 = B_k2_i2 X_e_i1_i2", "T", ["B", "X"]),
                    ("U1_e_k1_k2 = G_k1_i1 BX_e_i1_k2", "U1", ["G", "T"])],
     {"T": (5, 4, 4), "B": (4, 4), "G": (4, 4), "X": (5, 4, 4), "U1": (5, 4, 4)}, False),
    ("stiff2d_z", [("Z_m_e_k1_k2 = D_e_m_n_k1_k2 U_n_e_k1_k2", "Z", ["D", "U"])],
     {"Z": (2, 5, 4, 4), "D": (5, 2, 2, 4, 4), "U": (2, 5, 4, 4)}, False),
    ("stiff3d", [("S_e_i1_i2_i3_j1_j2_j3 = Bt1_i1_j1_k1_m_n Bt2_i2_j2_k2_m_n Bt3_i3_j3_k3_m_n D_e_k1_k2_k3_m_n",
                  "S", ["Bt1", "Bt2", "Bt3", "D"])],
     {"S": (2, 3, 3, 3, 3, 3, 3), "Bt1": (3, 3, 3, 3, 3), "Bt2": (3, 3, 3, 3, 3), "Bt3": (3, 3, 3, 3, 3),
      "D": (2, 3, 3, 3, 3, 3)}, False),
    ("dtensor2d", [("D_e_m_n_k1_k2 = W_e_k1_k2 C_e_k1_k2 Jdet_e_k1_k2 Jinv_e_k1_k2_m_j Jinv_e_k1_k2_n_j",
                    "D", ["W", "C", "Jdet", "Jinv", "Jinv"])],
     {"D": (10, 2, 2, 2, 2), "W": (10, 2, 2), "C": (10, 2, 2), "Jdet": (10, 2, 2), "Jinv": (10, 2, 2, 2, 2)}, False),
    ("dtensor3d", [("D_e_m_n_k1_k2_k3 = W_k1_k2_k3 C_e_k1_k2_k3 Jdet_e_k1_k2_k3 Jinv_e_k1_k2_k3_n_j Jinv_e_k1_k2_k3_m_j",
                    "D", ["W", "C", "Jdet", "Jinv", "Jinv"])],
     {"D": (4, 3, 3, 5, 5, 5), "W": (5, 5, 5), "C": (4, 5, 5, 5), "Jdet": (4, 5, 5, 5), "Jinv": (4, 5, 5, 5, 3, 3)}, False),
    ("batched_matmul", [("I_b_i_k = TI_b_i_j T_b_j_k", "I", ["TI", "T"])],
     {"I": (10, 3, 3), "TI": (10, 3, 3), "T": (10, 3, 3)}, False),
    ("accumulate", [("A_m_n+=B_m_j C_n_j", "A", ["B", "C"])], {"A": (3, 4), "B": (3, 5), "C": (4, 5)}, False),
    ("pointwise_2x2", [("D_p_m_n = S_p X_p_m_l Y_p_n_l", "D", ["S", "X", "Y"])],
     {"D": (37, 2, 2), "S": (37,), "X": (37, 2, 2), "Y": (37, 2, 2)}, False),
    ("three_contracted", [("A_i = B_i_j_k_l C_j D_k_l", "A", ["B", "C", "D"])],
     {"A": (6,), "B": (6, 3, 4, 5), "C": (3,), "D": (4, 5)}, False),
    ("long_dot_products", [("S_a = X_n_a Y_n_a", "S", ["X", "Y"])], {"S": (3,), "X": (40000, 3), "Y": (40000, 3)}, False),
    ("long_two_loop_sums", [("S_a_b += X_n_m_a Y_m_n_b W_m", "S", ["X", "Y", "W"])],
     {"S": (2, 3), "X": (300, 70, 2), "Y": (70, 300, 3), "W": (70,)}, False),
    ("pointwise_noscalar", [("D_p_m_n = X_p_m_l X_p_n_l", "D", ["X", "X"])], {"D": (300, 3, 3), "X": (300, 3, 3)}, False),
    # element products with both operands stored transposed; Gram forms (the same tensor twice; accumulate)
    ("batched_matmul_transposed", [("C_e_i_j = A_e_k_i B_e_j_k", "C", ["A", "B"])],
     {"C": (10, 5, 4), "A": (10, 6, 5), "B": (10, 4, 6)}, False),
    ("gram_normal_equations", [("S_a_b = X_n_a X_n_b", "S", ["X", "X"])], {"S": (6, 6), "X": (30000, 6)}, False),
    ("gram_accumulate", [("S_a_b += X_n_a Y_n_b", "S", ["X", "Y"])], {"S": (20, 24), "X": (4500, 20), "Y": (4500, 24)}, False),
]

SMALL_BATCH = {"cfg0": 1000, "cfg1": 6, "cfg2": 9, "cfg3": 7, "cfg4": 2}


def benchmark_cases():
    out = []
    for w in WORKLOADS:
        b = SMALL_BATCH[w.key]
        out.append((w.key + "_small", list(w.program), w.shapes(b), w.multi))
    return out


def all_cases():
    return REFERENCE_TEST_CASES + benchmark_cases()


def make_tensors(case, seed=7):
    """Seeded inputs in [-1, 1) (outputs start at a seeded value too, which matters for '+=')."""
    name, program, shapes, multi = case
    rng = np.random.default_rng([seed, len(name), sum(map(ord, name))])
    return {n: rng.random(s) * 2.0 - 1.0 for n, s in shapes.items()}


def digest(tensors):
    """Order-independent fingerprint of a dict of arrays (detects generator drift)."""
    import hashlib
    h = hashlib.sha256()
    for n in sorted(tensors):
        h.update(n.encode())
        h.update(np.ascontiguousarray(tensors[n]).tobytes())
    return h.hexdigest()


def written(case):
    return sorted({p[1] for p in case[1]})


def as_oracle_program(case, names):
    return [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in case[1]]


# ---------------------------------------------------------------- non-contraction operations
# (name, matrix dim, batch shape): batched inverse / determinant, as in
# unittest/kernel/test_TensorEngine.cpp:594-706 of the reference
OPS_INV_DET = [("invdet1", 1, (10,)), ("invdet2", 2, (10,)), ("invdet3", 3, (10,)), ("invdet3_batch2", 3, (4, 2)),
               ("invdet3_ragged", 3, (7, 64)), ("invdet2_big", 2, (1031,))]
# (name, domain size, range size): FlatIndexedScatter / FlatIndexedSumGather, :708-745
OPS_INDEXED = [("indexed_6_8", 6, 8), ("indexed_100_1000", 100, 1000), ("indexed_sparse", 50, 20)]


def make_matrices(name, dim, batch):
    rng = np.random.default_rng([11, dim, sum(map(ord, name))])
    a = rng.random(tuple(batch) + (dim, dim)) * 2.0 - 1.0
    a += 2.0 * np.eye(dim)          # comfortably invertible
    return a


def make_indexed(name, domain, rng_size):
    rng = np.random.default_rng([13, domain, rng_size])
    mapping = rng.integers(0, domain, rng_size).astype(np.int32)
    return mapping, rng.random(domain) * 2.0 - 1.0, rng.random(rng_size) * 2.0 - 1.0
