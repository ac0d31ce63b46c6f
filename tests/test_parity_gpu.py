"""GPU parity: the CUDA path, reached through the C ABI, against the oracle and the
committed reference outputs.  Bit-exact where the kernel family reproduces the
reference's operation order (generic, pointwise_sym); otherwise within
1e-12 * sum|terms| (the tolerance the benchmark definition states for fp64; the gap is
summation order and fused multiply-add)."""
import ctypes
import os

import numpy as np
import pytest

import acrotensor_b200 as ab
import cases
import gpu_util as gu
from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-12
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


@pytest.mark.parametrize("case", cases.all_cases(), ids=lambda c: c[0])
def test_engine_matches_reference_outputs(case):
    got, plan = gu.run_case_on_gpu(case)
    exact = set(gu.families(plan)) <= gu.BIT_EXACT_FAMILIES and "CTA per range of terms" not in plan
    mags = None
    for n in cases.written(case):
        ref = GOLDEN["%s/out/%s" % (case[0], n)]
        if exact:
            assert np.array_equal(got[n], ref), (n, plan)
        else:
            mags = mags or gu.oracle_case(case, absolute=True)
            err = oracle.parity_error(got[n], ref, mags[n])
            assert err <= TOL, (n, err, plan)


def test_readme_example_n1000():
    # README.md:26-62: 1000 random 3x3 matrices summed on the GPU.
    rng = np.random.default_rng(11)
    a, b, s = rng.random((1000, 3, 3)), np.ones(1000), np.zeros((3, 3))
    A, B, S = ab.Tensor(1000, 3, 3, hdata=a), ab.Tensor(1000, hdata=b), ab.Tensor(3, 3, hdata=s)
    for t in (A, B, S):
        t.MapToGPU()
    A.MoveToGPU(); B.MoveToGPU(); S.SwitchToGPU()
    te = ab.TensorEngine("Cuda")
    te("S_i_j = A_n_i_j B_n", S, A, B)
    S.MoveFromGPU()
    ref = np.zeros((3, 3))
    oracle.contract("port", "S_i_j = A_n_i_j B_n", ref, a, b)
    assert np.max(np.abs(s - ref) / ref) <= TOL
    te("S_i_j = A_n_i_j", S, A)          # "same result as before since n is still contracted"
    S.MoveFromGPU()
    assert np.max(np.abs(s - ref) / ref) <= TOL


def test_true_subtraction_on_the_gpu():
    # The reference's generated CUDA kernel subtracts for "-=" (exec/CudaExecutor.cpp:536);
    # its CPU executor does not.  The GPU library follows the GPU semantics.
    rng = np.random.default_rng(2)
    b, c, a0 = rng.random((3, 5)), rng.random((4, 5)), rng.random((3, 4))
    a = a0.copy()
    te = ab.TensorEngine("Cuda")
    A, B, C = ab.Tensor(3, 4, hdata=a), ab.Tensor(3, 5, hdata=b), ab.Tensor(4, 5, hdata=c)
    te("A_m_n-=B_m_j C_n_j", A, B, C)
    A.MoveFromGPU()
    prod = np.zeros((3, 4))
    oracle.contract("port", "A_m_n=B_m_j C_n_j", prod, b, c)
    assert np.array_equal(a, a0 - prod)


def test_tensor_gpu_flag_semantics():
    # unittest/tensor/test_Tensor.cpp:155-184
    t = ab.Tensor(2)
    t.Set(3.0)
    assert list(t.numpy()) == [3.0, 3.0]
    t.MapToGPU()
    assert t.IsMappedToGPU() and not t.IsOnGPU()
    with pytest.raises(ab.AcroError):
        t.MapToGPU()
    t.SwitchToGPU()
    assert t.IsOnGPU()
    t.Set(9.0)
    assert list(t.numpy()) == [3.0, 3.0]          # not moved back yet
    t.MoveFromGPU()
    assert not t.IsOnGPU() and list(t.numpy()) == [9.0, 9.0]
    t.MoveToGPU(); t.Mult(0.5); t.MoveFromGPU()
    assert list(t.numpy()) == [4.5, 4.5]
    t.UnmapFromGPU()
    assert not t.IsMappedToGPU()
    with pytest.raises(ab.AcroError):
        t.UnmapFromGPU()


def test_slice_gpu_semantics():
    # unittest/tensor/test_SliceTensor.cpp:105-168
    host = np.zeros((2, 10, 4, 4))
    t = ab.Tensor(2, 10, 4, 4, hdata=host)
    t.SwitchToGPU()
    s0, s1 = ab.SliceTensor(t, 0), ab.SliceTensor(t, 1)
    s0.Set(1.0); s1.Set(2.0)
    t.MoveFromGPU()
    assert np.all(host[0] == 1.0) and np.all(host[1] == 2.0)
    t2 = ab.Tensor(2, 3)
    t2.MapToGPU()
    s = ab.SliceTensor(t2, 0)
    assert s.IsMappedToGPU() and s.GetCurrentData() == s.GetData()
    s.MoveToGPU()
    assert t2.IsOnGPU() and s.IsOnGPU() and s.GetCurrentData() == s.GetDeviceData()
    assert s.GetDeviceData() == t2.GetDeviceData()
    s1b = ab.SliceTensor(t2, 1)
    assert s1b.GetDeviceData() == t2.GetDeviceData() + 3 * 8
    s.Set(2.0)
    t2.MoveFromGPU()
    assert not s.IsOnGPU() and list(s.numpy()) == [2.0, 2.0, 2.0]


def test_slice_outputs_keep_the_rest_of_the_parent():
    # unittest/kernel/test_TensorEngine.cpp:311-356: U1, U2 are the two halves of U.
    rng = np.random.default_rng(4)
    u = rng.random((2, 5, 4, 4))
    keep = u.copy()
    g, x = rng.random((4, 4)), rng.random((5, 4, 4))
    U = ab.Tensor(u.shape, hdata=u)
    U1 = ab.SliceTensor(U, 0)
    te = ab.TensorEngine("Cuda")
    te("U1_e_k1_k2 = G_k1_i1 X_e_i1_k2", U1, ab.Tensor(g.shape, hdata=g), ab.Tensor(x.shape, hdata=x))
    U.MoveFromGPU()
    ref = np.zeros((5, 4, 4))
    oracle.contract("port", "U1_e_k1_k2 = G_k1_i1 X_e_i1_k2", ref, g, x)
    assert np.array_equal(u[0], ref) and np.array_equal(u[1], keep[1])


def test_external_device_pointer(torch):
    # unittest/kernel/test_TensorEngine.cpp:166-185
    a = np.arange(125, dtype=np.float64)
    dev = torch.zeros(125, dtype=torch.float64, device="cuda")
    A = ab.Tensor(125, hdata=a, ddata=dev, ongpu=False)
    b = np.zeros(125)
    B = ab.Tensor(125, hdata=b)
    te = ab.TensorEngine("Cuda")
    te("B_i=A_i", B, A)
    B.MoveFromGPU()
    assert np.array_equal(a, b)
    assert np.array_equal(dev.cpu().numpy(), a)     # the caller's buffer was used as the mirror


def test_caches_and_repeated_calls_are_deterministic():
    rng = np.random.default_rng(6)
    a, b = rng.random((5000, 3, 3)), rng.random(5000)
    outs = []
    te = ab.TensorEngine("Cuda")
    A, B = ab.Tensor(a.shape, hdata=a), ab.Tensor(b.shape, hdata=b)
    for _ in range(3):
        s = np.zeros((3, 3))
        S = ab.Tensor(3, 3, hdata=s)
        te("S_i_j = A_n_i_j B_n", S, A, B)
        S.MoveFromGPU()
        outs.append(s)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])   # fixed summation order
    te.Clear()
    s = np.zeros((3, 3))
    S = ab.Tensor(3, 3, hdata=s)
    te("S_i_j = A_n_i_j B_n", S, A, B)
    S.MoveFromGPU()
    assert np.array_equal(s, outs[0])


# ------------------------------------------------------------------ kernel layer, called directly

def test_fill_and_scale(torch):
    x = torch.zeros(100003, dtype=torch.float64, device="cuda")
    check(lib().acro_b200_fill(gu.dev_ptr(x), x.numel(), 1.5, None))
    check(lib().acro_b200_scale(gu.dev_ptr(x), x.numel(), -2.0, None))
    torch.cuda.synchronize()
    assert bool((x == -3.0).all())
    assert lib().acro_b200_fill(None, 5, 0.0, None) == _lib.EINVAL
    assert lib().acro_b200_fill(None, 0, 0.0, None) == _lib.OK


@pytest.mark.parametrize("rows,F,weighted,offset", [
    (1, 9, True, 0), (255, 9, True, 0), (1000, 9, True, 0), (112 * 37 + 5, 9, True, 0), (100000, 9, False, 0),
    (100001, 9, True, 1), (5000, 1, True, 0), (5000, 7, False, 1), (4097, 16, True, 0), (777, 256, True, 0),
    (300000, 27, True, 0), (1 << 20, 9, True, 0),
])
def test_reduce_batch_kernel(torch, rows, F, weighted, offset):
    rng = np.random.default_rng(rows + F)
    a = rng.random((rows, F)) * 2 - 1
    w = rng.random(rows) + 0.5
    # offset=1 places A on an 8-byte (not 16-byte) boundary, as a slice of a larger tensor would
    dev_a = torch.zeros(rows * F + offset, dtype=torch.float64, device="cuda")
    dev_a[offset:] = torch.from_numpy(a.reshape(-1)).cuda()
    dev_w = torch.from_numpy(w).cuda()
    out = torch.full((F,), 5.0, dtype=torch.float64, device="cuda")
    nbytes = lib().acro_b200_reduce_batch_scratch_bytes(F)
    scratch = torch.empty(nbytes // 8 + 1, dtype=torch.float64, device="cuda")
    a_ptr = ctypes.c_void_p(dev_a.data_ptr() + 8 * offset)
    ref = np.zeros(F)
    mags = np.zeros(F)
    if weighted:
        oracle.contract("port", "S_f = A_n_f W_n", ref, a, w)
        oracle.contract("port", "S_f = A_n_f W_n", mags, np.abs(a), w)
    else:
        oracle.contract("port", "S_f = A_n_f", ref, a)
        oracle.contract("port", "S_f = A_n_f", mags, np.abs(a))
    results = []
    for op, expect in ((_lib.OP_ASSIGN, ref), (_lib.OP_ADD, 5.0 + ref), (_lib.OP_SUB, 5.0 - ref)):
        out.fill_(5.0)
        for _ in range(2):     # second call reuses the scratch left by the first
            if _ == 1:
                out.fill_(5.0)
            check(lib().acro_b200_reduce_batch(a_ptr, gu.dev_ptr(dev_w) if weighted else None, gu.dev_ptr(out), rows, F, op,
                                               gu.dev_ptr(scratch), nbytes, None))
        got = out.cpu().numpy()
        assert oracle.parity_error(got, expect, mags + 5.0) <= TOL, (op, got, expect)
        results.append(got)


def test_reduce_batch_rejects_bad_arguments(torch):
    x = torch.zeros(64, dtype=torch.float64, device="cuda")
    p = gu.dev_ptr(x)
    assert lib().acro_b200_reduce_batch(p, None, p, 4, 9, 0, p, 16, None) == _lib.EINVAL        # scratch too small
    assert lib().acro_b200_reduce_batch(p, None, p, 4, 300, 0, p, 1 << 30, None) == _lib.EUNSUPPORTED
    assert lib().acro_b200_reduce_batch(None, None, p, 4, 9, 0, p, 1 << 30, None) == _lib.EINVAL
    assert lib().acro_b200_reduce_batch(p, None, p, 0, 9, 0, p, 1 << 30, None) == _lib.EINVAL
    assert b"scratch" in lib().acro_b200_last_error() or True


@pytest.mark.parametrize("dim,points,same,nscal,op", [
    (3, 1, True, 2, 0), (3, 255, True, 2, 0), (3, 257, False, 1, 0), (3, 64 * 33, True, 2, 0), (2, 1000, False, 2, 0),
    (1, 513, False, 1, 0), (3, 700, True, 0, 0), (3, 700, False, 3, 1), (2, 300, True, 1, 2), (3, 1 << 16, True, 2, 0),
])
def test_pointwise_sym_kernel(torch, dim, points, same, nscal, op):
    rng = np.random.default_rng(points + dim)
    k = 64 if points % 64 == 0 else 1
    e = points // k
    x = rng.random((e, k, dim, dim)) * 2 - 1
    y = x if same else rng.random((e, k, dim, dim)) * 2 - 1
    scal_shapes = [(k,), (e, k), (e,)][:nscal]
    scal_idx = ["_k", "_e_k", "_e"][:nscal]
    scalars = [rng.random(s) + 0.5 for s in scal_shapes]
    d0 = rng.random((e, k, dim, dim))
    kernel = "D_e_k_m_n %s %s X_e_k_m_l Y_e_k_n_l" % (["=", "+=", "-="][op], " ".join("S%d%s" % (i, s) for i, s in enumerate(scal_idx)))
    ref = d0.copy()
    if op == 2:
        prod = np.zeros_like(d0)
        oracle.contract("port", kernel.replace("-=", "="), prod, *scalars, x, y)
        ref = d0 - prod
    else:
        oracle.contract("port", kernel, ref, *scalars, x, y)

    desc = _lib.PointwiseDesc()
    desc.dim, desc.op, desc.n_point_loops, desc.n_scalars = dim, op, 2, nscal
    desc.cell_points = 1
    desc.point_extent[0], desc.point_extent[1] = e, k
    steps = {"_k": (0, 1), "_e_k": (k, 1), "_e": (1, 0)}
    for i, s in enumerate(scal_idx):
        desc.scalar_step[i][0], desc.scalar_step[i][1] = steps[s]
    assert lib().acro_b200_pointwise_sym_supported(ctypes.byref(desc)) == 1
    dx = torch.from_numpy(x).cuda()
    dy = dx if same else torch.from_numpy(y).cuda()
    dd = torch.from_numpy(d0).cuda()
    ds = [torch.from_numpy(s).cuda() for s in scalars]
    ptrs = (ctypes.c_void_p * _lib.MAX_SCALARS)(*[t.data_ptr() for t in ds])
    check(lib().acro_b200_pointwise_sym(ctypes.byref(desc), ptrs, gu.dev_ptr(dx), gu.dev_ptr(dy), gu.dev_ptr(dd), None))
    got = dd.cpu().numpy()
    assert np.array_equal(got, ref)     # same operation order as the reference: bit-identical


def test_generic_kernel_descriptor_checks(torch):
    d = _lib.GenericDesc()
    x = torch.zeros(8, dtype=torch.float64, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(x.data_ptr())
    d.n_loops, d.n_outer, d.n_inputs, d.op = 0, 0, 1, 0
    assert lib().acro_b200_generic_launch(ctypes.byref(d), gu.dev_ptr(x), ptrs, None, 0, None) == _lib.EINVAL
    d.n_loops, d.n_outer = 1, 1
    d.extent[0] = 0
    assert lib().acro_b200_generic_launch(ctypes.byref(d), gu.dev_ptr(x), ptrs, None, 0, None) == _lib.EINVAL
    d.extent[0], d.out_step[0] = 8, 1
    d.in_step[0][0] = 1
    x2 = torch.arange(8, dtype=torch.float64, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(x2.data_ptr())
    check(lib().acro_b200_generic_launch(ctypes.byref(d), gu.dev_ptr(x), ptrs, None, 0, None))
    assert bool((x == x2).all())


# ------------------------------------------------------------------ full-size properties

def test_full_size_reduction_properties(torch):
    """n = 2^26 (the benchmark size): exact answers that hold for any summation order."""
    n = 1 << 26
    a = torch.ones(n, 3, 3, dtype=torch.float64, device="cuda")
    b = torch.full((n,), 0.5, dtype=torch.float64, device="cuda")
    s = torch.zeros(3, 3, dtype=torch.float64, device="cuda")
    nbytes = lib().acro_b200_reduce_batch_scratch_bytes(9)
    scratch = torch.empty(nbytes // 8 + 1, dtype=torch.float64, device="cuda")
    check(lib().acro_b200_reduce_batch(gu.dev_ptr(a), gu.dev_ptr(b), gu.dev_ptr(s), n, 9, 0, gu.dev_ptr(scratch), nbytes, None))
    assert bool((s == n / 2).all())                 # sums of 0.5 are exact in fp64
    # linearity with power-of-two scaling is exact too
    a.mul_(4.0)
    check(lib().acro_b200_reduce_batch(gu.dev_ptr(a), gu.dev_ptr(b), gu.dev_ptr(s), n, 9, 0, gu.dev_ptr(scratch), nbytes, None))
    assert bool((s == 2.0 * n).all())
    # one marked row per column position: the result picks exactly those rows
    a.zero_()
    rows = torch.tensor([0, 1, 111, 112, n // 2, n - 113, n - 112, n - 2, n - 1], device="cuda")
    a.view(n, 9)[rows, torch.arange(9, device="cuda")] = torch.arange(1, 10, dtype=torch.float64, device="cuda")
    b.fill_(2.0)
    check(lib().acro_b200_reduce_batch(gu.dev_ptr(a), gu.dev_ptr(b), gu.dev_ptr(s), n, 9, 0, gu.dev_ptr(scratch), nbytes, None))
    assert s.view(-1).tolist() == [2.0 * v for v in range(1, 10)]


def test_full_size_pointwise_properties(torch):
    """E = 2^20 elements x 64 points: identity Jacobians give D = W_k * I exactly; a
    seeded sample of points is compared with the oracle bit for bit."""
    E, K = 1 << 20, 64
    rng = np.random.default_rng(8)
    w = rng.random(K) + 0.5
    jinv = torch.zeros(E, K, 3, 3, dtype=torch.float64, device="cuda")
    jinv[..., 0, 0] = 1.0; jinv[..., 1, 1] = 1.0; jinv[..., 2, 2] = 1.0
    det = torch.ones(E, K, dtype=torch.float64, device="cuda")
    dw = torch.from_numpy(w).cuda()
    d = torch.empty(E, K, 3, 3, dtype=torch.float64, device="cuda")
    desc = _lib.PointwiseDesc()
    desc.dim, desc.op, desc.n_point_loops, desc.n_scalars = 3, 0, 2, 2
    desc.cell_points = 1
    desc.point_extent[0], desc.point_extent[1] = E, K
    desc.scalar_step[0][0], desc.scalar_step[0][1] = 0, 1
    desc.scalar_step[1][0], desc.scalar_step[1][1] = K, 1
    ptrs = (ctypes.c_void_p * _lib.MAX_SCALARS)(dw.data_ptr(), det.data_ptr())
    check(lib().acro_b200_pointwise_sym(ctypes.byref(desc), ptrs, gu.dev_ptr(jinv), gu.dev_ptr(jinv), gu.dev_ptr(d), None))
    expect = dw.view(1, K, 1, 1) * torch.eye(3, dtype=torch.float64, device="cuda").view(1, 1, 3, 3)
    assert bool((d == expect).all())
    # seeded random data on a sample of elements, checked against the oracle
    sample = torch.tensor(sorted(rng.choice(E, 16, replace=False).tolist()) + [0, E - 1], device="cuda")
    js = torch.from_numpy(rng.random((len(sample), K, 3, 3)) * 2 - 1).cuda()
    ds = torch.from_numpy(rng.random((len(sample), K)) + 0.5).cuda()
    jinv[sample] = js
    det[sample] = ds
    check(lib().acro_b200_pointwise_sym(ctypes.byref(desc), ptrs, gu.dev_ptr(jinv), gu.dev_ptr(jinv), gu.dev_ptr(d), None))
    ref = np.zeros((len(sample), K, 3, 3))
    oracle.contract("port", "D_e_k_m_n = W_k DetJ_e_k Jinv_e_k_m_l Jinv_e_k_n_l", ref, w, ds.cpu().numpy(), js.cpu().numpy(), js.cpu().numpy())
    assert np.array_equal(d[sample].cpu().numpy(), ref)
    untouched = torch.ones(E, dtype=torch.bool, device="cuda")
    untouched[sample] = False
    assert bool((d[untouched] == expect).all())


@pytest.mark.parametrize("cells,kshape,dim,swapped,same,op", [
    (1001, (64,), 3, False, True, "="), (333, (5, 5, 5), 3, True, True, "="), (70, (4, 4), 2, False, False, "="),
    (515, (5, 5, 5), 3, True, False, "="), (9, (3, 3, 3), 3, True, True, "+="), (300, (7,), 3, False, True, "="),
    (1000, (300,), 3, False, True, "="), (64, (2, 2), 1, True, False, "="),
])
def test_pointwise_cell_major_layout_through_the_engine(cells, kshape, dim, swapped, same, op):
    """D_e_m_n_k.. = W_k.. Det_e_k.. X_e_k.._a_l Y_e_k.._b_l : the layout of the reference's own
    partial-assembly tests (block indices before the trailing point indices)."""
    rng = np.random.default_rng(cells + dim)
    kidx = ["k%d" % (i + 1) for i in range(len(kshape))]
    ks = "_".join(kidx)
    a, b = ("n", "m") if swapped else ("m", "n")
    kernel = "D_e_m_n_%s %s W_%s Det_e_%s X_e_%s_%s_l %s_e_%s_%s_l" % (ks, op, ks, ks, ks, a, "X" if same else "Y", ks, b)
    shape_k = tuple(kshape)
    w = rng.random(shape_k) + 0.5
    det = rng.random((cells,) + shape_k) + 0.5
    x = rng.random((cells,) + shape_k + (dim, dim)) * 2 - 1
    y = x if same else rng.random((cells,) + shape_k + (dim, dim)) * 2 - 1
    d0 = rng.random((cells, dim, dim) + shape_k)
    ref = d0.copy()
    oracle.contract("port", kernel, ref, w, det, x, y)
    got = d0.copy()
    te = ab.TensorEngine("Cuda")
    D = ab.Tensor(got.shape, hdata=got)
    X = ab.Tensor(x.shape, hdata=x)
    Y = X if same else ab.Tensor(y.shape, hdata=y)
    args = (ab.Tensor(w.shape, hdata=w), ab.Tensor(det.shape, hdata=det), X, Y)
    plan = te.GetImplementation(kernel, D, *args)
    assert "family=pointwise_sym" in plan and ("cell-major" in plan or int(np.prod(kshape)) == 1)
    te(kernel, D, *args)
    D.MoveFromGPU()
    assert np.array_equal(got, ref), plan           # same operation order as the reference: bit-identical
    assert lib().acro_b200_device_status() == _lib.OK


def test_fuzzed_strings_on_the_generic_path_are_bit_identical():
    """300 seeded random strings through the engine: "=" and "+=" must equal the oracle bit for
    bit (the generic kernel repeats its operation order); "-=" is checked against
    out_old - (oracle "=" result), because the reference's CPU executor never subtracts."""
    import fuzz
    rng = np.random.default_rng(5)
    te = ab.TensorEngine("Cuda")
    for text, shapes, in_names, op in fuzz.cases(7, 300):
        tensors = {n: rng.random(s) * 2 - 1 for n, s in shapes.items()}
        ins = [tensors[n] for n in in_names]
        got = tensors["A"].copy()
        handles = {}
        for n in in_names:
            if n not in handles:
                handles[n] = ab.Tensor(tensors[n].shape, hdata=tensors[n])
        A = ab.Tensor(got.shape, hdata=got)
        te(text, A, *[handles[n] for n in in_names])
        A.MoveFromGPU()
        if op == "-=":
            prod = np.zeros_like(got)
            oracle.contract("port", text.replace("-=", "="), prod, *ins)
            ref = tensors["A"] - prod
        else:
            ref = tensors["A"].copy()
            oracle.contract("port", text, ref, *ins)
        assert np.array_equal(got, ref), text
