"""Non-contraction operations either side of the contraction path: batched 1x1 / 2x2 / 3x3
inverse and determinant, FlatIndexedScatter / FlatIndexedSumGather and IndexMapping.
CPU part: the C restatement against the reference outputs, and the inverse map.
GPU part (-m gpu): the CUDA kernels through the engine's C ABI, bit for bit."""
import ctypes
import os

import numpy as np
import pytest

import acrotensor_b200 as ab
import cases
from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib
from oracle import oracle

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


@pytest.mark.parametrize("case", cases.OPS_INV_DET, ids=lambda c: c[0])
def test_restated_inverse_and_determinant_match_reference_outputs(case):
    name, dim, batch = case
    a = cases.make_matrices(name, dim, batch)
    assert cases.digest({"A": a}) == str(GOLDEN[name + "/inputs_sha256"])
    inv, det = oracle.batch_inv_det("port", a)
    assert np.array_equal(inv, GOLDEN[name + "/out/inv"]) and np.array_equal(det, GOLDEN[name + "/out/det"])
    only_det = oracle.batch_inv_det("port", a, want_inv=False)[1]
    assert np.array_equal(only_det, det)


def test_three_by_three_inverse_keeps_the_reference_layout():
    # ops/NativeCPUOps.hpp:62-74 stores entry (r,c) of the true inverse at position (c,r)
    a = cases.make_matrices("layout", 3, (5,))
    inv, det = oracle.batch_inv_det("port", a)
    true_inv = np.linalg.inv(a)
    assert np.allclose(np.swapaxes(inv, -1, -2), true_inv, rtol=1e-12, atol=1e-12)
    assert np.allclose(det, np.linalg.det(a), rtol=1e-12)


@pytest.mark.parametrize("case", cases.OPS_INDEXED, ids=lambda c: c[0])
def test_restated_scatter_gather_match_reference_outputs(case):
    name, domain, rng_size = case
    mapping, dom_vals, rng_vals = cases.make_indexed(name, domain, rng_size)
    assert cases.digest({"M": mapping, "D": dom_vals, "R": rng_vals}) == str(GOLDEN[name + "/inputs_sha256"])
    assert np.array_equal(oracle.flat_indexed("port", dom_vals, mapping, domain, False), GOLDEN[name + "/out/scatter"])
    assert np.array_equal(oracle.flat_indexed("port", rng_vals, mapping, domain, True), GOLDEN[name + "/out/gather"])


@pytest.mark.parametrize("case", cases.OPS_INDEXED, ids=lambda c: c[0])
def test_inverse_map_is_a_stable_grouping(case):
    name, domain, rng_size = case
    mapping, _, _ = cases.make_indexed(name, domain, rng_size)
    m = ab.IndexMapping(domain, rng_size, mapping)
    assert m.inverse() is None
    m.ComputeInverse()
    inv, off = m.inverse()
    assert off[0] == 0 and off[-1] == rng_size and np.all(np.diff(off) >= 0)
    for d in range(domain):
        group = inv[off[d]:off[d + 1]]
        assert np.all(mapping[group] == d) and np.all(np.diff(group) > 0)      # ascending positions: stable
    assert sorted(inv.tolist()) == list(range(rng_size))
    with pytest.raises(ab.AcroError):
        m.ComputeInverse()                                                      # only once, as in the reference
    if oracle.have("ref") and len(set(mapping.tolist())) == domain:
        # with every domain entry referenced the arrays equal the reference's ComputeInverse()
        _, ref_inv, ref_off = oracle.flat_indexed("ref", np.zeros(rng_size), mapping, domain, True, with_inverse=True)
        assert np.array_equal(inv, ref_inv) and np.array_equal(off, ref_off)


def test_index_mapping_rejects_entries_outside_the_domain():
    m = ab.IndexMapping(4, 3, [0, 4, 1])
    with pytest.raises(ab.AcroError):
        m.ComputeInverse()


def test_matrix_batch_shape_rules():
    # unittest/kernel/test_TensorEngine.cpp:606-623
    te = ab.TensorEngine("Cuda")
    for bad in (ab.Tensor(10), ab.Tensor(3), ab.Tensor(3, 2), ab.Tensor(4, 4)):
        with pytest.raises(ab.AcroError):
            te.BatchMatrixInverse(bad, bad)
    with pytest.raises(ab.AcroError):
        te.BatchMatrixInverse(ab.Tensor(3, 3), ab.Tensor(2, 2))
    with pytest.raises(ab.AcroError):
        te.BatchMatrixDet(ab.Tensor(9), ab.Tensor(10, 3, 3))
    with pytest.raises(ab.AcroError):
        te.FlatIndexedScatter(ab.Tensor(7), ab.Tensor(6), ab.IndexMapping(6, 8))


# ---------------------------------------------------------------------------- GPU

@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.OPS_INV_DET, ids=lambda c: c[0])
def test_engine_inverse_and_determinant_bit_identical(case):
    name, dim, batch = case
    a = cases.make_matrices(name, dim, batch)
    inv, det = np.zeros_like(a), np.zeros(batch)
    te = ab.TensorEngine("Cuda")
    A, I, D = ab.Tensor(a.shape, hdata=a), ab.Tensor(a.shape, hdata=inv), ab.Tensor(det.shape, hdata=det)
    te.BatchMatrixInvDet(I, D, A)
    I.MoveFromGPU(); D.MoveFromGPU()
    assert np.array_equal(inv, GOLDEN[name + "/out/inv"]) and np.array_equal(det, GOLDEN[name + "/out/det"])
    det2 = np.zeros(batch)
    D2 = ab.Tensor(det2.shape, hdata=det2)
    te.BatchMatrixDet(D2, A)
    D2.MoveFromGPU()
    assert np.array_equal(det2, det)
    te.BatchMatrixInverse(A, A)                   # in place, as the reference's tests do
    A.MoveFromGPU()
    assert np.array_equal(a, GOLDEN[name + "/out/inv"])
    assert lib().acro_b200_device_status() == _lib.OK


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.OPS_INDEXED, ids=lambda c: c[0])
def test_engine_scatter_gather_bit_identical(case):
    name, domain, rng_size = case
    mapping, dom_vals, rng_vals = cases.make_indexed(name, domain, rng_size)
    te = ab.TensorEngine("Cuda")
    m = ab.IndexMapping(domain, rng_size, mapping)
    big, small = np.zeros(rng_size), np.zeros(domain)
    T = ab.Tensor(domain, hdata=dom_vals)
    B = ab.Tensor(rng_size, hdata=big)
    te.FlatIndexedScatter(B, T, m)
    B.MoveFromGPU()
    assert np.array_equal(big, GOLDEN[name + "/out/scatter"])
    S, R = ab.Tensor(domain, hdata=small), ab.Tensor(rng_size, hdata=rng_vals)
    te.FlatIndexedSumGather(S, R, m)
    S.MoveFromGPU()
    assert np.array_equal(small, GOLDEN[name + "/out/gather"])


@pytest.mark.gpu
def test_inverse_determinant_kernel_sizes_and_alignment():
    import torch
    rng = np.random.default_rng(21)
    for dim, count, offset in ((3, 1, 0), (3, 255, 0), (3, 256, 0), (3, 257, 0), (3, 100000, 0), (3, 1000, 1), (2, 5000, 0), (1, 777, 0)):
        a = rng.random((count, dim, dim)) * 2 - 1 + 2 * np.eye(dim)
        ref_inv, ref_det = oracle.batch_inv_det("port", a)
        flat = torch.zeros(a.size + offset, dtype=torch.float64, device="cuda")
        flat[offset:] = torch.from_numpy(a.reshape(-1)).cuda()
        inv = torch.zeros(a.size, dtype=torch.float64, device="cuda")
        det = torch.zeros(count, dtype=torch.float64, device="cuda")
        check(lib().acro_b200_batch_inv_det(ctypes.c_void_p(flat.data_ptr() + 8 * offset), ctypes.c_void_p(inv.data_ptr()),
                                            ctypes.c_void_p(det.data_ptr()), count, dim, None))
        assert np.array_equal(inv.cpu().numpy().reshape(a.shape), ref_inv), (dim, count, offset)
        assert np.array_equal(det.cpu().numpy(), ref_det.reshape(-1))
    assert lib().acro_b200_batch_inv_det(None, None, None, 5, 3, None) == _lib.EINVAL
    x = torch.zeros(64, dtype=torch.float64, device="cuda")
    p = ctypes.c_void_p(x.data_ptr())
    assert lib().acro_b200_batch_inv_det(p, p, None, 4, 4, None) == _lib.EUNSUPPORTED
    assert lib().acro_b200_device_status() == _lib.OK
