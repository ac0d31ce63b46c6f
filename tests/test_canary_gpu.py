"""Out-of-bounds write detection without a sanitizer: every output (and scratch-free input) of
each kernel family lives inside a larger device buffer whose margins hold a canary pattern;
after the run the margins must be untouched and the result must still match the oracle."""
import numpy as np
import pytest

import acrotensor_b200 as ab
from acrotensor_b200._lib import lib
from acrotensor_b200.runner import alloc_host
from acrotensor_b200.workloads import BY_KEY
from oracle import oracle

pytestmark = pytest.mark.gpu
PAD = 64            # doubles on each side (keeps 16-byte alignment)
CANARY = -7.25e77


class Guarded:
    """A device tensor of `shape` with canary margins, bound to a host array through acro Tensor."""

    def __init__(self, torch, host):
        self.host = host
        self.buf = torch.full((host.size + 2 * PAD,), CANARY, dtype=torch.float64, device="cuda")
        self.view = self.buf[PAD:PAD + host.size]
        self.view.copy_(torch.from_numpy(host.reshape(-1)))
        self.tensor = ab.Tensor(host.shape, hdata=host, ddata=self.buf.data_ptr() + 8 * PAD, ongpu=True)

    def intact(self):
        return bool((self.buf[:PAD] == CANARY).all()) and bool((self.buf[PAD + self.host.size:] == CANARY).all())


@pytest.mark.parametrize("key,batch", [("cfg0", 100003), ("cfg1", 1000), ("cfg1", 37), ("cfg2", 4099), ("cfg3", 1027), ("cfg4", 301)])
def test_benchmark_families_stay_inside_their_buffers(key, batch):
    import torch
    w = BY_KEY[key]
    host = alloc_host(w, batch, w.make_inputs(batch, seed=2))
    g = {n: Guarded(torch, host[n]) for n in host}
    for n in w.names("tmp"):
        g[n].tensor.SetTransient(True)
    te = ab.TensorEngine("Cuda")
    if w.multi:
        te.BeginMultiKernelLaunch()
    for kernel, out, ins in w.program:
        te(kernel, g[out].tensor, *[g[i].tensor for i in ins])
    if w.multi:
        te.EndMultiKernelLaunch()
    torch.cuda.synchronize()
    for n in host:
        assert g[n].intact(), (key, n)
    assert lib().acro_b200_device_status() == 0
    out = w.names("out")[0]
    g[out].tensor.MoveFromGPU()
    got = host[out].copy()
    names = sorted(host)
    prog = [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in w.program]
    mags = [np.abs(host[n]) for n in names]
    oracle.run("port", [host[n] for n in names], prog, multi=w.multi)
    oracle.run("port", mags, prog, multi=w.multi)
    assert oracle.parity_error(got, host[out], mags[names.index(out)]) <= 1e-12


def test_other_families_stay_inside_their_buffers():
    import torch
    rng = np.random.default_rng(4)
    te = ab.TensorEngine("Cuda")
    # cell-major pointwise (pipelined part + direct tail), batched inverse/determinant, scatter/gather, generic (both variants)
    x = rng.random((301, 5, 5, 5, 3, 3)) * 2 - 1
    det = rng.random((301, 5, 5, 5)) + 0.5
    d = np.zeros((301, 3, 3, 5, 5, 5))
    gx, gdet, gd = Guarded(torch, x), Guarded(torch, det), Guarded(torch, d)
    te("D_e_m_n_k1_k2_k3 = Det_e_k1_k2_k3 X_e_k1_k2_k3_n_j X_e_k1_k2_k3_m_j", gd.tensor, gdet.tensor, gx.tensor, gx.tensor)
    a = rng.random((1001, 3, 3)) + 2 * np.eye(3)
    inv, dets = np.zeros_like(a), np.zeros(1001)
    ga, gi, gdt = Guarded(torch, a), Guarded(torch, inv), Guarded(torch, dets)
    te.BatchMatrixInvDet(gi.tensor, gdt.tensor, ga.tensor)
    m = ab.IndexMapping(97, 1000, rng.integers(0, 97, 1000))
    dom, big, back = rng.random(97), np.zeros(1000), np.zeros(97)
    gdom, gbig, gback = Guarded(torch, dom), Guarded(torch, big), Guarded(torch, back)
    te.FlatIndexedScatter(gbig.tensor, gdom.tensor, m)
    te.FlatIndexedSumGather(gback.tensor, gbig.tensor, m)
    xs, ys, s3 = rng.random((40000, 3)), rng.random((40000, 3)), np.zeros(3)
    gxs, gys, gs3 = Guarded(torch, xs), Guarded(torch, ys), Guarded(torch, s3)
    te("S_a = X_n_a Y_n_a", gs3.tensor, gxs.tensor, gys.tensor)
    bt, tr = rng.random((37, 53)), np.zeros((53, 37))
    gbt, gtr = Guarded(torch, bt), Guarded(torch, tr)
    te("A_i_j = B_j_i", gtr.tensor, gbt.tensor)
    torch.cuda.synchronize()
    for g in (gx, gdet, gd, ga, gi, gdt, gdom, gbig, gback, gxs, gys, gs3, gbt, gtr):
        assert g.intact()
    gtr.tensor.MoveFromGPU()
    assert np.array_equal(tr, bt.T)
    gd.tensor.MoveFromGPU()
    ref = np.zeros_like(d)
    oracle.contract("port", "D_e_m_n_k1_k2_k3 = Det_e_k1_k2_k3 X_e_k1_k2_k3_n_j X_e_k1_k2_k3_m_j", ref, det, x, x)
    assert np.array_equal(d, ref)
    assert lib().acro_b200_device_status() == 0


@pytest.mark.parametrize("kernel,shapes", [
    # batched products: streaming variant (ragged last tile), zero-padded tensor-core variant, matrix-vector forms
    ("C_e_i_j = A_e_i_k B_e_k_j", [(1001, 5, 7), (1001, 5, 3), (1001, 3, 7)]),
    ("C_e_i_j += A_e_i_k B_e_k_j", [(203, 27, 27), (203, 27, 27), (203, 27, 27)]),
    ("C_e_i_j = A_e_i_k B_e_k_j", [(77, 33, 50), (77, 33, 64), (77, 64, 50)]),
    ("Y_e_i = M_e_i_j X_e_j", [(1003, 27), (1003, 27, 27), (1003, 27)]),
    ("Y_e_j = X_e_k M_e_k_j", [(501, 9), (501, 5), (501, 5, 9)]),
    # assembly strings through the GEMM (odd sizes: ragged tiles in every direction), the register-blocked generic kernel
    ("M_e_i_j = W_e_q B_q_i C_q_j", [(705, 9, 7), (705, 125), (125, 9), (125, 7)]),
    ("M_e_i1_i2_j1_j2=B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2", [(4100, 4, 4, 4, 4), (4, 4), (4, 4), (4, 4), (4, 4), (4100, 4, 4)]),
    ("T_e_i1_i2_k3 = B_k3_i3 U_e_i1_i2_i3", [(5003, 4, 4, 5), (5, 4), (5003, 4, 4, 4)]),
])
def test_matrix_families_stay_inside_their_buffers(kernel, shapes):
    import torch
    rng = np.random.default_rng(len(kernel))
    host = [rng.random(s) * 2 - 1 for s in shapes]
    start = host[0].copy()
    g = [Guarded(torch, h) for h in host]
    te = ab.TensorEngine("Cuda")
    te(kernel, g[0].tensor, *[x.tensor for x in g[1:]])
    torch.cuda.synchronize()
    for x in g:
        assert x.intact(), kernel
    assert lib().acro_b200_device_status() == 0
    g[0].tensor.MoveFromGPU()
    plain = kernel.replace("+=", "=")
    prod, mags = np.zeros_like(start), np.zeros_like(start)
    oracle.contract("port", plain, prod, *host[1:])
    oracle.contract("port", plain, mags, *[np.abs(h) for h in host[1:]])
    ref = start + prod if "+=" in kernel else prod
    assert oracle.parity_error(host[0], ref, mags + (np.abs(start) if "+=" in kernel else 0)) <= 1e-12
