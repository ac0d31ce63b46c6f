"""GPU parity of the fp64 tensor-core and fused-chain kernel families (rank1_gemm,
batched_gemm, sumfact_mass), through the kernel layer of the C ABI and through the engine.
These families reorder sums and use fused multiply-add / DMMA, so the gate is
|gpu - ref| <= 1e-12 * sum|terms| (the fp64 tolerance of the benchmark definition)."""
import ctypes

import numpy as np
import pytest

import acrotensor_b200 as ab
import gpu_util as gu
from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib
from acrotensor_b200.runner import Session, alloc_host
from acrotensor_b200.workloads import BY_KEY, MASS_CHAIN
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-12


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def to_dev(torch, arr, offset=0):
    """Device copy of arr; offset=1 puts it on an 8-byte (not 16-byte) boundary."""
    flat = torch.zeros(arr.size + offset, dtype=torch.float64, device="cuda")
    flat[offset:] = torch.from_numpy(np.ascontiguousarray(arr).reshape(-1)).cuda()
    return flat, ctypes.c_void_p(flat.data_ptr() + 8 * offset)


def status_ok():
    assert lib().acro_b200_device_status() == _lib.OK


@pytest.mark.parametrize("elements,ni,nj,op,offset,q", [
    (32, 27, 27, 0, 0, 64), (33, 27, 27, 0, 0, 64), (1, 27, 27, 0, 0, 64), (100, 27, 27, 1, 0, 64), (257, 27, 27, 2, 0, 64),
    (64, 5, 7, 0, 0, 64), (95, 32, 32, 0, 0, 64), (70, 27, 27, 0, 1, 64), (10000, 27, 27, 0, 0, 64), (40, 27, 27, 0, 2, 64),
    (75, 1, 1, 0, 0, 64), (50, 2, 2, 1, 0, 64), (64, 27, 27, 0, 0, 8), (100, 5, 7, 0, 0, 36), (33, 10, 10, 2, 0, 4),
    # contracted extents that are not multiples of four (zero-padded on chip); odd ones cannot travel as bulk copies
    (3000, 27, 27, 0, 0, 27), (77, 27, 27, 0, 2, 27), (100, 8, 8, 0, 0, 10), (41, 8, 9, 1, 1, 63), (65, 3, 3, 0, 0, 1), (90, 32, 32, 2, 0, 5),
])
def test_rank1_gemm_kernel(torch, elements, ni, nj, op, offset, q):
    rng = np.random.default_rng(elements + ni)
    w = rng.random((elements, q)) + 0.5
    b1 = rng.random((q, ni)) * 2 - 1
    # the same matrix twice selects the symmetric path; offset == 2 forces two distinct square matrices
    b2 = b1 if (ni == nj and offset != 2) else rng.random((q, nj)) * 2 - 1
    offset = offset % 2
    m0 = rng.random((elements, ni, nj))
    prod, mags = np.zeros_like(m0), np.zeros_like(m0)
    oracle.contract("port", "M_e_i_j = W_e_q B_q_i C_q_j", prod, w, b1, b2)
    oracle.contract("port", "M_e_i_j = W_e_q B_q_i C_q_j", mags, w, np.abs(b1), np.abs(b2))
    expect = [prod, m0 + prod, m0 - prod][op]
    keep_w, pw = to_dev(torch, w, offset)
    keep_1, p1 = to_dev(torch, b1)
    keep_2, p2 = (keep_1, p1) if b2 is b1 else to_dev(torch, b2)
    keep_m, pm = to_dev(torch, m0)
    assert lib().acro_b200_rank1_gemm_supported(q, ni, nj) == 1 and lib().acro_b200_rank1_gemm_supported(65, ni, nj) == 0
    check(lib().acro_b200_rank1_gemm(pw, p1, p2, pm, elements, q, ni, nj, op, None))
    status_ok()
    got = keep_m.cpu().numpy().reshape(m0.shape)
    assert oracle.parity_error(got, expect, mags + np.abs(m0)) <= TOL


@pytest.mark.parametrize("batch,op,offset,n", [(1, 0, 0, 64), (2, 1, 0, 64), (5, 2, 0, 64), (3, 0, 1, 64), (500, 0, 0, 64),
                                                 (1, 0, 0, 32), (7, 1, 1, 32), (3000, 0, 0, 32)])
def test_batched_gemm_kernel(torch, batch, op, offset, n):
    rng = np.random.default_rng(batch)
    a, b = rng.standard_normal((batch, n, n)), rng.standard_normal((batch, n, n))
    c0 = rng.random((batch, n, n))
    ka, pa = to_dev(torch, a, offset)
    kb, pb = to_dev(torch, b)
    kc, pc = to_dev(torch, c0)
    assert lib().acro_b200_batched_gemm_supported(n, n, n) == 1 and lib().acro_b200_batched_gemm_supported(n, n, 4097) == 0
    check(lib().acro_b200_batched_gemm(pa, pb, pc, batch, n, n, n, op, None))
    status_ok()
    got = kc.cpu().numpy().reshape(c0.shape)
    sample = sorted(set([0, batch // 2, batch - 1]))         # the oracle needs 262144 terms per matrix
    prod = np.zeros((len(sample), n, n))
    mags = np.zeros_like(prod)
    oracle.contract("port", "C_e_i_j = A_e_i_k B_e_k_j", prod, a[sample], b[sample])
    oracle.contract("port", "C_e_i_j = A_e_i_k B_e_k_j", mags, np.abs(a[sample]), np.abs(b[sample]))
    expect = [prod, c0[sample] + prod, c0[sample] - prod][op]
    assert oracle.parity_error(got[sample], expect, mags + np.abs(c0[sample])) <= TOL
    # every matrix against a float64 matmul (looser: numpy's own summation order differs too)
    ref = np.matmul(a, b)
    full = [ref, c0 + ref, c0 - ref][op]
    assert np.max(np.abs(got - full)) <= 1e-11


@pytest.mark.parametrize("batch,m,n,k,op,offset", [
    (1, 3, 3, 3, 0, 0), (1000, 3, 3, 3, 0, 0), (100001, 3, 3, 3, 0, 0), (4097, 4, 4, 4, 1, 0), (513, 8, 8, 8, 2, 0), (2050, 16, 16, 16, 0, 0),
    (777, 16, 16, 16, 1, 1), (300, 5, 7, 3, 0, 0), (301, 1, 1, 1, 0, 0), (64, 2, 16, 9, 2, 1), (9000, 16, 1, 16, 0, 0), (2500, 12, 12, 12, 1, 0),
    (33, 16, 15, 16, 0, 1)])
def test_small_batched_gemm_kernel_is_bit_identical(torch, batch, m, n, k, op, offset):
    """Matrices up to 16 x 16 x 16: the streaming variant, same operation order as the reference's CPU executor."""
    rng = np.random.default_rng(batch + m)
    a, b = rng.standard_normal((batch, m, k)), rng.standard_normal((batch, k, n))
    c0 = rng.random((batch, m, n))
    ka, pa = to_dev(torch, a, offset)
    kb, pb = to_dev(torch, b)
    kc, pc = to_dev(torch, c0, offset)
    assert lib().acro_b200_batched_gemm_supported(m, n, k) == 1 and lib().acro_b200_batched_gemm_supported(m, 0, k) == 0
    check(lib().acro_b200_batched_gemm(pa, pb, pc, batch, m, n, k, op, None))
    status_ok()
    got = kc[offset:].cpu().numpy().reshape(c0.shape)
    if op == 2:
        prod = np.zeros_like(c0)
        oracle.contract("port", "C_e_i_j = A_e_i_k B_e_k_j", prod, a, b)
        expect = c0 - prod
    else:
        expect = c0.copy()
        oracle.contract("port", "C_e_i_j %s A_e_i_k B_e_k_j" % ["=", "+="][op], expect, a, b)
    if m == 1 or n == 1:
        # one row or one column: the matrix-vector kernel, which sums in a rotated order with fused multiply-add
        mags = np.zeros_like(c0)
        oracle.contract("port", "C_e_i_j = A_e_i_k B_e_k_j", mags, np.abs(a), np.abs(b))
        assert oracle.parity_error(got, expect, mags + np.abs(c0)) <= TOL
    else:
        assert np.array_equal(got, expect)


@pytest.mark.parametrize("batch,m,n,k,op,offset", [
    (1, 27, 27, 27, 0, 0), (500, 27, 27, 27, 0, 0), (301, 27, 27, 27, 1, 1), (64, 20, 33, 17, 0, 0), (40, 64, 64, 48, 2, 0), (90, 17, 64, 5, 0, 0),
    (75, 33, 1, 64, 0, 1), (130, 48, 48, 48, 1, 0), (55, 18, 24, 30, 0, 0), (33, 32, 32, 31, 0, 0), (20, 63, 63, 63, 0, 1),
    # rows of an odd length, 17 .. 32: pairs of elements by bulk copy (an odd last element goes through the padded ring)
    (2, 27, 27, 27, 0, 0), (3, 27, 27, 27, 0, 0), (1301, 27, 27, 27, 2, 0), (640, 17, 19, 21, 0, 0), (77, 31, 29, 23, 1, 0), (250, 9, 25, 31, 0, 0),
    (300, 32, 27, 27, 0, 0), (123, 20, 31, 5, 2, 0),
    # above 64: tiles of every product through the GEMM kernel (odd sizes: shifted rows, 8-byte copies, ragged tiles)
    (7, 125, 125, 125, 0, 0), (5, 125, 125, 125, 1, 1), (3, 65, 200, 33, 2, 0), (4, 128, 64, 96, 0, 0), (9, 100, 3, 129, 0, 0),
    # matrix-vector forms on operands that are not 16-byte aligned (8-byte copies), ragged last tile
    (501, 27, 1, 27, 0, 1), (333, 1, 40, 33, 1, 1), (1000, 64, 1, 64, 2, 1)])
def test_padded_batched_gemm_kernel(torch, batch, m, n, k, op, offset):
    """Sizes between 17 and 64 that do not fill the 32- or 64-wide slots: zero-padded on chip, fp64 tensor cores."""
    rng = np.random.default_rng(batch + m + k)
    a, b = rng.standard_normal((batch, m, k)), rng.standard_normal((batch, k, n))
    c0 = rng.random((batch, m, n))
    ka, pa = to_dev(torch, a, offset)
    kb, pb = to_dev(torch, b)
    kc, pc = to_dev(torch, c0, offset)
    assert lib().acro_b200_batched_gemm_supported(m, n, k) == 1
    check(lib().acro_b200_batched_gemm(pa, pb, pc, batch, m, n, k, op, None))
    status_ok()
    got = kc[offset:].cpu().numpy().reshape(c0.shape)
    prod, mags = np.zeros_like(c0), np.zeros_like(c0)
    oracle.contract("port", "C_e_i_j = A_e_i_k B_e_k_j", prod, a, b)
    oracle.contract("port", "C_e_i_j = A_e_i_k B_e_k_j", mags, np.abs(a), np.abs(b))
    expect = [prod, c0 + prod, c0 - prod][op]
    assert oracle.parity_error(got, expect, mags + np.abs(c0)) <= TOL


def run_chain_oracle(b, u, w):
    e, p, q = u.shape[0], u.shape[1], w.shape[1]
    t = {"B": b, "U": u, "W": w, "T1": np.zeros((e, p, p, q)), "T2": np.zeros((e, p, q, q)), "X": np.zeros((e, q, q, q)),
         "Y1": np.zeros((e, p, q, q)), "Y2": np.zeros((e, p, p, q)), "V": np.zeros((e, p, p, p))}
    names = sorted(t)
    prog = [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in MASS_CHAIN]
    oracle.run("port", [t[n] for n in names], prog, multi=True)
    return t["V"]


@pytest.mark.parametrize("elements,offset,p,q", [(1, 0, 4, 5), (31, 0, 4, 5), (32, 0, 4, 5), (33, 0, 4, 5), (1000, 0, 4, 5), (65, 1, 4, 5),
                                                  (10007, 0, 4, 5), (1, 0, 3, 4), (100, 0, 3, 4), (5001, 1, 3, 4), (33, 0, 2, 3),
                                                  (20000, 0, 2, 3), (77, 1, 2, 3), (3001, 0, 2, 4), (95, 1, 2, 4), (2049, 0, 3, 5),
                                                  (64, 1, 3, 5), (1500, 0, 4, 6), (33, 1, 4, 6), (999, 0, 5, 6), (32, 1, 5, 6)])
def test_sumfact_mass_kernel(torch, elements, offset, p, q):
    rng = np.random.default_rng(elements)
    b = rng.random((q, p)) * 2 - 1
    u = rng.random((elements, p, p, p)) * 2 - 1
    w = rng.random((elements, q, q, q)) + 0.5
    ref = run_chain_oracle(b, u, w)
    mags = run_chain_oracle(np.abs(b), np.abs(u), w)
    kb, pb = to_dev(torch, b)
    ku, pu = to_dev(torch, u, offset)
    kw, pw = to_dev(torch, w)
    kv, pv = to_dev(torch, np.full(ref.shape, -1.0))
    assert lib().acro_b200_sumfact_mass_supported(p, q) == 1 and lib().acro_b200_sumfact_mass_supported(6, 7) == 0
    check(lib().acro_b200_sumfact_mass(pb, pu, pw, pv, elements, p, q, None))
    status_ok()
    got = kv.cpu().numpy().reshape(ref.shape)
    assert oracle.parity_error(got, ref, mags) <= TOL


def test_chain_through_the_engine_fused_and_unfused():
    w = BY_KEY["cfg2"]
    batch = 700
    host_f = alloc_host(w, batch, w.make_inputs(batch, seed=3))
    host_u = {k: v.copy() for k, v in host_f.items()}
    fused = Session(w, host_f, transient=True)
    assert "family=sumfact_mass" in fused.plan_text()
    fused.run(); fused.fetch()
    unfused = Session(w, host_u, transient=False)           # reference semantics: everything materialised
    unfused.run(); unfused.fetch(w.names("out") + w.names("tmp"))
    ref = run_chain_oracle(host_u["B"], host_u["U"], host_u["W"])
    mags = run_chain_oracle(np.abs(host_u["B"]), np.abs(host_u["U"]), host_u["W"])
    assert np.array_equal(host_u["V"], ref)                  # generic kernels: bit-identical, stage by stage
    assert np.any(host_u["T1"] != 0) and np.all(host_f["T1"] == 0)   # transient intermediates never materialised
    assert oracle.parity_error(host_f["V"], ref, mags) <= TOL
    assert lib().acro_b200_device_status() == _lib.OK


def test_benchmark_families_through_the_engine():
    for key, batch, family in (("cfg1", 200, "rank1_gemm"), ("cfg4", 4, "batched_gemm")):
        w = BY_KEY[key]
        host = alloc_host(w, batch, w.make_inputs(batch, seed=5))
        sess = Session(w, host)
        assert "family=" + family in sess.plan_text()
        sess.run(); sess.fetch()
        names = sorted(host)
        out = w.names("out")[0]
        got = host[out].copy()
        prog = [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in w.program]
        mags = [np.abs(host[n]) for n in names]
        oracle.run("port", [host[n] for n in names], prog)
        oracle.run("port", mags, prog)
        assert oracle.parity_error(got, host[out], mags[names.index(out)]) <= TOL
    assert lib().acro_b200_device_status() == _lib.OK


def test_full_size_tensor_core_properties(torch):
    # cfg 4 at E = 2^14: B_e = identity gives C_e = A_e exactly (products by 1, sums with 0)
    E = 1 << 14
    a = torch.randn(E, 64, 64, dtype=torch.float64, device="cuda")
    b = torch.eye(64, dtype=torch.float64, device="cuda").repeat(E, 1, 1)
    c = torch.empty_like(a)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    check(lib().acro_b200_batched_gemm(p(a), p(b), p(c), E, 64, 64, 64, 0, None))
    assert bool((c == a).all())
    check(lib().acro_b200_batched_gemm(p(b), p(a), p(c), E, 64, 64, 64, 0, None))
    assert bool((c == a).all())
    del a, b, c
    # cfg 1 at E = 2^18: W = 1 makes every element matrix the same Gram matrix; W = 2^k scales exactly
    E = 1 << 18
    rng = np.random.default_rng(1)
    bm = rng.random((64, 27)) * 2 - 1
    db = torch.from_numpy(bm).cuda()
    w = torch.ones(E, 64, dtype=torch.float64, device="cuda")
    w[1::2] = 4.0
    m = torch.empty(E, 27, 27, dtype=torch.float64, device="cuda")
    check(lib().acro_b200_rank1_gemm(p(w), p(db), p(db), p(m), E, 64, 27, 27, 0, None))
    assert bool((m[0::2] == m[0]).all()) and bool((m[1::2] == 4.0 * m[0]).all())
    ref, mags = np.zeros((1, 27, 27)), np.zeros((1, 27, 27))
    oracle.contract("port", "M_e_i_j = W_e_q B_q_i B_q_j", ref, np.ones((1, 64)), bm, bm)
    oracle.contract("port", "M_e_i_j = W_e_q B_q_i B_q_j", mags, np.ones((1, 64)), np.abs(bm), np.abs(bm))
    assert oracle.parity_error(m[0:1].cpu().numpy(), ref, mags) <= TOL
    del w, m
    # cfg 2 at E = 2^20: scaling U by 2 scales V by 2 exactly; a seeded sample matches the oracle
    E = 1 << 20
    gen = torch.Generator(device="cuda"); gen.manual_seed(9)
    bq = torch.rand(5, 4, generator=gen, device="cuda", dtype=torch.float64) * 2 - 1
    u = torch.rand(E, 4, 4, 4, generator=gen, device="cuda", dtype=torch.float64) * 2 - 1
    wq = torch.rand(E, 5, 5, 5, generator=gen, device="cuda", dtype=torch.float64) + 0.5
    v1, v2 = torch.empty_like(u), torch.empty_like(u)
    check(lib().acro_b200_sumfact_mass(p(bq), p(u), p(wq), p(v1), E, 4, 5, None))
    u.mul_(2.0)
    check(lib().acro_b200_sumfact_mass(p(bq), p(u), p(wq), p(v2), E, 4, 5, None))
    assert bool((v2 == 2.0 * v1).all())
    take = [0, 1, 31, 32, E // 2 + 7, E - 33, E - 1]
    ref = run_chain_oracle(bq.cpu().numpy(), u[take].cpu().numpy(), wq[take].cpu().numpy())
    mags = run_chain_oracle(bq.abs().cpu().numpy(), u[take].abs().cpu().numpy(), wq[take].cpu().numpy())
    assert oracle.parity_error(v2[take].cpu().numpy(), ref, mags) <= TOL
    assert lib().acro_b200_device_status() == _lib.OK
