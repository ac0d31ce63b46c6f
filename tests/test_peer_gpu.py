"""Sums over the ranks of a peer group (mailboxes in peer GPU memory): fused into the reduction kernel,
and as the all-reduce kernel that follows every other kernel family.  World size 1 runs on any GPU;
the two-rank tests need two GPUs and are skipped otherwise."""
import ctypes
import os
import socket

import numpy as np
import pytest

import acrotensor_b200 as ab
from acrotensor_b200 import _lib
from acrotensor_b200._lib import check, lib
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-12


def test_single_rank_group_gives_the_plain_result_and_survives_many_calls():
    import torch
    rng = np.random.default_rng(3)
    a, w = rng.random((50000, 9)) * 2 - 1, rng.random(50000) + 0.5
    da, dw = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    group = ab.PeerGroup(1, 0)
    nbytes = lib().acro_b200_reduce_batch_scratch_bytes(9)
    scratch = torch.empty(nbytes // 8 + 1, dtype=torch.float64, device="cuda")
    plain = torch.zeros(9, dtype=torch.float64, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    check(lib().acro_b200_reduce_batch(p(da), p(dw), p(plain), 50000, 9, 0, p(scratch), nbytes, None))
    for call in range(5):           # both mailbox parities, several sequence numbers
        fused = torch.full((9,), -1.0, dtype=torch.float64, device="cuda")
        check(lib().acro_b200_reduce_batch_allreduce(p(da), p(dw), p(fused), 50000, 9, 0, p(scratch), nbytes, group._h, None))
        assert torch.equal(fused, plain)
    assert lib().acro_b200_device_status() == _lib.OK
    # through the engine
    s = np.zeros((3, 3))
    te = ab.TensorEngine("Cuda")
    te.SetPeerGroup(group)
    S = ab.Tensor(3, 3, hdata=s)
    A, W = ab.Tensor(50000, 3, 3, hdata=a.reshape(50000, 3, 3)), ab.Tensor(50000, hdata=w)
    A.SetSharded(True)
    W.SetSharded(True)
    te("S_i_j = A_n_i_j B_n", S, A, W)
    S.MoveFromGPU()
    assert np.array_equal(s.reshape(-1), plain.cpu().numpy())
    assert lib().acro_b200_reduce_batch_allreduce(p(da), p(dw), p(plain), 50000, 9, 0, p(scratch), nbytes, None, None) == _lib.EINVAL


def test_single_rank_allreduce_kernel_and_engine_rule():
    """World size 1: the all-reduce kernel is the identity (every exchange length, every operator, in place), and
    the engine applies it exactly when an input whose leading index is contracted is flagged as a slab."""
    import torch
    group = ab.PeerGroup(1, 0)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    for n in (1, 9, 4095, 4096, 4097, 10000):
        src = torch.rand(n, generator=gen, device="cuda", dtype=torch.float64) - 0.5
        for op, expect in ((_lib.OP_ASSIGN, lambda old: src), (_lib.OP_ADD, lambda old: old + src), (_lib.OP_SUB, lambda old: old - src)):
            old = torch.rand(n, generator=gen, device="cuda", dtype=torch.float64)
            dst = old.clone()
            check(lib().acro_b200_peer_allreduce(p(dst), p(src), n, op, group._h, None))
            assert torch.equal(dst, expect(old)), (n, op)
        inplace = src.clone()
        check(lib().acro_b200_peer_allreduce(p(inplace), p(inplace), n, _lib.OP_ASSIGN, group._h, None))
        assert torch.equal(inplace, src)
    assert lib().acro_b200_device_status() == _lib.OK
    assert lib().acro_b200_peer_allreduce(p(src), p(src), 0, 0, group._h, None) == _lib.EINVAL
    assert lib().acro_b200_peer_allreduce(p(src), p(src), 4, 0, None, None) == _lib.EINVAL

    # engine: Gram form (its own family), with and without the flag, "=" and "+="
    rng = np.random.default_rng(8)
    x, y = rng.random((20000, 27)) - 0.5, rng.random((20000, 27)) - 0.5
    plain, flagged, added = np.zeros((27, 27)), np.zeros((27, 27)), np.ones((27, 27))
    te = ab.TensorEngine("Cuda")
    X, Y = ab.Tensor(x.shape, hdata=x), ab.Tensor(y.shape, hdata=y)
    P = ab.Tensor(27, 27, hdata=plain)
    te("S_a_b = X_n_a Y_n_b", P, X, Y)
    P.MoveFromGPU()
    te.SetPeerGroup(group)
    X.SetSharded(True)
    F, Acc = ab.Tensor(27, 27, hdata=flagged), ab.Tensor(27, 27, hdata=added)
    te("S_a_b = X_n_a Y_n_b", F, X, Y)
    te("S_a_b += X_n_a Y_n_b", Acc, X, Y)
    F.MoveFromGPU()
    Acc.MoveFromGPU()
    assert "family=gram" in te.GetImplementation("S_a_b = X_n_a Y_n_b", F, X, Y)
    assert np.array_equal(flagged, plain) and np.array_equal(added, 1.0 + plain)
    assert lib().acro_b200_device_status() == _lib.OK


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, n, out_dir):
    import torch
    import torch.distributed as dist
    from acrotensor_b200.runner import make_peer_group, slab
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # only carries the IPC handles
    try:
        rng = np.random.default_rng(17)
        a, w = rng.random((n, 3, 3)) * 2 - 1, rng.random(n) + 0.5     # every rank regenerates the global input
        b0, b1 = slab(n, rank, world)
        group = make_peer_group()
        te = ab.TensorEngine("Cuda")
        te.SetPeerGroup(group)
        A = ab.SlabTensor(ab.Tensor(a.shape, hdata=a), b0, b1)       # rows b0..b1 of the global tensor: flagged sharded
        W = ab.Tensor(b1 - b0, hdata=np.ascontiguousarray(w[b0:b1]))  # a per-rank tensor, flagged by hand
        W.SetSharded(True)
        results = []
        for call in range(4):
            s = np.zeros((3, 3))
            S = ab.Tensor(3, 3, hdata=s)
            te("S_i_j = A_n_i_j B_n", S, A, W)
            S.MoveFromGPU()
            results.append(s)
        status = lib().acro_b200_device_status()
        np.save(os.path.join(out_dir, "r%d.npy" % rank), np.stack(results + [np.full((3, 3), float(status))]))
        dist.barrier()       # nobody leaves while a peer may still read its mailbox
    finally:
        dist.destroy_process_group()


def test_two_ranks_on_two_gpus(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n, world = 300001, 2
    mp.spawn(_rank_main, args=(world, _free_port(), n, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(17)
    a, w = rng.random((n, 3, 3)) * 2 - 1, rng.random(n) + 0.5
    ref, mags = np.zeros((3, 3)), np.zeros((3, 3))
    oracle.contract("port", "S_i_j = A_n_i_j B_n", ref, a, w)
    oracle.contract("port", "S_i_j = A_n_i_j B_n", mags, np.abs(a), w)
    r0, r1 = (np.load(os.path.join(str(tmp_path), "r%d.npy" % r)) for r in range(world))
    assert r0[-1, 0, 0] == 0.0 and r1[-1, 0, 0] == 0.0           # no bounded wait gave up
    assert np.array_equal(r0[:-1], r1[:-1])                       # every rank holds the same bits
    for call in range(4):
        assert oracle.parity_error(r0[call], ref, mags) <= TOL


def _rank_absent_peer(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from acrotensor_b200.runner import make_peer_group
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        group = make_peer_group()
        outcome = []
        if rank == 0:
            # rank 1 never makes the matching call: the bounded wait must run out, report
            # ETIMEOUT to the host and leave the context usable
            a = torch.ones(4096, 9, dtype=torch.float64, device="cuda")
            out = torch.zeros(9, dtype=torch.float64, device="cuda")
            nbytes = lib().acro_b200_reduce_batch_scratch_bytes(9)
            scratch = torch.empty(nbytes // 8 + 1, dtype=torch.float64, device="cuda")
            p = lambda t: ctypes.c_void_p(t.data_ptr())
            check(lib().acro_b200_reduce_batch_allreduce(p(a), None, p(out), 4096, 9, 0, p(scratch), nbytes, group._h, None))
            outcome.append(lib().acro_b200_device_status())
            outcome.append(lib().acro_b200_device_status())          # the flag is cleared by the first read
            check(lib().acro_b200_reduce_batch(p(a), None, p(out), 4096, 9, 0, p(scratch), nbytes, None))
            outcome.append(float(out[0].item()))
            np.save(os.path.join(out_dir, "timeout.npy"), np.array(outcome, dtype=np.float64))
        dist.barrier()       # rank 1 keeps its mailbox alive until rank 0 is done
    finally:
        dist.destroy_process_group()


def test_absent_peer_times_out_instead_of_hanging(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_rank_absent_peer, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    first, second, plain = np.load(os.path.join(str(tmp_path), "timeout.npy"))
    assert int(first) == _lib.ETIMEOUT and int(second) == _lib.OK and plain == 4096.0


FAMILY_CASES = [
    # name, string, shapes of (out, in...) with None for the sharded extent, operator applied to an output of ones?
    ("reduction, short slab on rank 0", "S_i_j = A_n_i_j B_n", [(3, 3), (None, 3, 3), (None,)], False),
    ("gram 27x27", "S_a_b = X_n_a Y_n_b", [(27, 27), (None, 27), (None, 27)], False),
    ("gram 27x27 accumulated", "S_a_b += X_n_a Y_n_b", [(27, 27), (None, 27), (None, 27)], True),
    ("gram 8x8 subtracted", "S_a_b -= X_n_a Y_n_b", [(8, 8), (None, 8), (None, 8)], True),
    ("80x80 result in two exchanges", "S_a_b = X_n_a Y_n_b", [(80, 80), (None, 80), (None, 80)], False),
    ("column dot products", "S_a = X_n_a Y_n_a", [(5,), (None, 5), (None, 5)], False),
]


def _family_inputs(n):
    rng = np.random.default_rng(23)
    data = []
    for name, kernel, shapes, accumulate in FAMILY_CASES:
        data.append([rng.random(tuple(n if d is None else d for d in shape)) - 0.5 for shape in shapes[1:]])
    return data


def _rank_families(rank, world, port, n, cut, out_dir):
    import torch
    import torch.distributed as dist
    from acrotensor_b200.runner import make_peer_group
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b0, b1 = (0, cut) if rank == 0 else (cut, n)             # unequal slabs: rank 0 holds only `cut` rows
        group = make_peer_group()
        te = ab.TensorEngine("Cuda")
        te.SetPeerGroup(group)
        results, families = [], []
        for (name, kernel, shapes, accumulate), inputs in zip(FAMILY_CASES, _family_inputs(n)):
            parents = [ab.Tensor(x.shape, hdata=x) for x in inputs]
            slabs = [ab.SlabTensor(t, b0, b1) for t in parents]
            out = np.ones(shapes[0]) if accumulate else np.zeros(shapes[0])
            O = ab.Tensor(out.shape, hdata=out)
            te(kernel, O, *slabs)
            O.MoveFromGPU()
            results.append(out.reshape(-1).copy())
            families.append(te.GetImplementation(kernel, O, *slabs).split("family=")[1].split()[0])
        status = lib().acro_b200_device_status()
        np.save(os.path.join(out_dir, "f%d.npy" % rank), np.concatenate(results + [np.array([float(status)])]))
        with open(os.path.join(out_dir, "f%d.txt" % rank), "w") as f:
            f.write(" ".join(families))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_every_family_is_summed_over_two_ranks(tmp_path):
    """Strings that contract the sharded index, on whatever family each rank plans them (the ranks' slabs differ in
    length so much that they plan different families): every rank ends with the same bits, equal to the
    single-process result up to summation order."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n, cut, world = 120000, 100, 2
    mp.spawn(_rank_families, args=(world, _free_port(), n, cut, str(tmp_path)), nprocs=world, join=True)
    r0, r1 = (np.load(os.path.join(str(tmp_path), "f%d.npy" % r)) for r in range(world))
    fam0, fam1 = (open(os.path.join(str(tmp_path), "f%d.txt" % r)).read().split() for r in range(world))
    assert r0[-1] == 0.0 and r1[-1] == 0.0
    assert np.array_equal(r0, r1)
    assert fam0[0] == "generic" and fam1[0] == "reduce_batch" and fam1[1] == "gram"      # mixed families did meet in one exchange
    at = 0
    for (name, kernel, shapes, accumulate), inputs in zip(FAMILY_CASES, _family_inputs(n)):
        size = int(np.prod(shapes[0]))
        got = r0[at:at + size].reshape(shapes[0])
        at += size
        plain = kernel.replace("+=", "=").replace("-=", "=")
        ref, mags = np.zeros(shapes[0]), np.zeros(shapes[0])
        oracle.contract("port", plain, ref, *inputs)
        oracle.contract("port", plain, mags, *[np.abs(x) for x in inputs])
        if "+=" in kernel:
            ref = 1.0 + ref
        elif "-=" in kernel:
            ref = 1.0 - ref
        assert oracle.parity_error(got, ref, mags + 1.0) <= TOL, name


def _rank_late_peer(rank, world, port, out_dir):
    import time
    import torch
    import torch.distributed as dist
    from acrotensor_b200.runner import make_peer_group
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        group = make_peer_group()
        a = torch.ones(4096, 9, dtype=torch.float64, device="cuda")
        out = torch.zeros(9, dtype=torch.float64, device="cuda")
        nbytes = lib().acro_b200_reduce_batch_scratch_bytes(9)
        scratch = torch.empty(nbytes // 8 + 1, dtype=torch.float64, device="cuda")
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        dist.barrier()
        if rank == 1:
            time.sleep(4.0)          # longer than the bounded wait: rank 0 gives up on its first calls, host-side delay only
        record = []
        for call in range(12):
            t0 = time.perf_counter()
            check(lib().acro_b200_reduce_batch_allreduce(p(a), None, p(out), 4096, 9, 0, p(scratch), nbytes, group._h, None))
            status = lib().acro_b200_device_status()
            record.append([float(status), float(out[0].item()), time.perf_counter() - t0])
        np.save(os.path.join(out_dir, "late%d.npy" % rank), np.array(record))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_late_peer_times_out_then_the_exchange_recovers(tmp_path):
    """A rank whose host is several seconds late (no GPU is held up on purpose: the delay is a sleep on the host) makes its
    peer's bounded waits run out, which the peer sees as ETIMEOUT with the context intact; once the late rank has caught
    up the ranks meet again and later calls give the right sum on both, without any repair step."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_rank_late_peer, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    early, late = (np.load(os.path.join(str(tmp_path), "late%d.npy" % r)) for r in range(2))
    print("early rank: status, value, seconds per call:", early.tolist())
    assert int(early[0, 0]) == _lib.ETIMEOUT                      # the first wait of the early rank ran out ...
    assert 0.2 < early[0, 2] < 6.0                                  # ... after a bounded time
    assert np.all(late[:, 0] == _lib.OK)                          # the late rank finds every contribution already there
    assert int(early[-1, 0]) == _lib.OK and early[-1, 1] == 8192.0 and late[-1, 1] == 8192.0
    print("bounded wait took %.2f s; statuses of the early rank: %s" % (early[0, 2], early[:, 0].astype(int).tolist()))
    assert np.count_nonzero(early[:, 0]) < 12 and np.all(np.diff((early[:, 0] != 0).astype(int)) <= 0)      # give-ups first, then none
