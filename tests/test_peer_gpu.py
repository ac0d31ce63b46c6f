"""The reduction fused with the all-reduce over a peer group (mailboxes in peer GPU memory).
World size 1 runs on any GPU; the two-rank test needs two GPUs and is skipped otherwise."""
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
    te("S_i_j = A_n_i_j B_n", S, ab.Tensor(50000, 3, 3, hdata=a.reshape(50000, 3, 3)), ab.Tensor(50000, hdata=w))
    S.MoveFromGPU()
    assert np.array_equal(s.reshape(-1), plain.cpu().numpy())
    assert lib().acro_b200_reduce_batch_allreduce(p(da), p(dw), p(plain), 50000, 9, 0, p(scratch), nbytes, None, None) == _lib.EINVAL


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
        A = ab.Tensor(b1 - b0, 3, 3, hdata=np.ascontiguousarray(a[b0:b1]))
        W = ab.Tensor(b1 - b0, hdata=np.ascontiguousarray(w[b0:b1]))
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
