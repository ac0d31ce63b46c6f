"""The shared-entry exchange on the GPU: a sharded FlatIndexedSumGather whose shared domain
entries are summed over the ranks through inboxes in peer GPU memory.  One GPU is enough for
the first tests (the ranks of one process share it; every send is launched before the first
combine, so no kernel waits for a later one); the last two need two GPUs and are skipped
otherwise."""
import ctypes
import os
import socket

import numpy as np
import pytest

import acrotensor_b200 as ab
import shared_entries as se
from acrotensor_b200 import _lib
from acrotensor_b200._lib import lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,elements,per_element,stray", [(2, 4000, 4, 0.0), (3, 3000, 5, 0.02), (8, 2048, 3, 0.05), (4, 9, 2, 0.5)])
def test_ranks_of_one_process_on_one_gpu(world, elements, per_element, stray):
    import torch
    mapping, domain = se.mesh_mapping(elements, per_element, seed=world + elements, stray=stray)
    cuts = se.slabs(elements, per_element, world)
    values = np.random.default_rng(8).random(mapping.size) * 2 - 1
    local_maps = [np.ascontiguousarray(mapping[a:b]) for a, b in cuts]
    bitmaps = []
    for m in local_maps:
        b = ctypes.create_string_buffer((domain + 7) // 8)
        _lib.check(lib().acro_b200_halo_mark_touched(m.ctypes.data_as(ctypes.c_void_p), m.size, domain, b))
        bitmaps.append(b.raw)
    maps = [ab.IndexMapping(domain, m.size, m) for m in local_maps]
    xs = [ab.SharedEntryExchange(maps[r], world, r, lambda b: bitmaps, on_device=True, connect=False) for r in range(world)]
    inboxes = [x.inbox() for x in xs]
    for x in xs:
        x.connect_pointers(inboxes)
    partials = [se.local_sum_gather(values[a:b], m, domain) for (a, b), m in zip(cuts, local_maps)]
    want = se.emulate_exchange([x.plan() for x in xs], partials, [x.counts()[2] for x in xs])
    for call in range(3):                      # both inbox halves, growing sequence numbers
        dev = [torch.from_numpy(p).cuda() for p in partials]
        for x, d in zip(xs, dev):
            x.send(d.data_ptr())
        for x, d in zip(xs, dev):
            x.combine(d.data_ptr())
        torch.cuda.synchronize()
        assert lib().acro_b200_device_status() == _lib.OK
        for r in range(world):
            assert np.array_equal(dev[r].cpu().numpy(), want[r]), (call, r)
    full = se.local_sum_gather(values, mapping, domain)
    for r, (a, b) in enumerate(cuts):
        reached = np.zeros(domain, dtype=bool)
        reached[mapping[a:b]] = True
        assert np.allclose(want[r][reached], full[reached], rtol=0, atol=1e-12)


def test_single_rank_through_the_engine_equals_the_plain_sum_gather():
    mapping, domain = se.mesh_mapping(500, 4, seed=3, stray=0.1)
    values = np.random.default_rng(4).random(mapping.size)
    M = ab.IndexMapping(domain, mapping.size, mapping)
    x = ab.SharedEntryExchange(M, 1, 0)
    te = ab.TensorEngine("Cuda")
    plain, shared = np.zeros(domain), np.zeros(domain)
    A = ab.Tensor(mapping.size, hdata=values)
    P, S = ab.Tensor(domain, hdata=plain), ab.Tensor(domain, hdata=shared)
    te.FlatIndexedSumGather(P, A, M)
    te.FlatIndexedSumGather(S, A, M, x)
    P.MoveFromGPU(); S.MoveFromGPU()
    assert np.array_equal(plain, shared) and np.array_equal(plain, se.local_sum_gather(values, mapping, domain))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


ELEMENTS, PER_ELEMENT = 20000, 8


def _rank_main(rank, world, port, out_dir, absent):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # carries the bitmaps and the IPC handles
    try:
        mapping, domain = se.mesh_mapping(ELEMENTS, PER_ELEMENT, seed=21, stray=0.01)
        a, b = se.slabs(ELEMENTS, PER_ELEMENT, world)[rank]
        values = np.random.default_rng(6).random(mapping.size) * 2 - 1

        def exchange(mine):
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
            return everyone

        M = ab.IndexMapping(domain, b - a, np.ascontiguousarray(mapping[a:b]))
        x = ab.SharedEntryExchange(M, world, rank, exchange)
        te = ab.TensorEngine("Cuda")
        A = ab.Tensor(b - a, hdata=np.ascontiguousarray(values[a:b]))
        results = []
        if not absent:
            for call in range(3):
                out = np.zeros(domain)
                Out = ab.Tensor(domain, hdata=out)
                te.FlatIndexedSumGather(Out, A, M, x)
                Out.MoveFromGPU()
                results.append(out)
            results.append(np.full(domain, float(lib().acro_b200_device_status())))
            np.save(os.path.join(out_dir, "r%d.npy" % rank), np.stack(results))
        elif rank == 0:
            # rank 1 never makes the matching call: the bounded wait must run out, report ETIMEOUT
            # to the host and leave the context usable
            out = np.zeros(domain)
            Out = ab.Tensor(domain, hdata=out)
            te.FlatIndexedSumGather(Out, A, M, x)
            Out.MoveFromGPU()
            first, second = lib().acro_b200_device_status(), lib().acro_b200_device_status()
            plain = np.zeros(domain)
            Plain = ab.Tensor(domain, hdata=plain)
            te.FlatIndexedSumGather(Plain, A, M)
            Plain.MoveFromGPU()
            ok = np.array_equal(plain, se.local_sum_gather(values[a:b], mapping[a:b], domain))
            np.save(os.path.join(out_dir, "timeout.npy"), np.array([first, second, float(ok)], dtype=np.float64))
        dist.barrier()       # nobody leaves while a peer may still write into or read its inbox
    finally:
        dist.destroy_process_group()


def test_two_ranks_on_two_gpus(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path), False), nprocs=world, join=True)
    mapping, domain = se.mesh_mapping(ELEMENTS, PER_ELEMENT, seed=21, stray=0.01)
    values = np.random.default_rng(6).random(mapping.size) * 2 - 1
    cuts = se.slabs(ELEMENTS, PER_ELEMENT, world)
    partials = [se.local_sum_gather(values[a:b], mapping[a:b], domain) for a, b in cuts]
    touched = []
    for a, b in cuts:
        t = np.zeros(domain, dtype=bool)
        t[mapping[a:b]] = True
        touched.append(t)
    results = [np.load(os.path.join(str(tmp_path), "r%d.npy" % r)) for r in range(world)]
    for r in range(world):
        assert results[r][-1][0] == 0.0                        # no bounded wait gave up
        want = partials[r].copy()
        both = touched[0] & touched[1]
        want[both] = (0.0 + partials[0][both]) + partials[1][both]     # ascending rank order
        for call in range(3):
            assert np.array_equal(results[r][call], want), (r, call)
    assert int((touched[0] & touched[1]).sum()) > 100


def test_absent_rank_times_out_instead_of_hanging(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_rank_main, args=(2, _free_port(), str(tmp_path), True), nprocs=2, join=True)
    first, second, plain_ok = np.load(os.path.join(str(tmp_path), "timeout.npy"))
    assert int(first) == _lib.ETIMEOUT and int(second) == _lib.OK and plain_ok == 1.0
