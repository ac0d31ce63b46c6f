"""Host logic of the shared-entry exchange (a sharded FlatIndexedSumGather): the plan every rank
derives from the touched-entry bitmaps, checked without a GPU by emulating the inboxes in numpy,
in one process and as gloo ranks that really exchange the bitmaps."""
import ctypes
import os
import socket

import numpy as np
import pytest

import acrotensor_b200 as ab
import shared_entries as se
from acrotensor_b200._lib import check, lib


def bitmap_of(mapping, domain):
    b = ctypes.create_string_buffer((domain + 7) // 8)
    m = np.ascontiguousarray(mapping, dtype=np.int32)
    check(lib().acro_b200_halo_mark_touched(m.ctypes.data_as(ctypes.c_void_p), m.size, domain, b))
    return b.raw


def test_mark_touched_sets_exactly_the_reached_bits_and_rejects_bad_values():
    m = np.array([3, 3, 0, 17, 9], dtype=np.int32)
    bits = np.unpackbits(np.frombuffer(bitmap_of(m, 18), dtype=np.uint8), bitorder="little")[:18]
    assert np.flatnonzero(bits).tolist() == [0, 3, 9, 17]
    b = ctypes.create_string_buffer(3)
    bad = np.array([18], dtype=np.int32)
    assert lib().acro_b200_halo_mark_touched(bad.ctypes.data_as(ctypes.c_void_p), 1, 18, b) != 0


@pytest.mark.parametrize("world,elements,per_element,stray", [(1, 10, 4, 0.0), (2, 40, 4, 0.0), (3, 50, 5, 0.05), (8, 64, 3, 0.1),
                                                              (4, 9, 2, 0.5)])
def test_plan_sums_shared_entries_over_the_ranks(world, elements, per_element, stray):
    mapping, domain = se.mesh_mapping(elements, per_element, seed=world * 100 + elements, stray=stray)
    cuts = se.slabs(elements, per_element, world)
    rng = np.random.default_rng(5)
    values = rng.random(mapping.size) * 2 - 1
    local_maps = [mapping[a:b] for a, b in cuts]
    bitmaps = [bitmap_of(m, domain) for m in local_maps]
    plans, strides, partials = [], [], []
    for r in range(world):
        M = ab.IndexMapping(domain, local_maps[r].size, local_maps[r])
        x = ab.SharedEntryExchange(M, world, r, (lambda b: bitmaps) if world > 1 else None, on_device=False)
        ns, ne, stride = x.counts()
        plans.append(x.plan())
        strides.append(stride)
        partials.append(se.local_sum_gather(values[cuts[r][0]:cuts[r][1]], local_maps[r], domain))
        # the plan lists exactly the entries this rank reaches that another rank reaches too, ascending
        touched = [np.unpackbits(np.frombuffer(b, dtype=np.uint8), bitorder="little")[:domain] for b in bitmaps]
        others = np.sum([touched[p] for p in range(world) if p != r], axis=0) if world > 1 else np.zeros(domain)
        assert plans[r][0].tolist() == np.flatnonzero((touched[r] > 0) & (others > 0)).tolist()
        assert ne == int(sum(((touched[r] > 0) & (touched[p] > 0)).sum() for p in range(world) if p != r))
    got = se.emulate_exchange(plans, partials, strides)
    for r in range(world):
        reached = np.zeros(domain, dtype=bool)
        reached[local_maps[r]] = True
        # a rank-ordered sum of the partials, exactly what the kernels compute
        want = np.zeros(domain)
        for p in range(world):
            touched_p = np.zeros(domain, dtype=bool)
            touched_p[local_maps[p]] = True
            want = np.where(touched_p, want + partials[p], want)
        assert np.array_equal(got[r][reached], want[reached])
        assert np.array_equal(got[r][~reached], np.zeros(int((~reached).sum())))
        # and, to rounding, the single-rank sum-gather
        full = se.local_sum_gather(values, mapping, domain)
        assert np.allclose(got[r][reached], full[reached], rtol=0, atol=1e-13)


def test_an_exchange_made_as_a_plan_refuses_device_calls():
    mapping, domain = se.mesh_mapping(6, 3, seed=1, stray=0.0)
    M = ab.IndexMapping(domain, mapping.size, mapping)
    x = ab.SharedEntryExchange(M, 1, 0, on_device=False)
    assert x.counts()[0] == 0 and x.inbox() is None
    with pytest.raises(ab.AcroError):
        x.exchange_sum(4096)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_rank(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mapping, domain = se.mesh_mapping(31, 4, seed=9, stray=0.03)       # every rank regenerates the global map
        a, b = se.slabs(31, 4, world)[rank]
        values = np.random.default_rng(2).random(mapping.size)
        M = ab.IndexMapping(domain, b - a, mapping[a:b])

        def exchange(mine):
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
            return everyone

        x = ab.SharedEntryExchange(M, world, rank, exchange, on_device=False)
        partial = se.local_sum_gather(values[a:b], mapping[a:b], domain)
        everything = [None] * world
        dist.all_gather_object(everything, (x.plan(), x.counts()[2], partial))
        got = se.emulate_exchange([e[0] for e in everything], [e[2] for e in everything], [e[1] for e in everything])
        np.save(os.path.join(out_dir, "r%d.npy" % rank), got[rank])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_ranks_agree_on_the_plan(tmp_path, world):
    import torch.multiprocessing as mp
    mp.spawn(_gloo_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    mapping, domain = se.mesh_mapping(31, 4, seed=9, stray=0.03)
    values = np.random.default_rng(2).random(mapping.size)
    full = se.local_sum_gather(values, mapping, domain)
    results = [np.load(os.path.join(str(tmp_path), "r%d.npy" % r)) for r in range(world)]
    for r, (a, b) in enumerate(se.slabs(31, 4, world)):
        reached = np.zeros(domain, dtype=bool)
        reached[mapping[a:b]] = True
        assert np.allclose(results[r][reached], full[reached], rtol=0, atol=1e-13)
        for p in range(r):          # ranks sharing an entry hold identical bits
            both = reached & (results[p] != 0) & np.isin(np.arange(domain), mapping[slice(*se.slabs(31, 4, world)[p])])
            assert np.array_equal(results[r][both], results[p][both])
