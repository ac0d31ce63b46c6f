"""Multi-rank host logic on CPU (gloo, world size 2 and 3): batch slabs, replicated
batch-invariant tensors and the one all-reduce of a contracted batch index.  No GPU is
involved, so the per-rank compute is done by the C restatement of the reference executor;
what is under test is the sharding arithmetic of acrotensor_b200.runner."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from acrotensor_b200.runner import allreduce_partial, alloc_host, slab
from acrotensor_b200.workloads import BY_KEY
from oracle import oracle


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def oracle_run(w, host):
    names = sorted(host)
    prog = [(k, names.index(o), [names.index(i) for i in ins]) for k, o, ins in w.program]
    oracle.run("port", [host[n] for n in names], prog, multi=w.multi)


def worker(rank, world, port, key, batch, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = BY_KEY[key]
        full = w.make_inputs(batch, seed=11)                 # every rank can regenerate the global inputs
        b0, b1 = slab(batch, rank, world)
        mine = {n: (np.ascontiguousarray(full[n][b0:b1]) if w.batched(n) else full[n]) for n in full}
        host = alloc_host(w, b1 - b0, mine)
        oracle_run(w, host)
        out = w.names("out")[0]
        if w.batch_contracted:
            t = torch.from_numpy(host[out])
            allreduce_partial(t)                              # in place, every rank gets the total
            np.save(os.path.join(out_dir, "r%d.npy" % rank), t.numpy())
        else:
            np.save(os.path.join(out_dir, "r%d.npy" % rank), host[out])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("key,batch,world", [("cfg0", 1001, 2), ("cfg0", 1000, 3), ("cfg3", 7, 2), ("cfg2", 9, 2), ("cfg1", 5, 3)])
def test_sharded_run_matches_single_rank(tmp_path, key, batch, world):
    w = BY_KEY[key]
    port = free_port()
    mp.spawn(worker, args=(world, port, key, batch, str(tmp_path)), nprocs=world, join=True)
    full = w.make_inputs(batch, seed=11)
    host = alloc_host(w, batch, full)
    oracle_run(w, host)
    out = w.names("out")[0]
    parts = [np.load(os.path.join(str(tmp_path), "r%d.npy" % r)) for r in range(world)]
    if w.batch_contracted:
        for p in parts:                                      # all ranks hold the same total
            assert np.array_equal(p, parts[0])
        mags = np.zeros_like(host[out])
        oracle.contract("port", w.program[0][0], mags, np.abs(full["A"]), np.abs(full["B"]))
        assert oracle.parity_error(parts[0], host[out], mags) <= 1e-12     # only the summation order differs
    else:
        assert np.array_equal(np.concatenate(parts, axis=0), host[out])    # disjoint slabs: bit-identical


def test_slabs_partition_the_batch():
    for batch in (1, 7, 8, 1000, (1 << 26) + 3):
        for world in (1, 2, 3, 4, 8):
            edges = [slab(batch, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == batch
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1


def test_allreduce_is_a_no_op_without_a_process_group():
    t = torch.arange(9, dtype=torch.float64)
    assert torch.equal(allreduce_partial(t.clone()), t)


def plan_worker(rank, world, port, rows_of_rank, out_dir):
    import acrotensor_b200 as ab
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = rows_of_rank[rank]
        facts = []
        for kernel, shapes in (("S_i_j = A_n_i_j B_n", [(3, 3), (rows, 3, 3), (rows,)]),
                               ("S_a_b = X_n_a Y_n_b", [(27, 27), (rows, 27), (rows, 27)]),
                               ("C_e_i_j = A_e_i_k B_e_k_j", [(rows, 4, 4), (rows, 4, 4), (rows, 4, 4)])):
            text = ab.describe_plan([kernel], [shapes])
            family = text.split("family=")[1].split()[0]
            joins = "summed over the ranks" in text
            facts.append((kernel, family, joins))
        everyone = [None] * world
        dist.all_gather_object(everyone, facts)
        if rank == 0:
            import json
            with open(os.path.join(out_dir, "plans.json"), "w") as f:
                json.dump(everyone, f)
    finally:
        dist.destroy_process_group()


def test_ranks_with_unequal_slabs_agree_on_which_results_are_summed_over_ranks(tmp_path):
    """A rank with a short slab plans another kernel family than its peers (here 100 rows against 300000), but whether
    a result is summed over the ranks depends on the string alone, so every rank joins the same exchanges."""
    import json
    world = 2
    mp.spawn(plan_worker, args=(world, free_port(), [100, 300000], str(tmp_path)), nprocs=world, join=True)
    with open(os.path.join(str(tmp_path), "plans.json")) as f:
        short, long_ = json.load(f)
    assert [f[1] for f in short] == ["generic", "generic", "batched_gemm"]
    assert [f[1] for f in long_] == ["reduce_batch", "gram", "batched_gemm"]
    assert [f[2] for f in short] == [f[2] for f in long_] == [True, True, False]
