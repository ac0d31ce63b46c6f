"""Helpers of the shared-entry exchange tests: a mesh-like sharded mapping and a numpy
emulation of the exchange that works from the plan arrays alone."""
import numpy as np


def mesh_mapping(elements, per_element, seed, stray=0.02):
    """Element-local entries -> global entries, like a 1D chain of elements whose neighbours share
    one entry, plus a few random far references (`stray`).  Returns (map, domain_size)."""
    rng = np.random.default_rng(seed)
    domain = elements * (per_element - 1) + 1
    m = (np.arange(elements)[:, None] * (per_element - 1) + np.arange(per_element)[None, :]).astype(np.int32)
    far = rng.random(m.shape) < stray
    m[far] = rng.integers(0, domain, size=int(far.sum()), dtype=np.int32)
    return m.reshape(-1), domain


def slabs(elements, per_element, world):
    return [(elements * r // world * per_element, elements * (r + 1) // world * per_element) for r in range(world)]


def local_sum_gather(values, mapping, domain):
    """out[d] = sum of values[i] over the positions i with mapping[i] = d, in ascending position
    (ops/NativeCPUOps.cpp:127-144 of LLNL/acrotensor, through its CSR inverse)."""
    out = np.zeros(domain)
    for i in range(mapping.size):          # sequential adds in position order
        out[mapping[i]] += values[i]
    return out


def emulate_exchange(plans, partials, strides):
    """plans[r] = (shared_idx, entry_off, entry_peer, entry_send, entry_recv) of rank r;
    partials[r] = that rank's values over the whole domain.  Returns the combined values per rank,
    summing in ascending rank order like the combine kernel."""
    world = len(plans)
    inbox = [np.full(strides[r], np.nan) for r in range(world)]
    for r in range(world):
        idx, off, peer, send, recv = plans[r]
        for k in range(idx.size):
            for e in range(off[k], off[k + 1]):
                assert np.isnan(inbox[peer[e]][send[e]])            # nobody else writes this slot
                inbox[peer[e]][send[e]] = partials[r][idx[k]]
    out = [p.copy() for p in partials]
    for r in range(world):
        idx, off, peer, send, recv = plans[r]
        for k in range(idx.size):
            total, placed = 0.0, False
            for e in range(off[k], off[k + 1]):
                if not placed and peer[e] > r:
                    total, placed = total + partials[r][idx[k]], True
                total = total + inbox[r][recv[e]]
            if not placed:
                total = total + partials[r][idx[k]]
            out[r][idx[k]] = total
    return out
