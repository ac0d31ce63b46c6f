"""Generates tests/golden/reference_outputs.npz by running the UNMODIFIED reference
(LLNL/acrotensor, CPUInterpreted executor, compiled by oracle/Makefile into
oracle/_ref/libacro_ref.so) on the seeded inputs of tests/cases.py.

Run in a container that has the reference checkout:
    python tests/golden/make_golden.py
The file stores, per case, every written tensor AFTER the program ran, and a SHA-256 of
the seeded inputs (the tests regenerate the inputs from the seed and compare the digest,
so a generator change cannot go unnoticed).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    oracle.build()
    assert oracle.have("ref"), "the reference checkout is needed to generate golden vectors"
    blob = {}
    for case in cases.all_cases():
        name = case[0]
        tensors = cases.make_tensors(case)
        names = sorted(tensors)
        blob["%s/inputs_sha256" % name] = np.array(cases.digest(tensors))
        oracle.run("ref", [tensors[n] for n in names], cases.as_oracle_program(case, names), multi=case[3])
        for n in cases.written(case):
            blob["%s/out/%s" % (name, n)] = tensors[n]
    for name, dim, batch in cases.OPS_INV_DET:
        a = cases.make_matrices(name, dim, batch)
        blob["%s/inputs_sha256" % name] = np.array(cases.digest({"A": a}))
        inv, det = oracle.batch_inv_det("ref", a)
        blob["%s/out/inv" % name], blob["%s/out/det" % name] = inv, det
    for name, domain, rng_size in cases.OPS_INDEXED:
        mapping, dom_vals, rng_vals = cases.make_indexed(name, domain, rng_size)
        blob["%s/inputs_sha256" % name] = np.array(cases.digest({"M": mapping, "D": dom_vals, "R": rng_vals}))
        blob["%s/out/scatter" % name] = oracle.flat_indexed("ref", dom_vals, mapping, domain, False)
        blob["%s/out/gather" % name] = oracle.flat_indexed("ref", rng_vals, mapping, domain, True)
    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes,", len(cases.all_cases()), "cases")


if __name__ == "__main__":
    main()
