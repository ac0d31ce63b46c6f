"""Seeded random contraction strings for fuzz tests: 1-3 inputs of rank 1-4, small extents,
repeated indices inside a variable (diagonals), output-only indices (broadcast), and all three
assignment operators."""
import numpy as np


def random_case(rng):
    pool = ["i", "j", "k", "l", "m", "n", "p2", "q1"]
    n_idx = int(rng.integers(1, 6))
    names = list(rng.choice(pool, size=n_idx, replace=False))
    extent = {n: int(rng.integers(1, 5)) for n in names}
    n_in = int(rng.integers(1, 4))
    ins = []
    for _ in range(n_in):
        rank = int(rng.integers(1, 5))
        ins.append([str(x) for x in rng.choice(names, size=rank, replace=True)])
    used = sorted({x for v in ins for x in v})
    out_rank = int(rng.integers(1, 4))
    # mostly indices the inputs carry, sometimes one that only the output has (broadcast)
    candidates = used + ([n for n in names if n not in used][:1] if rng.random() < 0.3 else [])
    out = [str(x) for x in rng.choice(candidates, size=min(out_rank, len(candidates)), replace=False)]
    op = str(rng.choice(["=", "=", "+=", "-="]))
    var_names = ["B", "Cx", "D2"]
    text = "A_" + "_".join(out) + " " + op + " " + " ".join(var_names[v] + "_" + "_".join(ins[v]) for v in range(n_in))
    shapes = {"A": tuple(extent[x] for x in out)}
    for v in range(n_in):
        shapes[var_names[v]] = tuple(extent[x] for x in ins[v])
    return text, shapes, [var_names[v] for v in range(n_in)], op


def cases(seed, count):
    rng = np.random.default_rng(seed)
    return [random_case(rng) for _ in range(count)]
