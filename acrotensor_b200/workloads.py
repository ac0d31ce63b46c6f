"""The five benchmark contractions, as data: contraction strings, tensor shapes as a
function of the batch size, seeded synthetic input generators, and the algorithmic
byte / flop counts used for roofline fractions.

No public dataset is involved: shapes and value distributions are the ones the
benchmark definition states, inputs are seeded pseudo-random numbers.
"""
import numpy as np

MASS_CHAIN = [
    # (kernel string, output, inputs)
    ("T1_e_i1_i2_k3 = B_k3_i3 U_e_i1_i2_i3", "T1", ["B", "U"]),
    ("T2_e_i1_k2_k3 = B_k2_i2 T1_e_i1_i2_k3", "T2", ["B", "T1"]),
    ("X_e_k1_k2_k3 = B_k1_i1 T2_e_i1_k2_k3 W_e_k1_k2_k3", "X", ["B", "T2", "W"]),
    ("Y1_e_i1_k2_k3 = B_k1_i1 X_e_k1_k2_k3", "Y1", ["B", "X"]),
    ("Y2_e_i1_i2_k3 = B_k2_i2 Y1_e_i1_k2_k3", "Y2", ["B", "Y1"]),
    ("V_e_i1_i2_i3 = B_k3_i3 Y2_e_i1_i2_k3", "V", ["B", "Y2"]),
]


class Workload:
    """One benchmark configuration.

    tensors: name -> (shape function of the batch size, batched?, role)
             role in {"in", "out", "tmp"}; "tmp" tensors only link kernels of a chain.
    program: [(kernel string, output name, [input names])]
    """

    def __init__(self, key, title, batch, tensors, program, gen, bytes_fn, flops_fn, bound, multi=False,
                 batch_contracted=False, executed_flops_fn=None):
        self.key, self.title, self.batch = key, title, batch
        self.tensors, self.program, self.gen = tensors, program, gen
        self.bytes_fn, self.flops_fn, self.bound = bytes_fn, flops_fn, bound
        self.multi, self.batch_contracted = multi, batch_contracted
        # flops the kernel really executes when that differs from the algorithmic count
        self.executed_flops_fn = executed_flops_fn or flops_fn

    def shapes(self, batch):
        return {n: tuple(spec[0](batch)) for n, spec in self.tensors.items()}

    def names(self, role):
        return [n for n, spec in self.tensors.items() if spec[2] == role]

    def batched(self, name):
        return self.tensors[name][1]

    def make_inputs(self, batch, seed=0, rank=0):
        """Seeded host inputs (float64, C-contiguous) for one rank's slab of `batch` units."""
        rng = np.random.default_rng([0xAC20, self.index, seed, rank])
        shared = np.random.default_rng([0xAC20, self.index, seed, 10 ** 6])   # batch-invariant tensors
        return self.gen(self.shapes(batch), rng, shared)

    def make_inputs_device(self, batch, device, seed=0, rank=0):
        """The same distributions generated directly on a CUDA device with torch's seeded
        generator (full-size inputs are tens of GB: generating them on the host would
        dominate the run).  Returns name -> torch float64 tensor."""
        import torch
        gen = torch.Generator(device=device)
        gen.manual_seed(0xAC20_0000 + 1000 * self.index + 17 * seed + rank)
        shared = torch.Generator(device=device)
        shared.manual_seed(0xAC20_0000 + 1000 * self.index + 17 * seed + 999)
        shp = self.shapes(batch)

        def uni(g, shape, lo, hi):
            t = torch.rand(shape, generator=g, device=device, dtype=torch.float64)
            return t.mul_(hi - lo).add_(lo) if (lo, hi) != (0.0, 1.0) else t

        k = self.key
        if k == "cfg0":
            return {"A": uni(gen, shp["A"], 0.0, 1.0), "B": torch.ones(shp["B"], device=device, dtype=torch.float64)}
        if k == "cfg1":
            return {"W": uni(gen, shp["W"], 0.5, 1.5), "B": uni(shared, shp["B"], -1.0, 1.0)}
        if k == "cfg2":
            return {"B": uni(shared, shp["B"], -1.0, 1.0), "U": uni(gen, shp["U"], -1.0, 1.0),
                    "W": uni(gen, shp["W"], 0.5, 1.5)}
        if k == "cfg3":
            J = uni(gen, shp["Jinv"], -0.2, 0.2)
            for d in range(3):
                J[..., d, d] += 1.0
            a = [J[..., i // 3, i % 3] for i in range(9)]
            det = (a[0] * a[4] * a[8] + a[1] * a[5] * a[6] + a[2] * a[3] * a[7]
                   - a[6] * a[4] * a[2] - a[7] * a[5] * a[0] - a[8] * a[3] * a[1])
            inv = torch.empty_like(J)
            cof = [(4, 8, 5, 7), (2, 7, 1, 8), (1, 5, 2, 4), (5, 6, 3, 8), (0, 8, 2, 6), (2, 3, 0, 5),
                   (3, 7, 4, 6), (1, 6, 0, 7), (0, 4, 1, 3)]
            for i, (p, q, r, t) in enumerate(cof):
                inv[..., i // 3, i % 3] = (a[p] * a[q] - a[r] * a[t]) / det
            del J
            return {"W": uni(shared, shp["W"], 0.5, 1.5), "DetJ": det.contiguous(), "Jinv": inv}
        if k == "cfg4":
            return {"A": torch.randn(shp["A"], generator=gen, device=device, dtype=torch.float64),
                    "B": torch.randn(shp["B"], generator=gen, device=device, dtype=torch.float64)}
        raise KeyError(k)

    def bytes(self, batch):
        return self.bytes_fn(batch)

    def flops(self, batch):
        return self.flops_fn(batch)


def _uniform(rng, shape, lo, hi):
    out = rng.random(shape)
    if (lo, hi) != (0.0, 1.0):
        out *= (hi - lo)
        out += lo
    return out


def _gen_cfg0(shp, rng, shared):
    return {"A": _uniform(rng, shp["A"], 0.0, 1.0), "B": np.ones(shp["B"])}


def _gen_cfg1(shp, rng, shared):
    return {"W": _uniform(rng, shp["W"], 0.5, 1.5), "B": _uniform(shared, shp["B"], -1.0, 1.0)}


def _gen_cfg2(shp, rng, shared):
    return {"B": _uniform(shared, shp["B"], -1.0, 1.0), "U": _uniform(rng, shp["U"], -1.0, 1.0),
            "W": _uniform(rng, shp["W"], 0.5, 1.5)}


def inv_det_3x3(J):
    """Host-side inverse and determinant of a batch of 3x3 matrices (adjugate formula)."""
    a = [J[..., i // 3, i % 3] for i in range(9)]
    det = (a[0] * a[4] * a[8] + a[1] * a[5] * a[6] + a[2] * a[3] * a[7]
           - a[6] * a[4] * a[2] - a[7] * a[5] * a[0] - a[8] * a[3] * a[1])
    inv = np.empty_like(J)
    invdet = 1.0 / det
    inv[..., 0, 0] = invdet * (a[4] * a[8] - a[5] * a[7])
    inv[..., 0, 1] = invdet * (a[2] * a[7] - a[1] * a[8])
    inv[..., 0, 2] = invdet * (a[1] * a[5] - a[2] * a[4])
    inv[..., 1, 0] = invdet * (a[5] * a[6] - a[3] * a[8])
    inv[..., 1, 1] = invdet * (a[0] * a[8] - a[2] * a[6])
    inv[..., 1, 2] = invdet * (a[2] * a[3] - a[0] * a[5])
    inv[..., 2, 0] = invdet * (a[3] * a[7] - a[4] * a[6])
    inv[..., 2, 1] = invdet * (a[1] * a[6] - a[0] * a[7])
    inv[..., 2, 2] = invdet * (a[0] * a[4] - a[1] * a[3])
    return inv, det


def _gen_cfg3(shp, rng, shared):
    E = shp["Jinv"][0]
    jinv = np.empty(shp["Jinv"])
    det = np.empty(shp["DetJ"])
    chunk = 1 << 14
    for e0 in range(0, E, chunk):   # bounded temporaries at full size
        e1 = min(E, e0 + chunk)
        J = _uniform(rng, (e1 - e0,) + tuple(shp["Jinv"][1:]), -0.2, 0.2)
        J[..., 0, 0] += 1.0
        J[..., 1, 1] += 1.0
        J[..., 2, 2] += 1.0
        jinv[e0:e1], det[e0:e1] = inv_det_3x3(J)
    return {"W": _uniform(shared, shp["W"], 0.5, 1.5), "DetJ": det, "Jinv": jinv}


def _gen_cfg4(shp, rng, shared):
    return {"A": rng.standard_normal(shp["A"]), "B": rng.standard_normal(shp["B"])}


WORKLOADS = [
    Workload(
        "cfg0", "README reduction S_i_j = A_n_i_j B_n", 1 << 26,
        {"S": (lambda n: (3, 3), False, "out"), "A": (lambda n: (n, 3, 3), True, "in"),
         "B": (lambda n: (n,), True, "in")},
        [("S_i_j = A_n_i_j B_n", "S", ["A", "B"])], _gen_cfg0,
        lambda n: 80 * n + 72, lambda n: 18 * n, "hbm", batch_contracted=True),
    Workload(
        "cfg1", "element mass matrices M_e_i_j = W_e_q B_q_i B_q_j (Q2 hex, 27 dofs, 64 points)", 1 << 18,
        {"M": (lambda e: (e, 27, 27), True, "out"), "W": (lambda e: (e, 64), True, "in"),
         "B": (lambda e: (64, 27), False, "in")},
        [("M_e_i_j = W_e_q B_q_i B_q_j", "M", ["W", "B", "B"])], _gen_cfg1,
        lambda e: e * 6344 + 13824, lambda e: 2 * 64 * 729 * e, "fp64",
        # B is passed twice, so M_e is symmetric: the kernel computes 384 packed columns (378 + padding)
        executed_flops_fn=lambda e: 2 * 64 * 384 * e),
    Workload(
        "cfg2", "sum-factorised 3D mass operator, p=3 hex, six-stage chain", 1 << 20,
        {"B": (lambda e: (5, 4), False, "in"), "U": (lambda e: (e, 4, 4, 4), True, "in"),
         "W": (lambda e: (e, 5, 5, 5), True, "in"), "T1": (lambda e: (e, 4, 4, 5), True, "tmp"),
         "T2": (lambda e: (e, 4, 5, 5), True, "tmp"), "X": (lambda e: (e, 5, 5, 5), True, "tmp"),
         "Y1": (lambda e: (e, 4, 5, 5), True, "tmp"), "Y2": (lambda e: (e, 4, 4, 5), True, "tmp"),
         "V": (lambda e: (e, 4, 4, 4), True, "out")},
        MASS_CHAIN, _gen_cfg2, lambda e: e * 2024 + 160, lambda e: 5380 * e, "hbm", multi=True),
    Workload(
        "cfg3", "diffusion geometric factors D_e_k_m_n = W_k DetJ_e_k Jinv_e_k_m_l Jinv_e_k_n_l", 1 << 20,
        {"D": (lambda e: (e, 64, 3, 3), True, "out"), "W": (lambda e: (64,), False, "in"),
         "DetJ": (lambda e: (e, 64), True, "in"), "Jinv": (lambda e: (e, 64, 3, 3), True, "in")},
        [("D_e_k_m_n = W_k DetJ_e_k Jinv_e_k_m_l Jinv_e_k_n_l", "D", ["W", "DetJ", "Jinv", "Jinv"])], _gen_cfg3,
        lambda e: e * 9728 + 512, lambda e: 108 * 64 * e, "hbm"),
    Workload(
        "cfg4", "dense batched contraction C_e_i_j = A_e_i_k B_e_k_j (64^3)", 1 << 14,
        {"C": (lambda e: (e, 64, 64), True, "out"), "A": (lambda e: (e, 64, 64), True, "in"),
         "B": (lambda e: (e, 64, 64), True, "in")},
        [("C_e_i_j = A_e_i_k B_e_k_j", "C", ["A", "B"])], _gen_cfg4,
        lambda e: 98304 * e, lambda e: 524288 * e, "fp64"),
]
for _i, _w in enumerate(WORKLOADS):
    _w.index = _i
BY_KEY = {w.key: w for w in WORKLOADS}
