"""TEST INFRASTRUCTURE — ctypes access to the two CPU checkers.

* ``port``: ``libacro_oracle.so``, this repository's plain-C restatement
  (``acro_oracle.c``) of the reference's interpreted CPU executor
  (exec/CPUInterpretedExecutor.cpp:59-444).
* ``ref``:  ``_ref/libacro_ref.so``, the reference's own sources compiled
  unmodified and CPU-only, behind ``ref_shim.cpp``.

Only tests, the smoke check and the CPU-baseline legs of the benchmark may
import this module.  The product package never does.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "libacro_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libacro_ref.so")
# the reference checkout: ACRO_REFERENCE_DIR, else a directory "reference" beside this repository
REFERENCE_CHECKOUT = os.environ.get("ACRO_REFERENCE_DIR") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))

_libs = {}


def build(verbose=False):
    """Compile the C restatement and, when the reference checkout is present, the
    reference-backed checker and the reference's unit tests linked against the product
    library (otherwise the prebuilt ones are used).  The product library is built first."""
    targets = ["oracle"]
    if os.path.isdir(os.path.join(REFERENCE_CHECKOUT, "exec")):
        targets.append("ref")
    product = os.path.join(HERE, "..", "acrotensor_b200", "libacrotensor.so")
    if os.path.isdir(os.path.join(REFERENCE_CHECKOUT, "unittest")) and os.path.exists(product):
        targets.append("ref_tests")
    cmd = ["make", "-C", HERE, "REF=" + REFERENCE_CHECKOUT] + targets
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        print(res.stdout, res.stderr)
    if res.returncode:
        raise RuntimeError("oracle build failed")


def have(kind):
    return os.path.exists(PORT_SO if kind == "port" else REF_SO)


def _lib(kind):
    if kind in _libs:
        return _libs[kind]
    path = PORT_SO if kind == "port" else REF_SO
    if not os.path.exists(path):
        build()
    lib = ctypes.CDLL(path)
    prefix = "acro_oracle" if kind == "port" else "acro_ref"
    run = getattr(lib, prefix + "_run")
    run.restype = ctypes.c_int
    err = getattr(lib, prefix + "_last_error")
    err.restype = ctypes.c_char_p
    if kind == "ref":
        lib.acro_ref_run_slabs.restype = ctypes.c_int
        lib.acro_ref_hardware_threads.restype = ctypes.c_int
    else:
        lib.acro_oracle_parses.restype = ctypes.c_int
    _libs[kind] = (lib, run, err)
    return _libs[kind]


def _marshal(tensors, program):
    n = len(tensors)
    for t in tensors:
        assert t.dtype == np.float64 and t.flags.c_contiguous
    data = (ctypes.c_void_p * n)(*[t.ctypes.data for t in tensors])
    ranks = (ctypes.c_int * n)(*[t.ndim for t in tensors])
    flat = [d for t in tensors for d in t.shape]
    dims = (ctypes.c_int * len(flat))(*flat)
    nk = len(program)
    kern = (ctypes.c_char_p * nk)(*[p[0].encode() for p in program])
    out_idx = (ctypes.c_int * nk)(*[p[1] for p in program])
    n_in = (ctypes.c_int * nk)(*[len(p[2]) for p in program])
    flat_in = [i for p in program for i in p[2]]
    in_idx = (ctypes.c_int * max(1, len(flat_in)))(*flat_in)
    return n, data, ranks, dims, nk, kern, out_idx, n_in, in_idx


def run(kind, tensors, program, multi=False):
    """Execute ``program`` = [(kernel_string, out_index, [in_index, ...]), ...]
    over the list of float64 C-contiguous numpy arrays ``tensors`` in place."""
    lib, fn, err = _lib(kind)
    args = _marshal(tensors, program)
    rc = fn(*args, int(multi))
    if rc != 0:
        raise RuntimeError(err().decode())


def run_ref_slabs(tensors, program, batched, batch, threads, multi=False):
    """Reference executor over ``threads`` contiguous slabs of the batch index;
    ``batched[i]`` says whether tensor i carries the batch index as its leading
    dimension.  ``threads=1`` is the reference exactly as shipped."""
    lib, _, err = _lib("ref")
    n, data, ranks, dims, nk, kern, out_idx, n_in, in_idx = _marshal(tensors, program)
    b = (ctypes.c_int * n)(*[int(x) for x in batched])
    rc = lib.acro_ref_run_slabs(n, data, ranks, dims, b, ctypes.c_int64(batch), nk, kern, out_idx,
                                n_in, in_idx, int(multi), int(threads))
    if rc != 0:
        raise RuntimeError(err().decode())


def hardware_threads():
    return _lib("ref")[0].acro_ref_hardware_threads()


def parses(kernel):
    return _lib("port")[0].acro_oracle_parses(kernel.encode()) == 0


def contract(kind, kernel, out, *ins):
    """Single contraction convenience wrapper: writes ``out`` in place."""
    run(kind, [out] + list(ins), [(kernel, 0, list(range(1, len(ins) + 1)))])
    return out


def abs_reference(kind, tensors, program, written, multi=False):
    """Sum of |terms| behind every output element: the same program run on the
    absolute values of the inputs.  It is the scale that a summation-order
    difference is measured against (1e-12 * this)."""
    mags = [np.abs(t) for t in tensors]
    for w in written:
        mags[w] = np.zeros_like(tensors[w])
    run(kind, mags, program, multi)
    return mags


def parity_error(got, ref, ref_abs):
    """max over elements of |got-ref| / sum|terms|  (0/0 counts as 0)."""
    num = np.abs(np.asarray(got, dtype=np.float64) - ref)
    den = np.where(ref_abs > 0, ref_abs, 1.0)
    return float(np.max(num / den)) if num.size else 0.0


def batch_inv_det(kind, a, want_inv=True, want_det=True):
    """Inverse and/or determinant of the trailing dim x dim matrices of ``a``.
    Returns (ainv or None, adet or None)."""
    lib = _lib(kind)[0]
    a = np.ascontiguousarray(a, dtype=np.float64)
    dim = a.shape[-1]
    ainv = np.empty_like(a) if want_inv else None
    adet = np.empty(a.shape[:-2] if a.ndim > 2 else (1,)) if want_det else None
    pa = a.ctypes.data_as(ctypes.c_void_p)
    pi = ainv.ctypes.data_as(ctypes.c_void_p) if want_inv else None
    pd = adet.ctypes.data_as(ctypes.c_void_p) if want_det else None
    if kind == "port":
        lib.acro_oracle_batch_inv_det.restype = ctypes.c_int
        rc = lib.acro_oracle_batch_inv_det(pa, pi, pd, ctypes.c_int64(a.size // (dim * dim)), dim)
    else:
        lib.acro_ref_batch_inv_det.restype = ctypes.c_int
        dims = (ctypes.c_int * a.ndim)(*a.shape)
        rc = lib.acro_ref_batch_inv_det(pa, pi, pd, a.ndim, dims)
    if rc != 0:
        raise RuntimeError(_lib(kind)[2]().decode())
    return ainv, adet


def flat_indexed(kind, ain, mapping, domain, gather, with_inverse=False):
    """FlatIndexedScatter (gather=False: out[i] = in[M[i]]) or FlatIndexedSumGather
    (gather=True: out[M[i]] += in[i]).  With the reference library, ``with_inverse`` also
    returns its ComputeInverse() arrays."""
    lib = _lib(kind)[0]
    mapping = np.ascontiguousarray(mapping, dtype=np.int32)
    ain = np.ascontiguousarray(ain, dtype=np.float64)
    rng = mapping.size
    out = np.empty(domain if gather else rng)
    pm = mapping.ctypes.data_as(ctypes.c_void_p)
    po, pi = out.ctypes.data_as(ctypes.c_void_p), ain.ctypes.data_as(ctypes.c_void_p)
    if kind == "port":
        if gather:
            lib.acro_oracle_flat_sum_gather(po, pi, pm, ctypes.c_int64(domain), ctypes.c_int64(rng))
        else:
            lib.acro_oracle_flat_scatter(po, pi, pm, ctypes.c_int64(rng))
        return out
    inv = np.empty(rng, dtype=np.int32)
    off = np.empty(domain + 1, dtype=np.int32)
    lib.acro_ref_flat_indexed.restype = ctypes.c_int
    rc = lib.acro_ref_flat_indexed(po, pi, pm, int(domain), int(rng), int(bool(gather)),
                                   inv.ctypes.data_as(ctypes.c_void_p) if with_inverse else None,
                                   off.ctypes.data_as(ctypes.c_void_p) if with_inverse else None)
    if rc != 0:
        raise RuntimeError(_lib(kind)[2]().decode())
    return (out, inv, off) if with_inverse else out
