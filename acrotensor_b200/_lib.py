"""Loads ``libacrotensor.so`` (the C ABI declared in include/acro_b200.h).

The shared library carries the whole product: the acro:: C++ API, the planner
and the sm_100a kernels.  There is no Python or CPU fallback: when the library
is missing, importing this module fails, and when no CUDA device is present
every compute entry point returns ACRO_B200_ECUDA.
"""
import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libacrotensor.so")
CSRC = os.path.join(HERE, "csrc")

OK, EINVAL, EUNSUPPORTED, ECUDA, ETIMEOUT = 0, -1, -2, -3, -4
MAX_LOOPS, MAX_INPUTS, MAX_POINT_LOOPS, MAX_SCALARS = 24, 12, 6, 6
MAX_PEERS, IPC_HANDLE_BYTES = 16, 64
OP_ASSIGN, OP_ADD, OP_SUB = 0, 1, 2
SCRATCH_READY = 0x100


class AcroError(RuntimeError):
    """Raised when a C-ABI call reports a failure (the C++ API would throw)."""

    def __init__(self, status, text):
        super().__init__("acro_b200 status %d: %s" % (status, text))
        self.status = status


def build(verbose=False, jobs=8):
    """Compile libacrotensor.so in-tree with nvcc for sm_100a."""
    res = subprocess.run(["make", "-C", CSRC, "-j%d" % jobs], capture_output=True, text=True)
    if verbose or res.returncode:
        print(res.stdout[-4000:], res.stderr[-4000:])
    if res.returncode:
        raise RuntimeError("building libacrotensor.so failed")


class GenericDesc(ctypes.Structure):
    _fields_ = [("n_loops", ctypes.c_int32), ("n_outer", ctypes.c_int32), ("n_inputs", ctypes.c_int32),
                ("op", ctypes.c_int32), ("extent", ctypes.c_int64 * MAX_LOOPS),
                ("out_step", ctypes.c_int64 * MAX_LOOPS),
                ("in_step", (ctypes.c_int64 * MAX_LOOPS) * MAX_INPUTS)]


class PointwiseDesc(ctypes.Structure):
    _fields_ = [("dim", ctypes.c_int32), ("op", ctypes.c_int32), ("n_point_loops", ctypes.c_int32),
                ("n_scalars", ctypes.c_int32), ("point_extent", ctypes.c_int64 * MAX_POINT_LOOPS),
                ("scalar_step", (ctypes.c_int64 * MAX_POINT_LOOPS) * MAX_SCALARS),
                ("cell_points", ctypes.c_int64), ("swapped", ctypes.c_int32), ("reserved", ctypes.c_int32)]


_P = ctypes.c_void_p
_I = ctypes.c_int
_I64 = ctypes.c_int64
_D = ctypes.c_double
_SZ = ctypes.c_size_t
_S = ctypes.c_char_p

# name -> (restype, argtypes); every symbol include/acro_b200.h declares.
SIGNATURES = {
    "acro_b200_last_error": (_S, []),
    "acro_b200_device_count": (_I, []),
    "acro_b200_device_status": (_I, []),
    "acro_b200_set_context": (_I, [_P]),
    "acro_b200_fill": (_I, [_P, _I64, _D, _P]),
    "acro_b200_scale": (_I, [_P, _I64, _D, _P]),
    "acro_b200_generic_launch": (_I, [ctypes.POINTER(GenericDesc), _P, ctypes.POINTER(_P), _P, _SZ, _P]),
    "acro_b200_generic_scratch_bytes": (_SZ, [ctypes.POINTER(GenericDesc)]),
    "acro_b200_permute_supported": (_I, [ctypes.POINTER(GenericDesc)]),
    "acro_b200_permute": (_I, [ctypes.POINTER(GenericDesc), _P, _P, _P]),
    "acro_b200_generic_blocking": (_I, [ctypes.POINTER(GenericDesc), ctypes.POINTER(ctypes.c_int)]),
    "acro_b200_generic_uses_wide_kernel": (_I, [ctypes.POINTER(GenericDesc)]),
    "acro_b200_reduce_batch_scratch_bytes": (_SZ, [_I]),
    "acro_b200_reduce_batch_supported": (_I, [_I64, _I]),
    "acro_b200_reduce_batch": (_I, [_P, _P, _P, _I64, _I, _I, _P, _SZ, _P]),
    "acro_b200_peer_group_create": (_I, [_I, _I, ctypes.POINTER(_P), _P]),
    "acro_b200_peer_group_connect": (_I, [_P, _P]),
    "acro_b200_peer_group_destroy": (_I, [_P]),
    "acro_b200_peer_group_world": (_I, [_P]),
    "acro_b200_peer_group_is_connected": (_I, [_P]),
    "acro_b200_reduce_batch_allreduce": (_I, [_P, _P, _P, _I64, _I, _I, _P, _SZ, _P, _P]),
    "acro_b200_peer_allreduce": (_I, [_P, _P, _I64, _I, _P, _P]),
    "acro_engine_set_peer_group": (_I, [_P, _P]),
    "acro_b200_reduce_batch_noalloc_max_f": (_I, []),
    "acro_b200_reduce_batch_noalloc": (_I, [_P, _P, _P, _I64, _I, _I, _P]),
    "acro_b200_pointwise_sym_supported": (_I, [ctypes.POINTER(PointwiseDesc)]),
    "acro_b200_pointwise_sym": (_I, [ctypes.POINTER(PointwiseDesc), ctypes.POINTER(_P), _P, _P, _P, _P]),
    "acro_b200_rank1_gemm_supported": (_I, [_I, _I, _I]),
    "acro_b200_rank1_gemm": (_I, [_P, _P, _P, _P, _I64, _I, _I, _I, _I, _P]),
    "acro_b200_batched_gemm_supported": (_I, [_I, _I, _I]),
    "acro_b200_batched_gemm": (_I, [_P, _P, _P, _I64, _I, _I, _I, _I, _P]),
    "acro_b200_batched_gemm_t_supported": (_I, [_I, _I, _I, _I, _I]),
    "acro_b200_batched_gemm_by_pairs": (_I, [_I, _I, _I, _I, _I]),
    "acro_b200_batched_gemm_t": (_I, [_P, _P, _P, _I64, _I, _I, _I, _I, _I, _I, _P]),
    "acro_b200_gram_supported": (_I, [_I, _I]),
    "acro_b200_gram_scratch_bytes": (_SZ, [_I, _I]),
    "acro_b200_gram": (_I, [_P, _P, _P, _I64, _I, _I, _I, _P, _SZ, _P]),
    "acro_b200_gemm": (_I, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I, _P]),
    "acro_b200_gemm_batched": (_I, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I, _P]),
    "acro_b200_sumfact_mass_supported": (_I, [_I, _I]),
    "acro_b200_sumfact_mass": (_I, [_P, _P, _P, _P, _I64, _I, _I, _P]),
    "acro_b200_batch_inv_det": (_I, [_P, _P, _P, _I64, _I, _P]),
    "acro_b200_flat_scatter": (_I, [_P, _P, _P, _I64, _P]),
    "acro_b200_flat_sum_gather": (_I, [_P, _P, _P, _P, _I64, _P]),
    "acro_b200_halo_mark_touched": (_I, [_P, _I64, _I64, _P]),
    "acro_b200_halo_create": (_I, [_I, _I, _I64, _P, _I, ctypes.POINTER(_P), _P]),
    "acro_b200_halo_counts": (_I, [_P, ctypes.POINTER(_I64), ctypes.POINTER(_I64), ctypes.POINTER(_I64)]),
    "acro_b200_halo_copy_plan": (_I, [_P, _P, _P, _P, _P, _P]),
    "acro_b200_halo_connect": (_I, [_P, _P]),
    "acro_b200_halo_inbox": (_P, [_P]),
    "acro_b200_halo_connect_pointers": (_I, [_P, _P]),
    "acro_b200_halo_send": (_I, [_P, _P, _P]),
    "acro_b200_halo_combine": (_I, [_P, _P, _P]),
    "acro_b200_halo_exchange_sum": (_I, [_P, _P, _P]),
    "acro_b200_halo_destroy": (_I, [_P]),
    "acro_index_mapping_create": (_I, [_I, _I, ctypes.POINTER(_P)]),
    "acro_index_mapping_destroy": (_I, [_P]),
    "acro_index_mapping_data": (_P, [_P]),
    "acro_index_mapping_compute_inverse": (_I, [_P]),
    "acro_index_mapping_inverse": (_P, [_P]),
    "acro_index_mapping_inverse_offsets": (_P, [_P]),
    "acro_engine_batch_matrix_inverse": (_I, [_P, _P, _P]),
    "acro_engine_batch_matrix_det": (_I, [_P, _P, _P]),
    "acro_engine_batch_matrix_inv_det": (_I, [_P, _P, _P, _P]),
    "acro_engine_flat_indexed_scatter": (_I, [_P, _P, _P, _P]),
    "acro_engine_flat_indexed_sum_gather": (_I, [_P, _P, _P, _P]),
    "acro_engine_flat_indexed_sum_gather_shared": (_I, [_P, _P, _P, _P, _P]),
    "acro_tensor_create": (_I, [_I, ctypes.POINTER(_I), _P, _P, _I, ctypes.POINTER(_P)]),
    "acro_tensor_slice": (_I, [_P, _I, ctypes.POINTER(_I), ctypes.POINTER(_P)]),
    "acro_tensor_destroy": (_I, [_P]),
    "acro_tensor_rank": (_I, [_P]),
    "acro_tensor_size": (_I64, [_P]),
    "acro_tensor_dim": (_I, [_P, _I]),
    "acro_tensor_data": (_P, [_P]),
    "acro_tensor_device_data": (_P, [_P]),
    "acro_tensor_is_on_gpu": (_I, [_P]),
    "acro_tensor_is_mapped_to_gpu": (_I, [_P]),
    "acro_tensor_map_to_gpu": (_I, [_P]),
    "acro_tensor_move_to_gpu": (_I, [_P]),
    "acro_tensor_switch_to_gpu": (_I, [_P]),
    "acro_tensor_unmap_from_gpu": (_I, [_P]),
    "acro_tensor_move_from_gpu": (_I, [_P]),
    "acro_tensor_switch_from_gpu": (_I, [_P]),
    "acro_tensor_set": (_I, [_P, _D]),
    "acro_tensor_mult": (_I, [_P, _D]),
    "acro_tensor_reshape": (_I, [_P, _I, ctypes.POINTER(_I)]),
    "acro_tensor_retarget": (_I, [_P, _P, _P]),
    "acro_tensor_set_transient": (_I, [_P, _I]),
    "acro_b200_batch_slab": (_I, [_I64, _I, _I, ctypes.POINTER(_I64), ctypes.POINTER(_I64)]),
    "acro_tensor_slab": (_I, [_P, _I64, _I64, ctypes.POINTER(_P)]),
    "acro_tensor_set_sharded": (_I, [_P, _I]),
    "acro_tensor_is_sharded": (_I, [_P]),
    "acro_engine_create": (_I, [_S, ctypes.POINTER(_P)]),
    "acro_engine_destroy": (_I, [_P]),
    "acro_engine_set_executor_type": (_I, [_P, _S]),
    "acro_engine_exec_type": (_I, [_P, _P, _SZ]),
    "acro_engine_contract": (_I, [_P, _S, _P, _I, ctypes.POINTER(_P)]),
    "acro_engine_implementation": (_I, [_P, _S, _P, _I, ctypes.POINTER(_P), _P, _SZ]),
    "acro_engine_begin_multi": (_I, [_P]),
    "acro_engine_end_multi": (_I, [_P]),
    "acro_engine_end_multi_describe": (_I, [_P, _P, _SZ]),
    "acro_engine_clear": (_I, [_P]),
    "acro_engine_set_stream": (_I, [_P, _P]),
    "acro_b200_set_stream": (_I, [_P]),
    "acro_b200_describe_kernel": (_I, [_S, _P, _SZ]),
    "acro_b200_describe_plan": (_I, [_I, ctypes.POINTER(_S), ctypes.POINTER(_I), _I, _P, _SZ]),
}

_lib = None


def lib():
    """The loaded shared library with typed entry points."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "acrotensor_b200: %s is missing. Build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `make -C acrotensor_b200/csrc`; there is no fallback implementation." % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError = the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status):
    if status != OK:
        raise AcroError(status, lib().acro_b200_last_error().decode(errors="replace"))
    return status
