"""acrotensor_b200 — B200 (sm_100a) drop-in for LLNL/acrotensor's "Cuda" execution policy.

The product is ``libacrotensor.so`` (C++ ``acro::Tensor`` / ``acro::TensorEngine``
API + C ABI + hand-written CUDA kernels).  This package is the thin Python host
mirror of that API over the C ABI, used by the tests and the benchmark:

    >>> from acrotensor_b200 import Tensor, TensorEngine
    >>> A, B, S = Tensor(1000, 3, 3), Tensor(1000), Tensor(3, 3)
    >>> TE = TensorEngine("Cuda")
    >>> TE("S_i_j = A_n_i_j B_n", S, A, B); S.MoveFromGPU()
"""
from ._lib import AcroError, build, lib, LIB_PATH
from .host import (IndexMapping, PeerGroup, SharedEntryExchange, SlabTensor, SliceTensor, Tensor, TensorEngine, batch_slab, describe_kernel,
                   describe_plan, device_count, isCudaReady, set_stream)

__all__ = ["AcroError", "IndexMapping", "PeerGroup", "SharedEntryExchange", "SlabTensor", "SliceTensor", "Tensor", "TensorEngine", "batch_slab", "build", "describe_kernel", "describe_plan",
           "device_count", "isCudaReady", "lib", "set_stream", "LIB_PATH"]
