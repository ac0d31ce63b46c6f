"""Python mirror of acro::Tensor / acro::SliceTensor / acro::TensorEngine over the C ABI.

Method names and argument meaning follow the reference's C++ API
(tensor/Tensor.hpp:15-127, tensor/SliceTensor.hpp:14-57,
kernel/TensorEngine.hpp:26-86 of LLNL/acrotensor); failures raise AcroError
where the C++ API throws std::runtime_error.
"""
import ctypes

import numpy as np

from . import _lib
from ._lib import check, lib


def device_count():
    return lib().acro_b200_device_count()


def isCudaReady():
    return device_count() > 0


def set_stream(stream_ptr):
    """Library-wide CUDA stream (an integer cudaStream_t; 0 = legacy default stream)."""
    check(lib().acro_b200_set_stream(ctypes.c_void_p(stream_ptr or 0)))


def _text(fn, *args, size=1 << 16):
    buf = ctypes.create_string_buffer(size)
    check(fn(*args, buf, size))
    return buf.value.decode()


def describe_kernel(kernel):
    """Parser view of a contraction string (no device needed)."""
    return _text(lib().acro_b200_describe_kernel, kernel.encode())


def describe_plan(kernels, shapes, transient_intermediates=False):
    """Planner view of a kernel group bound to shapes (no device, no data needed).
    ``shapes[k]`` lists the output shape and then each input shape of kernel k."""
    n = len(kernels)
    ks = (ctypes.c_char_p * n)(*[k.encode() for k in kernels])
    flat = [d for per_kernel in shapes for shape in per_kernel for d in shape]
    dims = (ctypes.c_int * len(flat))(*flat)
    buf = ctypes.create_string_buffer(1 << 16)
    check(lib().acro_b200_describe_plan(n, ks, dims, int(transient_intermediates), buf, len(buf)))
    return buf.value.decode()


class Tensor:
    """acro::Tensor.  ``Tensor(d0, d1, ...)`` owns its host buffer; ``Tensor(shape, hdata=ndarray)``
    views a float64 C-contiguous numpy array; ``ddata`` is an integer device pointer (or an object
    with ``data_ptr()``, e.g. a torch CUDA tensor) used as the externally owned device mirror."""

    def __init__(self, *dims, hdata=None, ddata=None, ongpu=False, _handle=None, _keep=None):
        self._keep = [_keep, hdata, ddata]
        if _handle is not None:
            self._h = _handle
            return
        if len(dims) == 1 and isinstance(dims[0], (list, tuple)):
            dims = tuple(dims[0])
        if hdata is not None:
            if not (isinstance(hdata, np.ndarray) and hdata.dtype == np.float64 and hdata.flags.c_contiguous):
                raise TypeError("hdata must be a C-contiguous float64 numpy array")
            if not dims:
                dims = hdata.shape
        hptr = hdata.ctypes.data if hdata is not None else None
        dptr = ddata.data_ptr() if hasattr(ddata, "data_ptr") else ddata
        arr = (ctypes.c_int * len(dims))(*[int(d) for d in dims])
        h = ctypes.c_void_p()
        check(lib().acro_tensor_create(len(dims), arr, hptr, dptr, int(bool(ongpu)), ctypes.byref(h)))
        self._h = h

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h is not None and _lib._lib is not None:
            _lib._lib.acro_tensor_destroy(h)

    # shape ---------------------------------------------------------------
    def GetRank(self):
        return lib().acro_tensor_rank(self._h)

    def GetSize(self):
        return lib().acro_tensor_size(self._h)

    def GetDim(self, d):
        r = lib().acro_tensor_dim(self._h, d)
        if r < 0:
            raise IndexError("dimension out of range")
        return r

    @property
    def shape(self):
        return tuple(self.GetDim(d) for d in range(self.GetRank()))

    def Reshape(self, *dims):
        if len(dims) == 1 and isinstance(dims[0], (list, tuple)):
            dims = tuple(dims[0])
        arr = (ctypes.c_int * len(dims))(*dims)
        check(lib().acro_tensor_reshape(self._h, len(dims), arr))

    # data ----------------------------------------------------------------
    def GetData(self):
        return lib().acro_tensor_data(self._h)

    def GetDeviceData(self):
        return lib().acro_tensor_device_data(self._h)

    def GetCurrentData(self):
        return self.GetDeviceData() if self.IsOnGPU() else self.GetData()

    def numpy(self):
        """The host buffer as a numpy view (valid while this Tensor lives)."""
        n = self.GetSize()
        buf = (ctypes.c_double * n).from_address(self.GetData())
        return np.frombuffer(buf, dtype=np.float64).reshape(self.shape)

    def Retarget(self, hdata, ddata=None):
        self._keep = [None, hdata, ddata]      # the previous buffers are no longer referenced by this tensor
        dptr = ddata.data_ptr() if hasattr(ddata, "data_ptr") else ddata
        check(lib().acro_tensor_retarget(self._h, hdata.ctypes.data, dptr))

    # GPU motion ------------------------------------------------------------
    def MapToGPU(self):
        check(lib().acro_tensor_map_to_gpu(self._h))

    def MoveToGPU(self):
        check(lib().acro_tensor_move_to_gpu(self._h))

    def SwitchToGPU(self):
        check(lib().acro_tensor_switch_to_gpu(self._h))

    def UnmapFromGPU(self):
        check(lib().acro_tensor_unmap_from_gpu(self._h))

    def MoveFromGPU(self):
        check(lib().acro_tensor_move_from_gpu(self._h))

    def SwitchFromGPU(self):
        check(lib().acro_tensor_switch_from_gpu(self._h))

    def IsMappedToGPU(self):
        return bool(lib().acro_tensor_is_mapped_to_gpu(self._h))

    def IsOnGPU(self):
        return bool(lib().acro_tensor_is_on_gpu(self._h))

    def IsInitialized(self):
        return True

    def Set(self, val):
        check(lib().acro_tensor_set(self._h, float(val)))

    def Mult(self, c):
        check(lib().acro_tensor_mult(self._h, float(c)))

    def SetTransient(self, flag=True):
        check(lib().acro_tensor_set_transient(self._h, int(bool(flag))))

    def SetSharded(self, flag=True):
        """This tensor is this rank's slab of a tensor cut along its leading dimension over the ranks
        of a peer group (see TensorEngine.SetPeerGroup)."""
        check(lib().acro_tensor_set_sharded(self._h, int(bool(flag))))

    def IsSharded(self):
        return bool(lib().acro_tensor_is_sharded(self._h))


def batch_slab(batch, rank, world):
    """acro::SlabOf: the contiguous range [begin, end) of a batch index of extent `batch` owned by
    `rank` of `world` (host arithmetic of the library; no device needed)."""
    b, e = ctypes.c_int64(), ctypes.c_int64()
    check(lib().acro_b200_batch_slab(int(batch), int(rank), int(world), ctypes.byref(b), ctypes.byref(e)))
    return b.value, e.value


class SlabTensor(Tensor):
    """acro::SlabTensor(T, begin, end) / SlabTensor(T, rank=, world=): rows [begin, end) of the leading
    dimension of T, sharing T's host buffer, with a device mirror of the slab only; flagged sharded."""

    def __init__(self, parent, begin=None, end=None, rank=None, world=None):
        if begin is None:
            begin, end = batch_slab(parent.GetDim(0), rank, world)
        h = ctypes.c_void_p()
        check(lib().acro_tensor_slab(parent._h, int(begin), int(end), ctypes.byref(h)))
        super().__init__(_handle=h, _keep=parent)
        self.begin, self.end = int(begin), int(end)


class SliceTensor(Tensor):
    """acro::SliceTensor(T, i0, ...): the trailing dimensions of T at a fixed prefix."""

    def __init__(self, parent, *indices):
        arr = (ctypes.c_int * len(indices))(*indices)
        h = ctypes.c_void_p()
        check(lib().acro_tensor_slice(parent._h, len(indices), arr, ctypes.byref(h)))
        super().__init__(_handle=h, _keep=parent)


class IndexMapping:
    """acro::IndexMapping(domain_size, range_size): ``M[i]`` in [0, domain_size) for i < range_size."""

    def __init__(self, domain_size, range_size, values=None):
        h = ctypes.c_void_p()
        check(lib().acro_index_mapping_create(int(domain_size), int(range_size), ctypes.byref(h)))
        self._h = h
        self.domain_size, self.range_size = int(domain_size), int(range_size)
        if values is not None:
            self.numpy()[:] = values

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h is not None and _lib._lib is not None:
            _lib._lib.acro_index_mapping_destroy(h)

    def numpy(self):
        """The host map as a writable int32 numpy view."""
        buf = (ctypes.c_int * self.range_size).from_address(lib().acro_index_mapping_data(self._h))
        return np.frombuffer(buf, dtype=np.int32)

    def GetDomainSize(self):
        return self.domain_size

    def GetRangeSize(self):
        return self.range_size

    def ComputeInverse(self):
        check(lib().acro_index_mapping_compute_inverse(self._h))

    def inverse(self):
        """(InvMap, InvMapOffsets) as numpy copies, or None before ComputeInverse."""
        p, q = lib().acro_index_mapping_inverse(self._h), lib().acro_index_mapping_inverse_offsets(self._h)
        if not p or not q:
            return None
        inv = np.frombuffer((ctypes.c_int * self.range_size).from_address(p), dtype=np.int32).copy()
        off = np.frombuffer((ctypes.c_int * (self.domain_size + 1)).from_address(q), dtype=np.int32).copy()
        return inv, off


class PeerGroup:
    """The ranks (one process per GPU of a node) that hold slabs of a contracted batch index.
    ``exchange(handle_bytes) -> [handle_bytes of every rank in rank order]`` is supplied by the
    caller (e.g. torch.distributed.all_gather_object); world size 1 needs none."""

    def __init__(self, world, rank, exchange=None):
        h = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        check(lib().acro_b200_peer_group_create(int(world), int(rank), ctypes.byref(h), handle))
        self._h = h
        self.world, self.rank = int(world), int(rank)
        if world > 1:
            if exchange is None:
                raise ValueError("a peer group of more than one rank needs an exchange function")
            everyone = exchange(handle.raw)
            assert len(everyone) == world and all(len(b) == _lib.IPC_HANDLE_BYTES for b in everyone)
            check(lib().acro_b200_peer_group_connect(self._h, b"".join(everyone)))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h is not None and _lib._lib is not None:
            _lib._lib.acro_b200_peer_group_destroy(h)


class SharedEntryExchange:
    """Sums the domain entries of a sharded IndexMapping that several ranks reach (one process per GPU
    of one node); completes FlatIndexedSumGather when the range is cut into one slab per rank.
    ``exchange(bytes) -> [bytes of every rank in rank order]`` is supplied by the caller (e.g.
    torch.distributed.all_gather_object) and is called with the touched-entry bitmap, then with the CUDA
    IPC handle of this rank's inbox.  ``on_device=False`` builds the host-side plan only (no CUDA call);
    ``connect=False`` leaves the inboxes unconnected for :meth:`connect_pointers` (ranks of one process)."""

    def __init__(self, mapping, world, rank, exchange=None, on_device=True, connect=True):
        self.world, self.rank, self.domain_size = int(world), int(rank), mapping.GetDomainSize()
        nbytes = (self.domain_size + 7) // 8
        mine = ctypes.create_string_buffer(nbytes)
        m = np.ascontiguousarray(mapping.numpy(), dtype=np.int32)
        check(lib().acro_b200_halo_mark_touched(m.ctypes.data_as(ctypes.c_void_p), m.size, self.domain_size, mine))
        if world > 1:
            if exchange is None:
                raise ValueError("an exchange over more than one rank needs an exchange function")
            everyone = exchange(mine.raw)
            assert len(everyone) == world and all(len(b) == nbytes for b in everyone)
        else:
            everyone = [mine.raw]
        h = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        check(lib().acro_b200_halo_create(self.world, self.rank, self.domain_size, b"".join(everyone), int(bool(on_device)),
                                          ctypes.byref(h), handle))
        self._h = h
        if on_device and connect and world > 1:
            handles = exchange(handle.raw)
            assert len(handles) == world and all(len(b) == _lib.IPC_HANDLE_BYTES for b in handles)
            check(lib().acro_b200_halo_connect(self._h, b"".join(handles)))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h is not None and _lib._lib is not None:
            _lib._lib.acro_b200_halo_destroy(h)

    def counts(self):
        """(shared entries of this rank, (entry, other rank) pairs, doubles per half of this rank's inbox)."""
        a, b, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        check(lib().acro_b200_halo_counts(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
        return a.value, b.value, c.value

    def plan(self):
        """The plan arrays as numpy int32: shared_idx, entry_off, entry_peer, entry_send, entry_recv."""
        ns, ne, _ = self.counts()
        arrays = [np.zeros(n, dtype=np.int32) for n in (ns, ns + 1, ne, ne, ne)]
        check(lib().acro_b200_halo_copy_plan(self._h, *[a.ctypes.data_as(ctypes.c_void_p) for a in arrays]))
        return arrays

    def inbox(self):
        return lib().acro_b200_halo_inbox(self._h)

    def connect_pointers(self, inboxes):
        check(lib().acro_b200_halo_connect_pointers(self._h, (ctypes.c_void_p * self.world)(*inboxes)))

    def send(self, device_pointer, stream=None):
        check(lib().acro_b200_halo_send(self._h, ctypes.c_void_p(device_pointer), stream))

    def combine(self, device_pointer, stream=None):
        check(lib().acro_b200_halo_combine(self._h, ctypes.c_void_p(device_pointer), stream))

    def exchange_sum(self, device_pointer, stream=None):
        check(lib().acro_b200_halo_exchange_sum(self._h, ctypes.c_void_p(device_pointer), stream))


class TensorEngine:
    """acro::TensorEngine.  ``TE("S_i_j = A_n_i_j B_n", S, A, B)`` runs one contraction;
    Begin/EndMultiKernelLaunch record several and run them as one unit."""

    def __init__(self, exec_type="Cuda"):
        h = ctypes.c_void_p()
        check(lib().acro_engine_create(exec_type.encode(), ctypes.byref(h)))
        self._h = h

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h is not None and _lib._lib is not None:
            _lib._lib.acro_engine_destroy(h)

    def SetExecutorType(self, exec_type):
        check(lib().acro_engine_set_executor_type(self._h, exec_type.encode()))

    def GetExecType(self):
        return _text(lib().acro_engine_exec_type, self._h, size=64)

    @staticmethod
    def _handles(inputs):
        return (ctypes.c_void_p * len(inputs))(*[t._h for t in inputs])

    def __call__(self, kernel, out, *inputs):
        if len(inputs) == 1 and isinstance(inputs[0], (list, tuple)):
            inputs = tuple(inputs[0])
        check(lib().acro_engine_contract(self._h, kernel.encode(), out._h, len(inputs), self._handles(inputs)))

    def GetImplementation(self, kernel, out, *inputs):
        buf = ctypes.create_string_buffer(1 << 16)
        check(lib().acro_engine_implementation(self._h, kernel.encode(), out._h, len(inputs),
                                               self._handles(inputs), buf, len(buf)))
        return buf.value.decode()

    def BeginMultiKernelLaunch(self):
        check(lib().acro_engine_begin_multi(self._h))

    def EndMultiKernelLaunch(self):
        check(lib().acro_engine_end_multi(self._h))

    def EndMultiKernelLaunchDescribe(self):
        return _text(lib().acro_engine_end_multi_describe, self._h)

    def BatchMatrixInverse(self, Ainv, A):
        check(lib().acro_engine_batch_matrix_inverse(self._h, Ainv._h, A._h))

    def BatchMatrixDet(self, Adet, A):
        check(lib().acro_engine_batch_matrix_det(self._h, Adet._h, A._h))

    def BatchMatrixInvDet(self, Ainv, Adet, A):
        check(lib().acro_engine_batch_matrix_inv_det(self._h, Ainv._h, Adet._h, A._h))

    def FlatIndexedScatter(self, Aout, Ain, M):
        check(lib().acro_engine_flat_indexed_scatter(self._h, Aout._h, Ain._h, M._h))

    def FlatIndexedSumGather(self, Aout, Ain, M, shared=None):
        """``shared``: a SharedEntryExchange when M maps this rank's slab of a sharded range; the domain
        entries shared with other ranks are then summed over them (collective over the ranks)."""
        if shared is None:
            check(lib().acro_engine_flat_indexed_sum_gather(self._h, Aout._h, Ain._h, M._h))
        else:
            check(lib().acro_engine_flat_indexed_sum_gather_shared(self._h, Aout._h, Ain._h, M._h, shared._h))

    def Clear(self):
        check(lib().acro_engine_clear(self._h))

    def IsGPUAvailable(self):
        return isCudaReady()

    def SetPeerGroup(self, group):
        """Attach a PeerGroup (None detaches): a contraction that sums over the leading index of an
        input flagged sharded (SlabTensor, Tensor.SetSharded) then returns the sum over all ranks'
        slabs on every rank (inside the kernel for the reduce_batch family, by an all-reduce kernel
        after the step for every other family)."""
        self._peer_group = group
        check(lib().acro_engine_set_peer_group(self._h, group._h if group is not None else None))

    def SetCudaStream(self, stream_ptr):
        check(lib().acro_engine_set_stream(self._h, ctypes.c_void_p(stream_ptr or 0)))
