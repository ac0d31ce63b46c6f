"""Runs a benchmark Workload through the public engine API, on one rank's slab of the batch.

Multi-GPU model (one process per GPU): the batch (element) index is cut into contiguous
slabs, one per rank; batch-invariant tensors are replicated.  No data-path collective is
needed unless the batch index is contracted away (the README reduction): then every rank
holds a partial result and one all-reduce(sum) of the small output finishes the job.
"""
import numpy as np

from .host import Tensor, TensorEngine, batch_slab


def slab(batch, rank, world):
    """Contiguous range [begin, end) of the batch index owned by `rank` of `world` (acro::SlabOf)."""
    return batch_slab(batch, rank, world)


class Session:
    """Binds host (numpy) and optional device (torch CUDA) buffers of one workload to
    acro Tensors and runs its contraction program.

    host:   name -> float64 C-contiguous ndarray for every tensor of the workload
    device: name -> torch CUDA float64 tensor used as the externally owned device mirror
            (optional; without it MapToGPU allocates).
    transient: flag chain intermediates as transient so a fused plan may keep them on chip.
    sharded: the batched tensors are this rank's slabs of the batch index (Tensor.SetSharded): with a
            peer group attached to the engine a contraction over the batch index is summed over ranks.
    """

    def __init__(self, workload, host, device=None, transient=True, engine=None, sharded=False):
        self.w = workload
        self.host = host
        self.device = device or {}
        self.te = engine or TensorEngine("Cuda")
        self.t = {}
        for name in workload.tensors:
            self.t[name] = Tensor(host[name].shape, hdata=host[name], ddata=self.device.get(name))
            if transient and workload.tensors[name][2] == "tmp":
                self.t[name].SetTransient(True)
            if sharded and workload.batched(name):
                self.t[name].SetSharded(True)

    def to_device(self, names=None):
        for name in names or self.w.names("in"):
            self.t[name].SwitchFromGPU()
            self.t[name].MoveToGPU()

    def mark_outputs_on_device(self):
        for name in self.w.names("out") + self.w.names("tmp"):
            self.t[name].SwitchToGPU()

    def run(self):
        te = self.te
        if self.w.multi:
            te.BeginMultiKernelLaunch()
        for kernel, out, ins in self.w.program:
            te(kernel, self.t[out], *[self.t[i] for i in ins])
        if self.w.multi:
            te.EndMultiKernelLaunch()

    def fetch(self, names=None):
        for name in names or self.w.names("out"):
            self.t[name].MoveFromGPU()

    def plan_text(self):
        te = self.te
        if not self.w.multi:
            kernel, out, ins = self.w.program[0]
            return te.GetImplementation(kernel, self.t[out], *[self.t[i] for i in ins])
        te.BeginMultiKernelLaunch()
        for kernel, out, ins in self.w.program:
            te(kernel, self.t[out], *[self.t[i] for i in ins])
        return te.EndMultiKernelLaunchDescribe()


def make_peer_group():
    """PeerGroup of all ranks of the initialised torch.distributed job (one process per GPU of one
    node); the CUDA IPC handles of the mailboxes are exchanged with all_gather_object."""
    import torch.distributed as dist
    from .host import PeerGroup
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return PeerGroup(1, 0)

    def exchange(mine):
        everyone = [None] * dist.get_world_size()
        dist.all_gather_object(everyone, mine)
        return everyone

    return PeerGroup(dist.get_world_size(), dist.get_rank(), exchange)


def allreduce_partial(device_tensor, group=None):
    """Sum the per-rank partial results of a contracted batch index in place
    (torch.distributed; NCCL on GPUs, gloo in the CPU tests)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(device_tensor, op=dist.ReduceOp.SUM, group=group)
    return device_tensor


def alloc_host(workload, batch, inputs):
    """Host arrays for every tensor of the workload: the given inputs plus zeroed
    outputs / intermediates."""
    host = dict(inputs)
    for name, shape in workload.shapes(batch).items():
        if name not in host:
            host[name] = np.zeros(shape)
    return host
