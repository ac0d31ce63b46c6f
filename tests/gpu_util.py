"""Helpers of the GPU parity tests: run a case through the engine's C ABI and fetch results."""
import ctypes

import numpy as np

import acrotensor_b200 as ab
import cases
from oracle import oracle


def run_case_on_gpu(case, transient=False, tensors=None):
    """Executes the case's program through acro_engine_* with host inputs; returns
    (tensors after the run, plan text)."""
    name, program, shapes, multi = case
    tensors = tensors or cases.make_tensors(case)
    t = {n: ab.Tensor(tensors[n].shape, hdata=tensors[n]) for n in tensors}
    outs = cases.written(case)
    if transient:
        for n in outs[:-1]:
            t[n].SetTransient(True)
    te = ab.TensorEngine("Cuda")
    if multi:
        te.BeginMultiKernelLaunch()
    for kernel, out, ins in program:
        te(kernel, t[out], *[t[i] for i in ins])
    if multi:
        te.EndMultiKernelLaunch()
    for n in outs:
        t[n].MoveFromGPU()
    if multi:
        te.BeginMultiKernelLaunch()
        for kernel, out, ins in program:
            te(kernel, t[out], *[t[i] for i in ins])
        plan = te.EndMultiKernelLaunchDescribe()
    else:
        kernel, out, ins = program[0]
        plan = "\n".join(te.GetImplementation(k, t[o], *[t[i] for i in ii]) for k, o, ii in program)
    return tensors, plan


def oracle_case(case, kind="port", tensors=None, absolute=False):
    tensors = tensors or cases.make_tensors(case)
    names = sorted(tensors)
    # absolute=True gives sum|terms| per output entry, the scale rounding differences are measured against
    work = {n: (np.abs(tensors[n]) if absolute else tensors[n].copy()) for n in names}
    oracle.run(kind, [work[n] for n in names], cases.as_oracle_program(case, names), multi=case[3])
    return work


def families(plan):
    return [line.split("family=")[1].split()[0] for line in plan.splitlines() if "family=" in line]


BIT_EXACT_FAMILIES = {"generic", "pointwise_sym", "permute"}


def dev_ptr(t):
    return ctypes.c_void_p(t.data_ptr())
