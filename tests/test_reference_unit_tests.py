"""The reference's own unit tests (unittest/tensor/*.cpp, unittest/kernel/*.cpp), compiled where they lie
and linked against this library by `make -C oracle ref_tests`.

They are the strongest statement of "drop-in" available: the same test sources a user of the reference
runs, against these headers and this shared library.  The binaries are built on a machine that has the
reference checkout and travel with the tree; where they are absent the tests skip.

  * acro_unit_tests       built as a CPU-only user builds (no ACRO_HAVE_CUDA): the Tensor, SliceTensor,
                          TensorKernel and DimensionedKernel cases need no device and run anywhere.
  * acro_unit_tests_cuda  built with -DACRO_HAVE_CUDA: every case, including the engine suite
                          (unittest/kernel/test_TensorEngine.cpp: basic computations, an externally created
                          context, externally allocated device memory, multi-kernel launches, the finite
                          element contractions, batched inverses / determinants, scatter and sum-gather).
                          The engine the test asks for as "CPUInterpreted" is created as "Cuda"
                          (oracle/ref_unit_tests_engine.hpp): this library has no CPU executor.
"""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "..", "oracle", "_ref")


def run_cases(binary, *spec):
    path = os.path.join(REF_OUT, binary)
    if not os.path.exists(path):
        pytest.skip(f"{binary} was not built (needs the reference checkout: make -C oracle ref_tests)")
    done = subprocess.run([path, *spec], capture_output=True, text=True, timeout=300)
    tail = (done.stdout + done.stderr)[-3000:]
    assert done.returncode == 0, tail
    assert "All tests passed" in done.stdout, tail
    return done.stdout


@pytest.mark.parametrize("tag", ["[Tensor]", "[SliceTensor]", "[TensorKernel]", "[DimensionedKernel]"])
def test_reference_host_cases(tag):
    out = run_cases("acro_unit_tests", tag)
    assert "in 1 test case" in out


def test_reference_engine_case_fails_loudly_without_a_device():
    """Without a device the engine case must stop with the library's error, not compute on the CPU."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    path = os.path.join(REF_OUT, "acro_unit_tests")
    if not os.path.exists(path):
        pytest.skip("acro_unit_tests was not built")
    done = subprocess.run([path, "[TensorEngine]"], capture_output=True, text=True, timeout=300)
    assert done.returncode != 0
    assert "no CPU execution path" in done.stdout + done.stderr


@pytest.mark.gpu
def test_reference_unit_tests_on_device():
    out = run_cases("acro_unit_tests_cuda")
    assert "5 test cases" in out
