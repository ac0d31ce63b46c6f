"""The C++ API (include/*.hpp + libacrotensor.so) used the way user code written against the
reference uses it: a small C++ program is compiled with g++ and run.  Host-only checks run
everywhere; with -m gpu the same program must also pass its device section.  When the
reference checkout is present, its own host-only unit tests (unittest/tensor/*.cpp,
unittest/kernel/test_TensorKernel.cpp, test_DimensionedKernel.cpp) are compiled unmodified
against THIS library's headers and run too."""
import os
import subprocess

import pytest

import acrotensor_b200 as ab

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("ACRO_REFERENCE_DIR", "/root/reference")
LIBDIR = os.path.dirname(ab.LIB_PATH)


def build(tmp_path, sources, name, extra_inc=()):
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++17", "-O1", "-w", "-I" + os.path.join(ROOT, "include")] + ["-I" + i for i in extra_inc] + \
        list(sources) + ["-L" + LIBDIR, "-lacrotensor", "-Wl,-rpath," + LIBDIR, "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-4000:]
    return exe


@pytest.fixture(scope="module")
def api_check(tmp_path_factory):
    return build(tmp_path_factory.mktemp("cpp"), [os.path.join(ROOT, "tests", "cpp", "api_check.cpp")], "api_check")


def test_cpp_api_host_side(api_check):
    res = subprocess.run([api_check], capture_output=True, text=True)
    assert res.returncode == 0 and "OK" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_api_on_device(api_check):
    res = subprocess.run([api_check, "gpu"], capture_output=True, text=True)
    assert res.returncode == 0 and "with device" in res.stdout, res.stdout + res.stderr


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "unittest")), reason="reference checkout not present")
def test_reference_host_unit_tests_compile_and_pass_against_this_library(tmp_path):
    ut = os.path.join(REF, "unittest")
    sources = [os.path.join(ut, "unit_test_main.cpp"), os.path.join(ut, "tensor", "test_Tensor.cpp"),
               os.path.join(ut, "tensor", "test_SliceTensor.cpp"), os.path.join(ut, "kernel", "test_TensorKernel.cpp"),
               os.path.join(ut, "kernel", "test_DimensionedKernel.cpp")]
    exe = build(tmp_path, sources, "ref_unittests", extra_inc=[ut])
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode == 0, (res.stdout + res.stderr)[-4000:]
    assert "All tests passed" in res.stdout
