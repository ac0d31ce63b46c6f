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
# the reference checkout: ACRO_REFERENCE_DIR, else a directory "reference" beside this repository
REF = os.environ.get("ACRO_REFERENCE_DIR") or os.path.normpath(os.path.join(ROOT, "..", "reference"))
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


def test_dropin_artefacts_link_like_the_reference_build(tmp_path):
    """`make dropin` leaves lib/libacrotensor.a, lib/shared/libacrotensor.so and inc/*.hpp, the names the reference's
    makefile produces; a program built against nothing but those (and the CUDA runtime) passes the host checks."""
    prefix = tmp_path / "acro"
    res = subprocess.run(["make", "-C", os.path.join(ROOT, "acrotensor_b200", "csrc"), "dropin", "PREFIX=" + str(prefix)],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    for rel in ("lib/libacrotensor.a", "lib/shared/libacrotensor.so", "inc/AcroTensor.hpp", "inc/acro_b200.h"):
        assert (prefix / rel).exists(), rel
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "api_static")
    cmd = ["g++", "-std=c++17", "-O1", "-w", "-I" + str(prefix / "inc"), os.path.join(ROOT, "tests", "cpp", "api_check.cpp"),
           "-L" + str(prefix / "lib"), "-l:libacrotensor.a", "-L" + os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread",
           "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0 and "OK" in run.stdout, run.stdout + run.stderr


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
