"""A C++ program written against include/hexb.h only (tests/cpp/wrapper_check.cpp, in the shape of the
reference's MLIR-file wrappers) builds and links against libhexb200.so on any box, and on a GPU runs
the two wrapper cases end to end and leaves a Test_Info report the reference's tooling can parse."""
import os
import shutil
import subprocess

import pytest

import hexb200
from hexb200 import report

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "hexagon-mlir_b200")


@pytest.fixture(scope="module")
def wrapper_binary(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++ on this box")
    hexb200.load()  # the library must exist (and export its symbols) before anything links against it
    out = tmp_path_factory.mktemp("cpp") / "wrapper_check"
    cmd = [gxx, "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "wrapper_check.cpp"), "-o", str(out),
           "-L", LIBDIR, "-lhexb200", f"-Wl,-rpath,{LIBDIR}"]
    cuda_lib = "/usr/local/cuda/lib64"
    if os.path.isdir(cuda_lib):
        cmd += [f"-Wl,-rpath-link,{cuda_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return str(out)


def test_cpp_program_builds_and_links_against_the_c_abi(wrapper_binary):
    res = subprocess.run([wrapper_binary], capture_output=True, text=True)   # no arguments: usage, no GPU call
    assert res.returncode == 2 and "usage" in res.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["hexkl_linalg_matmul", "hexkl_attention"])
def test_cpp_wrapper_case_passes_and_reports(wrapper_binary, tmp_path, case):
    path = tmp_path / "perf.txt"
    res = subprocess.run([wrapper_binary, case, str(path)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    rep = report.TestReport.parse(path.read_text())
    assert rep.name == case and rep.result == "Pass" and rep.units == "microseconds" and rep.perf > 0
