"""GPU: the reference's own Triton test modules, unmodified, run against this library.

Needs a checkout of qualcomm/hexagon-mlir: set HEXAGON_MLIR_REF to it (the test is skipped otherwise;
nothing under that path is read by any other test).  pytest is started as a child process on the
checkout's test/python/triton directory with the plugin hexb200.pytest_plugin, which installs the
triton shim before the first module is imported; every test function of every module must pass.
The checkout may be read-only: the child writes no cache or bytecode files.
"""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_triton_tests_pass_unmodified():
    ref = os.environ.get("HEXAGON_MLIR_REF")
    if not ref or not os.path.isdir(os.path.join(ref, "test", "python", "triton")):
        pytest.skip("set HEXAGON_MLIR_REF to a checkout of qualcomm/hexagon-mlir to run its own tests")
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), PYTHONDONTWRITEBYTECODE="1")
    cmd = [sys.executable, "-m", "pytest", "-q", "-p", "hexb200.pytest_plugin", "-p", "no:cacheprovider",
           "--rootdir", os.path.join(ref, "test"), "-o", "addopts=", os.path.join(ref, "test", "python", "triton")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1200, cwd=ROOT)
    tail = (r.stdout + r.stderr)[-3000:]
    m = re.search(r"(\d+) passed", r.stdout)
    assert r.returncode == 0 and m, tail
    assert not re.search(r"\d+ (failed|error)", r.stdout), tail
    assert int(m.group(1)) >= 40, tail        # 24 modules, 49 parametrised cases in the checkout this was written against
    print(tail.strip().splitlines()[-1])
