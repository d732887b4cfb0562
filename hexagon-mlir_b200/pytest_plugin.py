"""pytest plugin that runs the reference's own test directory against this library, unedited:

    PYTHONPATH=<this repo> python -m pytest -p hexb200.pytest_plugin -p no:cacheprovider \
        <checkout of qualcomm/hexagon-mlir>/test/python/triton

Loading the plugin installs hexb200.triton_shim before pytest imports the first test module, so the
modules' own ``from triton.backends.qcom_hexagon_backend.driver import HexagonDriver``,
``triton.runtime.driver.set_active(HexagonDriver())`` and ``@triton.jit`` (test/python/triton/
test_softmax.py:13-44) resolve to the stub driver and to launchers of the CUDA kernels.  The test
bodies -- shapes, CPU tensors, HexagonOptions keywords, torch comparisons and tolerances -- run as written.
"""
from . import triton_shim

triton_shim.install()
