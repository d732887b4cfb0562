"""Lets test files written for the reference run against this library without edits.

The reference's tests ``import triton``, import ``HexagonDriver`` from
``triton.backends.qcom_hexagon_backend.driver``, call ``triton.runtime.driver.set_active(...)`` at
import time and define their kernels under ``@triton.jit`` (test/python/triton/test_softmax.py:13-44).
``install()`` provides those names: the driver module is a stub, ``set_active`` accepts it, and
``triton.jit`` returns an object whose ``[grid](...)`` looks the kernel up by function name in
``hexb200.kernels`` and launches the CUDA implementation.  The body of the decorated function is
never compiled or executed.  This is test-time glue; the library itself does not import triton.
"""
from __future__ import annotations

import sys
import types

from . import kernels


class HexagonDriver:
    """Stand-in for qcom_hexagon_backend/backend/driver.py:117-168 (no device, nothing to drive)."""

    def get_current_target(self):
        return ("b200", 100, 32)


class _JitShim:
    def __init__(self, fn):
        self.fn = fn
        self.__name__ = getattr(fn, "__name__", "kernel")

    def __getitem__(self, grid):
        return kernels.lookup(self.__name__)[grid]

    def __call__(self, *a, **k):
        raise RuntimeError("a @triton.jit function can only be launched as kernel[grid](...)")


def jit(fn=None, **_kw):
    if fn is None:
        return lambda f: _JitShim(f)
    return _JitShim(fn)


def install():
    """Registers the stub modules and patches ``triton.jit`` / ``set_active``; returns the triton module."""
    try:
        import triton  # the stock package, if present, keeps providing triton.language etc.
    except Exception:  # pragma: no cover - triton is optional
        triton = types.ModuleType("triton")
        triton.language = types.ModuleType("triton.language")
        triton.language.constexpr = int
        triton.next_power_of_2 = lambda n: 1 << (max(int(n), 1) - 1).bit_length()
        triton.runtime = types.ModuleType("triton.runtime")
        triton.runtime.driver = types.SimpleNamespace()
        sys.modules.update({"triton": triton, "triton.language": triton.language,
                            "triton.runtime": triton.runtime})
    backends = sys.modules.get("triton.backends") or types.ModuleType("triton.backends")
    pkg = types.ModuleType("triton.backends.qcom_hexagon_backend")
    drv = types.ModuleType("triton.backends.qcom_hexagon_backend.driver")
    drv.HexagonDriver = HexagonDriver
    pkg.driver = drv
    sys.modules.setdefault("triton.backends", backends)
    sys.modules["triton.backends.qcom_hexagon_backend"] = pkg
    sys.modules["triton.backends.qcom_hexagon_backend.driver"] = drv
    setattr(sys.modules["triton.backends"], "qcom_hexagon_backend", pkg)
    triton.jit = jit
    try:
        triton.runtime.driver.set_active = lambda *_a, **_k: None
    except Exception:  # pragma: no cover
        pass
    return triton
