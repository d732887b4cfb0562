"""Import shim: makes the package directory ``hexagon-mlir_b200/`` importable as ``hexb200``.

The directory name carries a hyphen (it mirrors the upstream project's name), which Python's import
statement cannot spell; this module loads that directory as a regular package under the name
``hexb200`` and replaces itself in ``sys.modules`` with it.
"""
import importlib.util
import os
import sys

_pkg_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hexagon-mlir_b200")
_spec = importlib.util.spec_from_file_location(
    "hexb200", os.path.join(_pkg_dir, "__init__.py"), submodule_search_locations=[_pkg_dir]
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules["hexb200"] = _mod
_spec.loader.exec_module(_mod)
