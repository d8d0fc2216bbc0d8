"""Import shim: registers the package directory `granite-4-rtx-4070-ti-super_b200/` (whose
name is not a valid Python identifier) as the importable package `granite4_b200`.

    import granite4_b200
    from granite4_b200 import kernels, capi
"""
import importlib.util
import os
import sys

_PKG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)),
                        "granite-4-rtx-4070-ti-super_b200")
_spec = importlib.util.spec_from_file_location(
    "granite4_b200", os.path.join(_PKG_DIR, "__init__.py"),
    submodule_search_locations=[_PKG_DIR])
_pkg = importlib.util.module_from_spec(_spec)
sys.modules["granite4_b200"] = _pkg
_spec.loader.exec_module(_pkg)
