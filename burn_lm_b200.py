"""Import shim: the package lives in the folder `burn-lm_b200/`, whose name Python cannot import.

`import burn_lm_b200` finds this file, loads that folder as the package `burn_lm_b200` and puts it
in `sys.modules` under this name, so that submodules (`burn_lm_b200.engine`, ...) resolve there.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "burn-lm_b200")
_spec = importlib.util.spec_from_file_location(
    "burn_lm_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_pkg = importlib.util.module_from_spec(_spec)
sys.modules["burn_lm_b200"] = _pkg
_spec.loader.exec_module(_pkg)
