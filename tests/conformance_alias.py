"""pytest plugin (``-p conformance_alias``): makes ``import tilefish`` resolve to this package, so that the reference's own
CPU test files exercise this package's typed front end. Used only by tests/test_reference_conformance.py, in a child process."""

import importlib
import os
import pkgutil
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import tilefish_b200  # noqa: E402

sys.modules["tilefish"] = tilefish_b200
for _m in pkgutil.iter_modules(tilefish_b200.__path__):
    if _m.name in ("csrc", "runtime", "native_plan", "kernels", "mlp", "collective", "_native"):
        continue  # the run-time half (torch, the CUDA library) is not what these tests look at
    sys.modules["tilefish." + _m.name] = importlib.import_module("tilefish_b200." + _m.name)
