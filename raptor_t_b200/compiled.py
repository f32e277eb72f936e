"""Loader of the compiled pybind11 module `raptor_t` (csrc/pybind_shim.cpp): the reference's
extension-module API (python/pybind.cpp:11-80) as a real extension module, every method a
sequence of calls into the C ABI.  `raptor_t_b200.raptor_t` is the same API bound with ctypes."""
import importlib.util
import sys

from . import build as _build
from . import capi  # noqa: F401  (loads libraptor_b200.so first; fails loudly if it cannot be built)


def load():
    """Build (if stale) and import the module; returns it.  Also registered as sys.modules['raptor_t'],
    the name the reference's Python layer imports (python/modeling_bert.py:9)."""
    if "raptor_t" in sys.modules and getattr(sys.modules["raptor_t"], "__file__", "").endswith("raptor_t.so"):
        return sys.modules["raptor_t"]
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    path = _build.build_shim()
    spec = importlib.util.spec_from_file_location("raptor_t", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["raptor_t"] = mod
    return mod
