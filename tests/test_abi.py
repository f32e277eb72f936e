"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "raptor_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from raptor_t_b200 import capi
    names = _declared()
    assert len(names) >= 35
    for n in names:
        assert hasattr(capi.lib, n), f"{n} declared in include/raptor_b200.h but not exported"
    assert capi.lib.rt_version() >= 100


def test_bindings_cover_the_header():
    from raptor_t_b200 import capi
    assert set(_declared()) <= set(capi._SIGS), set(_declared()) - set(capi._SIGS)


def test_no_cpu_fallback_and_errors_are_messages():
    import torch
    from raptor_t_b200 import capi
    if torch.cuda.is_available():
        pytest.skip("CPU-only behaviour")
    cfg = capi.make_config(hidden=128, heads=2, ffn=256, layers=1)
    h = ctypes.c_void_p()
    rc = capi.lib.rt_encoder_create(ctypes.byref(cfg), ctypes.byref(h))
    assert rc == 3 and b"no CUDA device" in capi.lib.rt_last_error()
    from raptor_t_b200.engine import Encoder
    with pytest.raises(RuntimeError):
        Encoder(cfg)
    bad = capi.make_config(hidden=100, heads=2)
    rc = capi.lib.rt_count_visits(ctypes.byref(bad), capi.i32_array([64]), 1, ctypes.byref(ctypes.c_int64()))
    assert rc == 2 and b"heads*64" in capi.lib.rt_last_error()


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "raptor_t_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
