"""CPU checks of the boundary: the library builds for sm_100a, loads, exports
every symbol the header declares, and refuses to run without a device."""
import ctypes as C
import os
import re

import pytest

from fast_llm_b200 import build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return capi.load()


def test_header_symbols_all_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "fl_b200.h")).read()
    declared = set(re.findall(r"\b(fl_b200_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(capi.SYMBOLS)
    for s in declared:
        assert hasattr(lib, s), s
    assert lib.fl_b200_abi_version() == 1


def test_task_record_layout():
    assert C.sizeof(capi.Task) == 256
    assert capi.Task.w.offset == 40 and capi.Task.aux.offset == 104 and capi.Task.ystride.offset == 128


def test_no_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    rc = lib.fl_b200_create(0, C.byref(h))
    assert rc != 0 and not h.value
    assert b"no CPU path" in lib.fl_b200_last_error()


def test_product_does_not_use_the_oracle():
    pkg = os.path.join(ROOT, "fast-llm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower() or f == "__init__.py", os.path.join(dirpath, f)
