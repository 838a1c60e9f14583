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


def test_reference_binding_links(lib):
    """The reference's runtime.cpp, compiled with its GPU backend switched on, links against the six gpu_*
    functions of oracle/gpu_exec_b200_check.cpp (forwarding to the C ABI) with no undefined symbol:
    the signatures are those of src/runtime/runtime_internal.h:288-301. Needs the reference checkout."""
    import subprocess
    from oracle import pyoracle
    if not os.path.isdir(os.path.join(pyoracle.REF_SRC, "src", "runtime")):
        pytest.skip("reference checkout not present")
    if not os.path.exists("/usr/local/cuda/include/cuda_runtime.h") and not os.environ.get("CUDA_HOME"):
        pytest.skip("CUDA headers not present")
    out = os.path.join(ROOT, "oracle", "_ref", "libfastllm_b200_binding.so")
    if os.path.exists(out):
        os.remove(out)
    res = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "binding", "REF=" + pyoracle.REF_SRC],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0 and os.path.exists(out), res.stdout
    syms = subprocess.run(["nm", "-D", "--defined-only", out], stdout=subprocess.PIPE, text=True).stdout
    for name in ("gpu_make_stream", "gpu_start", "gpu_resident_blocks", "gpu_stop_sync", "gpu_calibrate_clock",
                 "gpu_default_blocks"):
        assert name in syms, name
