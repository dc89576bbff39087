"""The C-ABI library loads without a GPU and exports what include/lzb200.h
declares; compute entry points fail loudly when no B200 is present."""
import os
import re

import pytest

from conftest import ROOT


def _declared(header="lzb200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lzb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lzb):
    assert _declared() == sorted(lzb.SYMBOLS)


def test_library_exports_every_declared_symbol(lzb):
    lib = lzb.lib()
    missing = [s for s in _declared() if not hasattr(lib, s)]
    assert not missing, missing


def test_scheduler_library_exports_its_header(lzb):
    """libcudapipe.so (the C++ CUDAPipe with its C view) against include/lzb200_sched.h."""
    assert _declared("lzb200_sched.h") == sorted(lzb.SCHED_SYMBOLS)
    lib = lzb.sched_lib()
    missing = [s for s in _declared("lzb200_sched.h") if not hasattr(lib, s)]
    assert not missing, missing


def test_scheduler_c_view_refuses_bad_calls(lzb):
    """Argument and call-order errors of include/lzb200_sched.h come back as
    status codes with a text, without a GPU being touched."""
    import ctypes
    L = lzb.sched_lib()
    h = ctypes.c_void_p()
    ids = (ctypes.c_int * 1)(0)
    assert L.lzb_sched_create(ctypes.byref(h), ids, 1, 0, 8, lzb.FP16, 0) == 1      # batch size 0
    assert b"bad arguments" in L.lzb_sched_last_error()
    assert L.lzb_sched_create(ctypes.byref(h), ids, 1, 8, 8, 99, 0) == 1            # unknown precision
    assert L.lzb_sched_create(ctypes.byref(h), ids, 1, 8, 8, lzb.FP16_X2, 1) == 0
    x = (ctypes.c_float * 8)()
    assert L.lzb_sched_forward(h, x, 1, x, x) == 1                                   # not started
    assert b"not started" in L.lzb_sched_last_error()
    assert L.lzb_sched_drain(h) == 1 and L.lzb_sched_resume(h) == 1
    fp = ctypes.cast(x, ctypes.POINTER(ctypes.c_float))
    assert L.lzb_sched_add_conv(h, None, 18, 8, fp, fp) == 1                         # null weights
    assert L.lzb_sched_start(h, 8, None, fp) == 1
    out = (ctypes.c_ulonglong * 8)()
    assert L.lzb_sched_stats(h, out) == 0 and out[0] == 0
    L.lzb_sched_destroy(h)


def test_no_cpu_fallback(lzb):
    """Without a CUDA device the library must refuse, not compute elsewhere."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(lzb.LzbError):
        lzb.device_count()
    net = lzb.weights.synthetic_network(1, 8, 1)
    with pytest.raises(lzb.LzbError):
        lzb.Pipe(net, "fp32")
    with pytest.raises(RuntimeError):
        lzb.Scheduler(lzb.weights.prepare(lzb.weights.synthetic_raw_network(1, 8, 1)), "fp32")


def test_product_does_not_touch_the_oracle():
    """Nothing under the package may import, link or open the checker."""
    pkg = os.path.join(ROOT, "leela-zero_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".hpp", ".mk")) or f == "Makefile":
                text = open(os.path.join(base, f), errors="ignore").read()
                assert "oracle" not in text.lower(), os.path.join(base, f)
