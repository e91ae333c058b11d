"""The C-ABI library loads without a GPU and exports every symbol the headers declare."""
import ctypes as C
import os
import re

import pytest

from hopper_spmm_b200 import _capi as capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in ("b200_spmm.h", "b200_spmm_kat.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(b200spmm_\w+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported_and_bound():
    lib = C.CDLL(capi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), n
    assert names == set(capi.SIGNATURES), names ^ set(capi.SIGNATURES)


def test_status_strings():
    lib = capi.lib()
    assert lib.b200spmm_status_string(0) == b"ok"
    seen = {lib.b200spmm_status_string(s) for s in range(-7, 1)}
    assert len(seen) == 8 and b"unknown status" not in seen
    assert lib.b200spmm_status_string(-99) == b"unknown status"
    assert lib.b200spmm_version() >= 100


def test_invalid_arguments_return_codes():
    lib = capi.lib()
    out = C.c_void_p()
    assert lib.b200spmm_csr2btcf_nobitmap(4, 4, 0, None, None, None, 0, 16, 0, 0, C.byref(out)) == capi.ERR_INVALID_ARG
    assert lib.b200spmm_plan_create(None, 0, 0, C.byref(out)) == capi.ERR_INVALID_ARG
    assert lib.b200spmm_spmm(None, None, 0, 0, None, 0, 0, None) == capi.ERR_INVALID_ARG
    assert lib.b200spmm_plan_sync(None, None) == capi.ERR_INVALID_ARG


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", "/nonexistent/libb200spmm.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        capi.lib()


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    import numpy as np
    import hopper_spmm_b200 as hs
    rp = np.array([0, 1], np.uint32)
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(1, 1, rp, np.zeros(1, np.uint32), np.ones(1, np.float16)))
    with pytest.raises(capi.SpmmError) as e:
        hs.SpmmPlan(f)
    assert e.value.status == capi.ERR_NO_DEVICE


def test_sharded_operator_argument_checks_need_no_device():
    import numpy as np
    lib = capi.lib()
    rp = np.array([0, 1, 2], np.uint32)
    ci = np.array([0, 1], np.uint32)
    v = np.ones(2, np.float16)
    out = C.c_void_p()
    two = (C.c_int * 2)(0, 0)  # the same device twice
    args = (2, 2, 2, rp.ctypes.data, ci.ctypes.data, v.ctypes.data, capi.F16)
    assert lib.b200spmm_sharded_create(*args, two, 2, 6, C.byref(out)) == capi.ERR_INVALID_ARG
    assert lib.b200spmm_sharded_create(*args, None, 1, 6, C.byref(out)) == capi.ERR_INVALID_ARG
    bad = np.array([0, 5], np.uint32)  # a column past the end is caught before any device is touched
    one = (C.c_int * 1)(0)
    assert lib.b200spmm_sharded_create(2, 2, 2, rp.ctypes.data, bad.ctypes.data, v.ctypes.data, capi.F16, one, 1, 6,
                                       C.byref(out)) == capi.ERR_BAD_CSR
    assert lib.b200spmm_sharded_sync(None) == capi.ERR_INVALID_ARG
    assert lib.b200spmm_allgather_c(None, None, 8, 0) == capi.ERR_INVALID_ARG
    import torch
    if not torch.cuda.is_available():
        assert lib.b200spmm_sharded_create(*args, one, 1, 6, C.byref(out)) == capi.ERR_NO_DEVICE
