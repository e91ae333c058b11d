"""The C-ABI library loads without a GPU and exports every symbol the headers declare."""
import ctypes as C
import os
import re

import numpy as np

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


def test_allgather_plan_moves_every_byte_to_every_device():
    # The plan of the C library's all-gather of unequal ranges, simulated on intervals: after the sends of step 1
    # (only bytes the sender holds may be sent; a receive must match the peer's send) and the all-gather of the
    # even shares (every device must hold its own share by then), every device holds every byte.  Crafted and
    # seeded random ranges, byte counts around the 512-byte rounding of the shares.
    rng = np.random.default_rng(5)
    cases = [[0, 10, 20], [0, 0, 7], [0, 4096, 4096 * 8], [0, 100, 300, 5000, 100000], [0, 512 * 3, 512 * 3, 512 * 9 + 5],
             [0, 1 << 20, 3 << 20, 9 << 20, 10 << 20, 11 << 20, 20 << 20, 21 << 20, 64 << 20]]
    for _ in range(60):
        n = int(rng.integers(2, 9))
        total = int(rng.integers(1, 1 << int(rng.integers(4, 24))))
        cases.append([0] + sorted(int(x) for x in rng.integers(0, total + 1, n - 1)) + [total])
    two_step = 0
    for cut in cases:
        n = len(cut) - 1
        c = np.asarray(cut, np.uint64)
        part = C.c_uint64()
        pieces = np.zeros((n, n - 1, 10), np.uint64)
        assert capi.lib().b200spmm_allgather_plan(c.ctypes.data, n, C.byref(part), pieces.ctypes.data) == capi.OK
        part = int(part.value)
        total = cut[-1]
        have = [np.zeros(total, bool) for _ in range(n)]
        for d in range(n):
            have[d][cut[d]:cut[d + 1]] = True
        sends = {}
        for d in range(n):
            for k in range(n - 1):
                to, frm, s_lo, s_hi, t_lo, t_hi = (int(x) for x in pieces[d, k, :6])
                assert to == (d + k + 1) % n and frm == (d - k - 1) % n
                for lo, hi in ((s_lo, s_hi), (t_lo, t_hi)):
                    if hi > lo:
                        assert cut[d] <= lo and hi <= cut[d + 1], "a device sends only what it holds"
                sends[(d, to)] = ((s_lo, s_hi), (t_lo, t_hi))
        for d in range(n):
            for k in range(n - 1):
                frm = int(pieces[d, k, 1])
                got = tuple((int(pieces[d, k, 6 + 2 * i]), int(pieces[d, k, 7 + 2 * i])) for i in range(2))
                want = sends[(frm, d)]
                for (lo, hi), (wlo, whi) in zip(got, want):
                    assert (hi > lo) == (whi > wlo) and (hi <= lo or (lo, hi) == (wlo, whi)), "a receive matches the peer's send"
                    if hi > lo:
                        have[d][lo:hi] = True
        if part:
            two_step += 1
            assert part * n <= total
            for q in range(n):
                assert have[q][part * q:part * (q + 1)].all(), "every device holds its even share before the all-gather"
            for d in range(n):
                have[d][:part * n] = True
        for d in range(n):
            assert have[d].all(), (cut, part)
    assert 0 < two_step < len(cases)
