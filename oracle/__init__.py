"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import
this package; the shipped library never does.  ``liboracle.so`` is the plain-C restatement
(``spmm_oracle.c``); ``_ref/libref_{fp16,tf32}.so`` wrap the reference project's own
converter (``src/utils/convert.h:146-225``) where they have been built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
IDX_MAX = 0xFFFFFFFF

_i64 = C.c_int64
_p = C.c_void_p


def reference_dir() -> str:
    """Where the reference project's sources are mounted: $HOPPER_SPMM_REFERENCE, else the default
    mount point.  Only the build of the harness reads it; nothing needs it at run time."""
    return os.environ.get("HOPPER_SPMM_REFERENCE", "/root/reference")


def build(with_ref: bool = False) -> None:
    """Compile the oracle with make; ``with_ref`` also builds the reference harness."""
    targets = ["all"] + (["ref"] if with_ref else [])
    subprocess.run(["make", "-s", "-C", _HERE, "REF=" + reference_dir()] + targets, check=True)


def _load() -> C.CDLL:
    if not os.path.exists(_LIB_PATH):
        build()
    lib = C.CDLL(_LIB_PATH)
    lib.oracle_btcf_count.argtypes = [_i64, _p, _p, C.c_int, C.c_int, C.POINTER(_i64), C.POINTER(_i64)]
    lib.oracle_csr2btcf_nobitmap.argtypes = [_i64, _p, _p, _p, C.c_int, C.c_int, C.c_int, C.c_int, _p, _p, _p, _p]
    lib.oracle_spmm_csr_f16.argtypes = [_i64, _p, _p, _p, _p, _i64, _i64, _p, _i64, _i64, _i64, C.c_int]
    lib.oracle_spmm_csr_f32.argtypes = [_i64, _p, _p, _p, _p, _i64, _i64, _p, _i64, _i64, _i64, C.c_int, C.c_int]
    lib.oracle_spmm_btcf.argtypes = [_i64, _i64, _p, _p, _p, _p, C.c_int, C.c_int, C.c_int, _p, _i64, _i64, _p,
                                     _i64, C.c_int, C.c_int]
    lib.oracle_tile_accumulate.argtypes = [_p, _p, _p, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.oracle_rand_fill.argtypes = [C.c_uint, _p, _i64]
    lib.oracle_compare.argtypes = [_p, _p, _i64, _i64, _i64, _i64, C.c_double, C.POINTER(C.c_double),
                                   C.POINTER(C.c_double)]
    lib.oracle_compare.restype = _i64
    lib.oracle_compare_abs.argtypes = [_p, _p, _i64, C.c_double]
    lib.oracle_compare_abs.restype = _i64
    lib.oracle_half_to_float.argtypes = [_p, _p, _i64]
    lib.oracle_float_to_half.argtypes = [_p, _p, _i64]
    lib.oracle_max_threads.restype = C.c_int
    return lib


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


class Btcf:
    """Field set of the reference's BTCF_MTX_NO_BITMAP (src/utils/class.h:74-85)."""

    def __init__(self, rows, cols, nnz, row_window, col_window, rowOffset, tcA2B, data, rowIdx):
        self.rows, self.cols, self.nnzs = int(rows), int(cols), int(nnz)
        self.row_window, self.col_window = int(row_window), int(col_window)
        self.total_row_windows = (self.rows + row_window - 1) // row_window
        self.rowOffset, self.tcA2B, self.data, self.rowIdx = rowOffset, tcA2B, data, rowIdx
        self.eff_row_windows = len(rowIdx)
        self.total_tiles = int(rowOffset[-1]) if len(rowOffset) else 0


def csr2btcf_nobitmap(rows, cols, row_ptr, col_idx, values, row_window, col_window, col_major_tiles=False) -> Btcf:
    """Restated CSR2BTCFNOBITMAP (convert.h:146-225) with run-time window shape."""
    row_ptr = _c(row_ptr, np.uint32)
    col_idx = _c(col_idx, np.uint32)
    values = np.ascontiguousarray(values)
    assert values.dtype in (np.float16, np.float32, np.uint16)
    eff, tiles = _i64(), _i64()
    rc = lib().oracle_btcf_count(rows, _ptr(row_ptr), _ptr(col_idx), row_window, col_window, C.byref(eff),
                                 C.byref(tiles))
    assert rc == 0
    eff, tiles = eff.value, tiles.value
    rowOffset = np.zeros(eff + 1, np.uint32)
    tcA2B = np.zeros(tiles * col_window, np.uint32)
    data = np.zeros(tiles * row_window * col_window, values.dtype)
    rowIdx = np.zeros(eff, np.uint32)
    rc = lib().oracle_csr2btcf_nobitmap(rows, _ptr(row_ptr), _ptr(col_idx), _ptr(values), values.dtype.itemsize,
                                        row_window, col_window, int(bool(col_major_tiles)), _ptr(rowOffset),
                                        _ptr(tcA2B), _ptr(data), _ptr(rowIdx))
    assert rc == 0
    return Btcf(rows, cols, len(col_idx), row_window, col_window, rowOffset, tcA2B, data, rowIdx)


def spmm_csr(rows, row_ptr, col_idx, values, B, n_threads=1, tf32_mode=0, row_begin=0, row_end=None) -> np.ndarray:
    """O1: direct CSR SpMM in the reference verifiers' arithmetic; returns fp32 C [rows, N]."""
    row_ptr = _c(row_ptr, np.uint32)
    col_idx = _c(col_idx, np.uint32)
    B = np.ascontiguousarray(B)
    n = B.shape[1]
    out = np.zeros((rows, n), np.float32)
    row_end = rows if row_end is None else row_end
    if B.dtype == np.float16:
        values = _c(values, np.float16)
        lib().oracle_spmm_csr_f16(rows, _ptr(row_ptr), _ptr(col_idx), _ptr(values), _ptr(B), B.shape[1], n,
                                  _ptr(out), n, row_begin, row_end, n_threads)
    else:
        values = _c(values, np.float32)
        B = _c(B, np.float32)
        lib().oracle_spmm_csr_f32(rows, _ptr(row_ptr), _ptr(col_idx), _ptr(values), _ptr(B), B.shape[1], n,
                                  _ptr(out), n, row_begin, row_end, tf32_mode, n_threads)
    return out


def spmm_btcf(f: Btcf, B, tf32_mode=0, n_threads=0) -> np.ndarray:
    """O2: verify_result's loop nest (tf32.cu:20-28) over the converted format."""
    B = np.ascontiguousarray(B)
    n = B.shape[1]
    out = np.zeros((f.rows, n), np.float32)
    is_half = int(B.dtype == np.float16)
    lib().oracle_spmm_btcf(f.rows, f.eff_row_windows, _ptr(f.rowOffset), _ptr(f.tcA2B), _ptr(f.data),
                           _ptr(f.rowIdx), is_half, f.row_window, f.col_window, _ptr(B), B.shape[1], n, _ptr(out),
                           n, tf32_mode, n_threads)
    return out


def tile_accumulate(A, B, tile_m, tile_n, tile_k, tile_num) -> np.ndarray:
    A, B = _c(A, np.float32), _c(B, np.float32)
    out = np.zeros((tile_m, tile_n), np.float32)
    lib().oracle_tile_accumulate(_ptr(A), _ptr(B), _ptr(out), tile_m, tile_n, tile_k, tile_num)
    return out


def rand_fill(seed: int, n: int) -> np.ndarray:
    out = np.zeros(n, np.float32)
    lib().oracle_rand_fill(seed, _ptr(out), n)
    return out


def compare(got, ref, rel_tol):
    """verify_result's rule (tf32.cu:38-71). Returns (n_bad, max_rel, max_abs)."""
    got, ref = _c(got, np.float32), _c(ref, np.float32)
    assert got.shape == ref.shape and got.ndim == 2
    mr, ma = C.c_double(), C.c_double()
    bad = lib().oracle_compare(_ptr(got), _ptr(ref), got.shape[0], got.shape[1], got.shape[1], ref.shape[1],
                               rel_tol, C.byref(mr), C.byref(ma))
    return int(bad), mr.value, ma.value


def compare_abs(a, b, abs_tol=1.0) -> int:
    a, b = _c(a, np.float32), _c(b, np.float32)
    return int(lib().oracle_compare_abs(_ptr(a), _ptr(b), a.size, abs_tol))


def half_to_float(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.zeros(h.shape, np.float32)
    lib().oracle_half_to_float(_ptr(h), _ptr(out), h.size)
    return out


def float_to_half(f) -> np.ndarray:
    f = _c(f, np.float32)
    out = np.zeros(f.shape, np.uint16)
    lib().oracle_float_to_half(_ptr(f), _ptr(out), f.size)
    return out


# ------------------------------------------------------------------ reference harness


def ref_available(flavour: str) -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", f"libref_{flavour}.so"))


def ref_convert(flavour: str, rows, cols, row_ptr, col_idx, values) -> Btcf:
    """Run the reference's own CSR2BTCFNOBITMAP (8x16 for 'fp16', 8x8 for 'tf32')."""
    r = C.CDLL(os.path.join(_HERE, "_ref", f"libref_{flavour}.so"))
    r.ref_convert.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, _p, _p, _p, _p]
    r.ref_fetch.argtypes = [_p, _p, _p, _p]
    row_ptr, col_idx = _c(row_ptr, np.uint32), _c(col_idx, np.uint32)
    dt = np.float16 if flavour == "fp16" else np.float32
    values = _c(values, dt)
    assert r.ref_elt_size() == values.dtype.itemsize
    sizes = np.zeros(5, np.uint64)
    r.ref_convert(rows, cols, len(col_idx), _ptr(row_ptr), _ptr(col_idx), _ptr(values), _ptr(sizes))
    eff, tiles, _, n_a2b, n_data = (int(x) for x in sizes)
    rowOffset = np.zeros(eff + 1, np.uint32)
    tcA2B = np.zeros(n_a2b, np.uint32)
    data = np.zeros(n_data, dt)
    rowIdx = np.zeros(eff, np.uint32)
    r.ref_fetch(_ptr(rowOffset), _ptr(tcA2B), _ptr(data), _ptr(rowIdx))
    rw, cw = r.ref_row_window(), r.ref_col_window()
    r.ref_release()
    out = Btcf(rows, cols, len(col_idx), rw, cw, rowOffset, tcA2B, data, rowIdx)
    assert out.total_tiles == tiles
    return out


# ------------------------------------------------------------------ bitmap and group formats


class BtcfBitmap:
    """Field set of the reference's BTCF_MTX (src/utils/class.h:55-67)."""

    def __init__(self, row_window, col_window, rowOffset, nnzOffset, tcA2B, tcBit, data, rowIdx):
        self.row_window, self.col_window = int(row_window), int(col_window)
        self.rowOffset, self.nnzOffset, self.tcA2B, self.tcBit = rowOffset, nnzOffset, tcA2B, tcBit
        self.data, self.rowIdx = data, rowIdx
        self.eff_row_windows = len(rowIdx)
        self.total_tiles = int(rowOffset[-1]) if len(rowOffset) else 0


def csr2btcf_bitmap(rows, row_ptr, col_idx, values, row_window, col_window, legacy_word_index=False) -> BtcfBitmap:
    """Restated CSR2BTCF (convert.h:22-139); legacy_word_index repeats the reference's fp16 bitmap
    word addressing (convert.h:98-102) for the comparison with the reference itself."""
    row_ptr, col_idx = _c(row_ptr, np.uint32), _c(col_idx, np.uint32)
    values = np.ascontiguousarray(values)
    eff, tiles = _i64(), _i64()
    assert lib().oracle_btcf_count(rows, _ptr(row_ptr), _ptr(col_idx), row_window, col_window, C.byref(eff),
                                   C.byref(tiles)) == 0
    eff, tiles, words = eff.value, tiles.value, row_window * col_window // 64
    rowOffset, nnzOffset = np.zeros(eff + 1, np.uint32), np.zeros(tiles + 1, np.uint32)
    tcA2B, tcBit = np.zeros(tiles * col_window, np.uint32), np.zeros(tiles * words, np.uint64)
    data, rowIdx = np.zeros(len(col_idx), values.dtype), np.zeros(eff, np.uint32)
    fn = lib().oracle_csr2btcf_bitmap
    fn.argtypes = [C.c_int64, _p, _p, _p, C.c_int, C.c_int, C.c_int, C.c_int, _p, _p, _p, _p, _p, _p]
    assert fn(rows, _ptr(row_ptr), _ptr(col_idx), _ptr(values), values.dtype.itemsize, row_window, col_window,
              int(bool(legacy_word_index)), _ptr(rowOffset), _ptr(nnzOffset), _ptr(tcA2B), _ptr(tcBit), _ptr(data),
              _ptr(rowIdx)) == 0
    return BtcfBitmap(row_window, col_window, rowOffset, nnzOffset, tcA2B, tcBit, data, rowIdx)


def btcf2gbtcf(rowOffset, rowIdx):
    """Restated BTCF2GBTCF (convert.h:232-276): (groupOffset, rowIdx, atomic, group_len)."""
    rowOffset, rowIdx = _c(rowOffset, np.uint32), _c(rowIdx, np.uint32)
    fn = lib().oracle_btcf2gbtcf
    fn.argtypes = [_p, _p, C.c_int64, _p, _p, _p, C.POINTER(C.c_int64), C.POINTER(C.c_uint32)]
    groups, length = C.c_int64(), C.c_uint32()
    assert fn(_ptr(rowOffset), _ptr(rowIdx), len(rowIdx), None, None, None, C.byref(groups), C.byref(length)) == 0
    go, gr, at = np.zeros(groups.value + 1, np.uint32), np.zeros(groups.value, np.uint32), np.zeros(groups.value, np.uint8)
    assert fn(_ptr(rowOffset), _ptr(rowIdx), len(rowIdx), _ptr(go), _ptr(gr), _ptr(at), C.byref(groups),
              C.byref(length)) == 0
    return go, gr, at, int(length.value)


_MTX_ENTRY = None


def load_matrix_text(text: str, dtype=np.float16):
    """Restated load_matrix (load.h:152-322) over the file's text: (rows, cols, row_ptr, col_idx,
    values).  Pure Python, for small files."""
    import re
    global _MTX_ENTRY
    if _MTX_ENTRY is None:
        num = r"[+-]?(?:\d+\.?\d*(?:[eE][+-]?\d+)?|\.\d+(?:[eE][+-]?\d+)?|inf(?:inity)?|nan)"
        _MTX_ENTRY = re.compile(r"^\s*\+?(\d+)\s+\+?(\d+)\s+(" + num + ")", re.IGNORECASE)
    lines = text.split("\n")
    k = 0
    while k < len(lines) and lines[k].startswith("%"):  # load.h:189-193
        k += 1
    rows, cols, declared = (int(x) for x in lines[k].split()[:3])  # load.h:196
    entries = []
    for line in lines[k + 1:]:
        if len(entries) >= declared:  # load.h:214
            break
        m = _MTX_ENTRY.match(line)
        if m:  # other lines are ignored (load.h:218)
            entries.append((int(m.group(1)) - 1, int(m.group(2)) - 1, float(m.group(3))))
    order = sorted(range(len(entries)), key=lambda i: (entries[i][0], entries[i][1]))  # load.h:256
    row_ptr = np.zeros(rows + 1, np.uint32)
    for r, _, _ in entries:
        row_ptr[r + 1] += 1
    row_ptr = np.cumsum(row_ptr, dtype=np.uint64).astype(np.uint32)
    col_idx = np.array([entries[i][1] for i in order], np.uint32)
    values = np.array([entries[i][2] for i in order], np.float32).astype(dtype)  # fp16: round to nearest even (load.h:225)
    return rows, cols, row_ptr, col_idx, values


def _ref_lib(flavour: str):
    return C.CDLL(os.path.join(_HERE, "_ref", f"libref_{flavour}.so"))


def ref_convert_bitmap(flavour: str, rows, cols, row_ptr, col_idx, values):
    """The reference's own CSR2BTCF followed by its BTCF2GBTCF: (BtcfBitmap, (groupOffset, rowIdx, atomic))."""
    r = _ref_lib(flavour)
    r.ref_convert_bitmap.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, _p, _p, _p, _p]
    r.ref_fetch_bitmap.argtypes = [_p] * 6
    r.ref_group.argtypes = [_p]
    r.ref_fetch_groups.argtypes = [_p] * 3
    row_ptr, col_idx = _c(row_ptr, np.uint32), _c(col_idx, np.uint32)
    dt = np.float16 if flavour == "fp16" else np.float32
    values = _c(values, dt)
    assert r.ref_map_word_size() == 8
    sizes = np.zeros(5, np.uint64)
    r.ref_convert_bitmap(rows, cols, len(col_idx), _ptr(row_ptr), _ptr(col_idx), _ptr(values), _ptr(sizes))
    eff, n_off, n_a2b, n_bit, n_data = (int(x) for x in sizes)
    rowOffset, nnzOffset = np.zeros(eff + 1, np.uint32), np.zeros(n_off, np.uint32)
    tcA2B, tcBit = np.zeros(n_a2b, np.uint32), np.zeros(n_bit, np.uint64)
    data, rowIdx = np.zeros(n_data, dt), np.zeros(eff, np.uint32)
    assert r.ref_fetch_bitmap(_ptr(rowOffset), _ptr(nnzOffset), _ptr(tcA2B), _ptr(tcBit), _ptr(data), _ptr(rowIdx)) == 0
    groups = np.zeros(1, np.uint64)
    assert r.ref_group(_ptr(groups)) == 0
    g = int(groups[0])
    go, gr, at = np.zeros(g + 1, np.uint32), np.zeros(g, np.uint32), np.zeros(g, np.uint8)
    assert r.ref_fetch_groups(_ptr(go), _ptr(gr), _ptr(at)) == 0
    return (BtcfBitmap(r.ref_row_window(), r.ref_col_window(), rowOffset, nnzOffset, tcA2B, tcBit, data, rowIdx),
            (go, gr, at))


def ref_load_matrix(flavour: str, path: str):
    """The reference's own load_matrix: (rows, cols, row_ptr, col_idx, values)."""
    r = _ref_lib(flavour)
    r.ref_load.argtypes = [C.c_char_p, _p]
    r.ref_fetch_loaded.argtypes = [_p] * 3
    dims = np.zeros(3, np.uint32)
    assert r.ref_load(path.encode(), _ptr(dims)) == 0
    rows, cols, nnz = (int(x) for x in dims)
    dt = np.float16 if flavour == "fp16" else np.float32
    row_ptr, col_idx, values = np.zeros(rows + 1, np.uint32), np.zeros(nnz, np.uint32), np.zeros(nnz, dt)
    assert r.ref_fetch_loaded(_ptr(row_ptr), _ptr(col_idx), _ptr(values)) == 0
    return rows, cols, row_ptr, col_idx, values
