"""The reference's other host-side formats and its file loader, over the C ABI:

  BTCF_MTX / CSR2BTCF        bitmap-compressed condensed format (src/utils/class.h:55-67,
                             src/utils/convert.h:22-139)
  GBTCF_MTX / BTCF2GBTCF     windows split into groups of tiles (src/utils/class.h:93-108,
                             src/utils/convert.h:232-276), validateBTCF2GBTCFConversion (:283)
  load_matrix                MatrixMarket coordinate text -> CSR_MTX (src/utils/load.h:152-322)
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi as capi
from .spmm import BTCF_MTX_NO_BITMAP, CSR_MTX, ROW_WINDOW, _dtype_code


def _view(ptr, count, dt):
    """Read-only numpy view of `count` elements of library-owned memory."""
    if count == 0 or not ptr:
        return np.zeros(0, dt)
    buf = (C.c_char * (count * np.dtype(dt).itemsize)).from_address(ptr)
    a = np.frombuffer(buf, dtype=dt, count=count)
    a.flags.writeable = False
    return a


class BTCF_MTX:
    """src/utils/class.h:55-67, filled by CSR2BTCF.  tcBit holds bitmap_words 64-bit words per
    tile (word j of tile t at t*bitmap_words + j); data holds the stored values only."""

    def __init__(self):
        self._h = None
        self.rows = self.cols = self.nnzs = 0
        self.total_row_windows = self.eff_row_windows = self.total_tiles = 0
        self.row_window, self.col_window, self.bitmap_words = 8, 0, 0
        self.rowOffset = self.nnzOffset = self.tcA2B = self.tcBit = self.data = self.rowIdx = None
        self.dtype = None

    def _adopt(self, handle):
        lib = capi.lib()
        self._h = handle
        info, words = capi.BtcfInfo(), C.c_int()
        capi.check(lib.b200spmm_btcfb_info(handle, C.byref(info), C.byref(words)), "b200spmm_btcfb_info")
        self.rows, self.cols, self.nnzs = info.rows, info.cols, info.nnzs
        self.total_row_windows, self.eff_row_windows = info.total_row_windows, info.eff_row_windows
        self.total_tiles = info.total_tiles
        self.row_window, self.col_window, self.bitmap_words = info.row_window, info.col_window, words.value
        self.dtype = np.float16 if info.dtype == capi.F16 else np.float32
        self.rowOffset = _view(lib.b200spmm_btcfb_rowOffset(handle), self.eff_row_windows + 1, np.uint32)
        self.nnzOffset = _view(lib.b200spmm_btcfb_nnzOffset(handle), self.total_tiles + 1, np.uint32)
        self.tcA2B = _view(lib.b200spmm_btcfb_tcA2B(handle), self.total_tiles * self.col_window, np.uint32)
        self.tcBit = _view(lib.b200spmm_btcfb_tcBit(handle), self.total_tiles * self.bitmap_words, np.uint64)
        self.data = _view(lib.b200spmm_btcfb_data(handle), self.nnzs, self.dtype)
        self.rowIdx = _view(lib.b200spmm_btcfb_rowIdx(handle), self.eff_row_windows, np.uint32)

    def expand(self) -> BTCF_MTX_NO_BITMAP:
        """The same matrix with dense tiles (what SpmmPlan takes)."""
        h = C.c_void_p()
        capi.check(capi.lib().b200spmm_btcfb_expand(self._h, C.byref(h)), "b200spmm_btcfb_expand")
        out = BTCF_MTX_NO_BITMAP()
        out._adopt(h)
        return out

    def __del__(self):
        if getattr(self, "_h", None):
            self.rowOffset = self.nnzOffset = self.tcA2B = self.tcBit = self.data = self.rowIdx = None
            try:
                capi.lib().b200spmm_btcfb_destroy(self._h)
            except Exception:  # interpreter shutdown
                pass
            self._h = None


def CSR2BTCF(csr: CSR_MTX, btcf: BTCF_MTX | None = None, row_window: int = 8, col_window: int = 0) -> BTCF_MTX:
    """src/utils/convert.h:22-139.  row_window defaults to the reference's 8; 16 gives the windows the
    SpMM kernels multiply.  Rows must hold strictly ascending columns."""
    btcf = btcf if btcf is not None else BTCF_MTX()
    if btcf._h is not None:
        raise ValueError("CSR2BTCF expects a fresh BTCF_MTX")
    h = C.c_void_p()
    st = capi.lib().b200spmm_csr2btcf(csr.rows, csr.cols, csr.nnzs, csr.row_ptr.ctypes.data, csr.col_idx.ctypes.data,
                                      csr.values.ctypes.data, _dtype_code(csr.values.dtype), row_window, col_window, 0,
                                      C.byref(h))
    capi.check(st, "b200spmm_csr2btcf")
    btcf._adopt(h)
    return btcf


class GBTCF_MTX:
    """src/utils/class.h:93-108: the group arrays; the tile arrays are those of the source format."""

    def __init__(self):
        self._h = None
        self.total_groups = 0
        self.group_len = 0
        self.groupOffset = self.rowIdx = self.atomic = None

    def __del__(self):
        if getattr(self, "_h", None):
            self.groupOffset = self.rowIdx = self.atomic = None
            try:
                capi.lib().b200spmm_gbtcf_destroy(self._h)
            except Exception:
                pass
            self._h = None


def BTCF2GBTCF(btcf, gbtcf: GBTCF_MTX | None = None) -> GBTCF_MTX:
    """src/utils/convert.h:232-276; takes a BTCF_MTX or a BTCF_MTX_NO_BITMAP (only rowOffset and
    rowIdx are read)."""
    gbtcf = gbtcf if gbtcf is not None else GBTCF_MTX()
    lib = capi.lib()
    ro = np.ascontiguousarray(btcf.rowOffset, np.uint32)
    ri = np.ascontiguousarray(btcf.rowIdx, np.uint32)
    h = C.c_void_p()
    capi.check(lib.b200spmm_btcf2gbtcf(ro.ctypes.data, ri.ctypes.data, len(ri), C.byref(h)), "b200spmm_btcf2gbtcf")
    gbtcf._h = h
    groups, length = C.c_uint64(), C.c_uint32()
    capi.check(lib.b200spmm_gbtcf_info(h, C.byref(groups), C.byref(length)), "b200spmm_gbtcf_info")
    gbtcf.total_groups, gbtcf.group_len = groups.value, length.value
    gbtcf.groupOffset = _view(lib.b200spmm_gbtcf_groupOffset(h), gbtcf.total_groups + 1, np.uint32)
    gbtcf.rowIdx = _view(lib.b200spmm_gbtcf_rowIdx(h), gbtcf.total_groups, np.uint32)
    gbtcf.atomic = _view(lib.b200spmm_gbtcf_atomic(h), gbtcf.total_groups, np.uint8)
    return gbtcf


def validateBTCF2GBTCFConversion(btcf, gbtcf) -> bool:
    """What src/utils/convert.h:283-402 set out to check (see b200spmm_gbtcf_validate)."""
    ro = np.ascontiguousarray(btcf.rowOffset, np.uint32)
    ri = np.ascontiguousarray(btcf.rowIdx, np.uint32)
    go = np.ascontiguousarray(gbtcf.groupOffset, np.uint32)
    gr = np.ascontiguousarray(gbtcf.rowIdx, np.uint32)
    at = np.ascontiguousarray(gbtcf.atomic, np.uint8)
    bad = C.c_uint64()
    st = capi.lib().b200spmm_gbtcf_validate(ro.ctypes.data, ri.ctypes.data, len(ri), go.ctypes.data, gr.ctypes.data,
                                            at.ctypes.data, len(gr), C.byref(bad))
    if st not in (capi.OK, capi.ERR_BAD_CSR):
        capi.check(st, "b200spmm_gbtcf_validate")
    return st == capi.OK


def load_matrix(filename: str, dtype=np.float16) -> CSR_MTX:
    """src/utils/load.h:152-322: MatrixMarket coordinate text -> CSR_MTX with fp16 (default, as the
    reference's fp16 build) or fp32 values."""
    lib = capi.lib()
    h = C.c_void_p()
    capi.check(lib.b200spmm_load_matrix(filename.encode(), _dtype_code(np.dtype(dtype)), C.byref(h)), "b200spmm_load_matrix")
    try:
        rows, cols, nnz, declared = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        capi.check(lib.b200spmm_csr_info(h, C.byref(rows), C.byref(cols), C.byref(nnz), C.byref(declared)), "b200spmm_csr_info")
        rp = _view(lib.b200spmm_csr_row_ptr(h), rows.value + 1, np.uint32).copy()
        ci = _view(lib.b200spmm_csr_col_idx(h), nnz.value, np.uint32).copy()
        v = _view(lib.b200spmm_csr_values(h), nnz.value, np.dtype(dtype)).copy()
    finally:
        lib.b200spmm_csr_destroy(h)
    m = CSR_MTX(rows.value, cols.value, rp, ci, v)
    m.declared_nnzs = declared.value
    return m
