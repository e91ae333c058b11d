"""Host-side mirror of the reference's operator interface, over the C ABI.

Names and argument meaning follow the reference (Ritt2020/hopper_spmm):

    CSR_MTX / DENSE_MTX / BTCF_MTX_NO_BITMAP      src/utils/class.h:30-85
    CSR2BTCFNOBITMAP(csr, btcf)                    src/utils/convert.h:146-225
    fp16_spmm(btcf, B, C) -> PERF_RESULT           src/fp16.cu:221-281
    tf32_spmm(btcf, B, C) -> PERF_RESULT           (src/tf32.cu has no operator; same shape)
    PERF_RESULT, WARMUP_RUNS, RUNS                 src/common.h:48-59

Everything that computes runs inside libb200spmm.so; torch is used only to hold device
memory and to name the stream.  There is no CPU path: without the library or without an
sm_100 device the calls raise.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _capi as capi

WARMUP_RUNS = 3  # src/common.h:48
RUNS = 5         # src/common.h:49
ROW_WINDOW = 16  # the sm_100a kernels consume 16-row windows (the reference's macro is 8)
IDX_MAX = 0xFFFFFFFF


@dataclass
class PERF_RESULT:
    """src/common.h:51-59."""
    time: float  # ms over all runs
    runs: int

    def print(self):
        print(f"SPMM total: {self.time:.3f} ms, runs: {self.runs}, average: {self.time / self.runs:.3f} ms")


class CSR_MTX:
    """src/utils/class.h:30-37.  values: float16 (fp16 path) or float32 (tf32 path)."""

    def __init__(self, rows, cols, row_ptr, col_idx, values):
        self.rows, self.cols = int(rows), int(cols)
        self.row_ptr = np.ascontiguousarray(row_ptr, dtype=np.uint32)
        self.col_idx = np.ascontiguousarray(col_idx, dtype=np.uint32)
        self.values = np.ascontiguousarray(values)
        if self.values.dtype not in (np.float16, np.float32):
            raise TypeError("values must be float16 or float32")
        self.nnzs = int(self.col_idx.size)


class DENSE_MTX:
    """src/utils/class.h:44-48: row-major rows x cols host array."""

    def __init__(self, rows, cols, values=None, dtype=np.float32):
        self.rows, self.cols = int(rows), int(cols)
        self.values = (np.zeros((self.rows, self.cols), dtype) if values is None
                       else np.ascontiguousarray(values).reshape(self.rows, self.cols))


def _dtype_code(np_dtype) -> int:
    return capi.F16 if np_dtype == np.float16 else capi.TF32


class BTCF_MTX_NO_BITMAP:
    """src/utils/class.h:74-85, filled by CSR2BTCFNOBITMAP.  The arrays are read-only numpy
    views of memory owned by the library."""

    def __init__(self):
        self._h = None
        self.rows = self.cols = self.nnzs = 0
        self.total_row_windows = self.eff_row_windows = self.total_tiles = 0
        self.row_window, self.col_window = ROW_WINDOW, 0
        self.rowOffset = self.tcA2B = self.data = self.rowIdx = None
        self.dtype = None
        self.col_major_tiles = False

    def _adopt(self, handle):
        lib = capi.lib()
        self._h = handle
        info = capi.BtcfInfo()
        capi.check(lib.b200spmm_btcf_info(handle, C.byref(info)), "b200spmm_btcf_info")
        self.rows, self.cols, self.nnzs = info.rows, info.cols, info.nnzs
        self.total_row_windows, self.eff_row_windows = info.total_row_windows, info.eff_row_windows
        self.total_tiles = info.total_tiles
        self.row_window, self.col_window = info.row_window, info.col_window
        self.dtype = np.float16 if info.dtype == capi.F16 else np.float32

        def view(ptr, count, dt):
            if count == 0:
                return np.zeros(0, dt)
            buf = (C.c_char * (count * np.dtype(dt).itemsize)).from_address(ptr)
            a = np.frombuffer(buf, dtype=dt, count=count)
            a.flags.writeable = False
            return a

        self.rowOffset = view(lib.b200spmm_btcf_rowOffset(handle), self.eff_row_windows + 1, np.uint32)
        self.tcA2B = view(lib.b200spmm_btcf_tcA2B(handle), self.total_tiles * self.col_window, np.uint32)
        self.data = view(lib.b200spmm_btcf_data(handle), self.total_tiles * self.row_window * self.col_window,
                         self.dtype)
        self.rowIdx = view(lib.b200spmm_btcf_rowIdx(handle), self.eff_row_windows, np.uint32)

    def __del__(self):
        if getattr(self, "_h", None):
            self.rowOffset = self.tcA2B = self.data = self.rowIdx = None
            try:
                capi.lib().b200spmm_btcf_destroy(self._h)
            except Exception:  # interpreter shutdown
                pass
            self._h = None


def transpose_tiles(btcf: BTCF_MTX_NO_BITMAP) -> BTCF_MTX_NO_BITMAP:
    """Rewrites the tiles of ``btcf`` in place from row-major to column-major storage or back: what the
    reference's SPARSE_A_TRANSPOSE build stores (src/utils/convert.h:207-213).  ``btcf.col_major_tiles`` says
    which it holds; the kernels (and SpmmPlan) take row-major tiles only."""
    capi.check(capi.lib().b200spmm_btcf_transpose_tiles(btcf._h), "b200spmm_btcf_transpose_tiles")
    btcf.col_major_tiles = bool(capi.lib().b200spmm_btcf_tiles_col_major(btcf._h))
    return btcf


def CSR2BTCFNOBITMAP(csr: CSR_MTX, btcf: BTCF_MTX_NO_BITMAP | None = None, row_window: int = ROW_WINDOW,
                     col_window: int = 0, n_threads: int = 0) -> BTCF_MTX_NO_BITMAP:
    """src/utils/convert.h:146-225.  Fills (and returns) ``btcf``; like the reference it expects
    a fresh struct.  col_window 0 = the reference's choice for the element type (16 / 8)."""
    btcf = btcf if btcf is not None else BTCF_MTX_NO_BITMAP()
    if btcf._h is not None:
        raise ValueError("CSR2BTCFNOBITMAP expects a fresh BTCF_MTX_NO_BITMAP")
    h = C.c_void_p()
    st = capi.lib().b200spmm_csr2btcf_nobitmap(
        csr.rows, csr.cols, csr.nnzs, csr.row_ptr.ctypes.data, csr.col_idx.ctypes.data, csr.values.ctypes.data,
        _dtype_code(csr.values.dtype), row_window, col_window, n_threads, C.byref(h))
    capi.check(st, "b200spmm_csr2btcf_nobitmap")
    btcf._adopt(h)
    return btcf


def rewindow(rows: int, cols: int, nnzs: int, rowOffset, tcA2B, data, rowIdx, row_window_in: int = 8,
             row_window: int = ROW_WINDOW, n_threads: int = 0) -> BTCF_MTX_NO_BITMAP:
    """A BTCF_MTX_NO_BITMAP given as its arrays - e.g. one the reference's own CSR2BTCFNOBITMAP built
    with its fixed 8-row windows (src/common.h:17, src/utils/convert.h:146-225) - brought to the
    ``row_window`` the kernels consume.  Bit-identical to converting the matrix at that height."""
    data = np.ascontiguousarray(data)
    if data.dtype not in (np.float16, np.float32):
        raise TypeError("data must be float16 or float32")
    rowOffset = np.ascontiguousarray(rowOffset, np.uint32)
    tcA2B = np.ascontiguousarray(tcA2B, np.uint32)
    rowIdx = np.ascontiguousarray(rowIdx, np.uint32)
    if rowOffset.size < 1 or rowIdx.size != rowOffset.size - 1:
        raise ValueError("rowOffset holds one entry more than rowIdx")
    tiles = int(rowOffset[-1])
    if tiles and (tcA2B.size % tiles or data.size != tiles * row_window_in * (tcA2B.size // tiles)):
        raise ValueError("tcA2B and data do not describe rowOffset[-1] tiles of row_window_in rows")
    info = capi.BtcfInfo()
    info.rows, info.cols, info.nnzs = rows, cols, nnzs
    info.total_row_windows = (rows + row_window_in - 1) // row_window_in
    info.eff_row_windows, info.total_tiles = rowIdx.size, tiles
    info.row_window = row_window_in
    info.col_window = tcA2B.size // tiles if tiles else (16 if data.dtype == np.float16 else 8)
    info.dtype, info.elt_size = _dtype_code(data.dtype), data.dtype.itemsize
    h = C.c_void_p()
    st = capi.lib().b200spmm_btcf_rewindow(C.byref(info), rowOffset.ctypes.data, tcA2B.ctypes.data, data.ctypes.data,
                                           rowIdx.ctypes.data, row_window, n_threads, C.byref(h))
    capi.check(st, "b200spmm_btcf_rewindow")
    out = BTCF_MTX_NO_BITMAP()
    out._adopt(h)
    return out


class DeviceBtcf:
    """BTCF_MTX_NO_BITMAP (src/utils/class.h:74-85) resident on the GPU, made by the device-side
    converter from CSR tensors that already live there."""

    def __init__(self, rows, cols, row_ptr, col_idx, values, row_window: int = ROW_WINDOW, col_window: int = 0,
                 device: int = 0):
        """row_ptr / col_idx: CUDA int32 tensors (bit patterns of uint32), values: CUDA float16 or
        float32; columns ascending and distinct inside every row."""
        import torch
        if not (row_ptr.is_cuda and col_idx.is_cuda and values.is_cuda):
            raise ValueError("DeviceBtcf takes CUDA tensors")
        if row_ptr.dtype != torch.int32 or col_idx.dtype != torch.int32 or values.dtype not in (torch.float16, torch.float32):
            raise TypeError("row_ptr/col_idx must be int32, values float16 or float32")
        lib = capi.lib()
        self._h = C.c_void_p()
        dtype = capi.F16 if values.dtype == torch.float16 else capi.TF32
        s = torch.cuda.current_stream(values.device).cuda_stream
        st = lib.b200spmm_csr2btcf_nobitmap_device(rows, cols, col_idx.numel(), row_ptr.data_ptr(), col_idx.data_ptr(),
                                                   values.data_ptr(), dtype, row_window, col_window, device, s,
                                                   C.byref(self._h))
        capi.check(st, "b200spmm_csr2btcf_nobitmap_device")
        self.info = capi.BtcfInfo()
        capi.check(lib.b200spmm_dbtcf_info(self._h, C.byref(self.info)), "b200spmm_dbtcf_info")
        self.device = device
        self.dtype = np.float16 if dtype == capi.F16 else np.float32
        for k in ("rows", "cols", "nnzs", "total_row_windows", "eff_row_windows", "total_tiles", "row_window",
                  "col_window"):
            setattr(self, k, getattr(self.info, k))
        self.ptr = {k: getattr(lib, f"b200spmm_dbtcf_{k}")(self._h) for k in ("rowOffset", "tcA2B", "data", "rowIdx")}

    def to_host(self):
        """The four arrays copied to numpy (for comparison with the host converter)."""
        cw, rw = self.col_window, self.row_window
        out = {"rowOffset": np.zeros(self.eff_row_windows + 1, np.uint32),
               "tcA2B": np.zeros(self.total_tiles * cw, np.uint32),
               "data": np.zeros(self.total_tiles * rw * cw, self.dtype),
               "rowIdx": np.zeros(self.eff_row_windows, np.uint32)}
        capi.check(capi.lib().b200spmm_dbtcf_copy_to_host(self._h, *(out[k].ctypes.data if out[k].size else
                                                                     np.zeros(1, np.uint32).ctypes.data
                                                                     for k in ("rowOffset", "tcA2B", "data", "rowIdx"))),
                   "b200spmm_dbtcf_copy_to_host")
        return out

    def close(self):
        if getattr(self, "_h", None):
            capi.lib().b200spmm_dbtcf_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_rows(rows: int, row_ptr, parts: int, row_window: int = ROW_WINDOW, row_charge: int = 0) -> np.ndarray:
    """Row cuts on window boundaries balanced on nnz + row_charge * rows: part p owns rows
    [cuts[p], cuts[p+1]).  row_charge 0 is plain nnz balance."""
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.uint32)
    cuts = np.zeros(parts + 1, np.uint64)
    capi.check(capi.lib().b200spmm_shard_rows_weighted(rows, row_ptr.ctypes.data, row_window, parts, row_charge,
                                                       cuts.ctypes.data), "b200spmm_shard_rows_weighted")
    return cuts


class SpmmPlan:
    """Device-resident matrix + persistent schedule (b200spmm_plan_*).  Replaces the
    allocate / copy / build-descriptor prologue of fp16_spmm (src/fp16.cu:236-252)."""

    def __init__(self, btcf: BTCF_MTX_NO_BITMAP | None = None, device: int = 0, n_ctas: int = 0, *,
                 device_arrays=None):
        lib = capi.lib()
        self._p = C.c_void_p()
        self._keep = device_arrays  # borrowed device tensors must outlive the plan
        if isinstance(btcf, DeviceBtcf):
            self._keep = btcf  # the plan borrows the arrays
            st = lib.b200spmm_plan_create_device(C.byref(btcf.info), btcf.ptr["rowOffset"], btcf.ptr["tcA2B"],
                                                 btcf.ptr["data"], btcf.ptr["rowIdx"], device, n_ctas, C.byref(self._p))
            capi.check(st, "b200spmm_plan_create_device")
        elif device_arrays is not None:
            info, d_rowOffset, d_tcA2B, d_data, d_rowIdx = device_arrays
            st = lib.b200spmm_plan_create_device(C.byref(info), d_rowOffset.data_ptr(), d_tcA2B.data_ptr(),
                                                 d_data.data_ptr(), d_rowIdx.data_ptr(), device, n_ctas,
                                                 C.byref(self._p))
            capi.check(st, "b200spmm_plan_create_device")
        else:
            capi.check(lib.b200spmm_plan_create(btcf._h, device, n_ctas, C.byref(self._p)), "b200spmm_plan_create")
        info = capi.BtcfInfo()
        capi.check(lib.b200spmm_plan_info(self._p, C.byref(info)), "b200spmm_plan_info")
        self.info = info
        self.device = device
        self.rows, self.cols = info.rows, info.cols
        self.is_f16 = info.dtype == capi.F16

    def close(self):
        if self._p:
            capi.lib().b200spmm_plan_destroy(self._p)
            self._p = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- device tensors (torch) ------------------------------------------------------------
    def spmm(self, B, C_out=None, c_half: bool = False, stream=None, sync: bool = True):
        """C = A @ B for a torch CUDA tensor B [cols, n]; returns C [rows, n] (fp32, or fp16)."""
        import torch
        want = torch.float16 if self.is_f16 else torch.float32
        if not B.is_cuda or B.dtype != want or B.dim() != 2 or B.stride(1) != 1 or B.shape[0] != self.cols:
            raise ValueError(f"B must be a CUDA {want} tensor of shape [{self.cols}, n] with unit column stride")
        n = B.shape[1]
        cdt = torch.float16 if c_half else torch.float32
        if C_out is None:
            C_out = torch.empty((self.rows, n), dtype=cdt, device=B.device)
        elif (not C_out.is_cuda or C_out.dtype != cdt or C_out.shape != (self.rows, n) or C_out.stride(1) != 1):
            raise ValueError("C has the wrong shape, dtype or layout")
        s = (stream or torch.cuda.current_stream(B.device)).cuda_stream
        fn = capi.lib().b200spmm_fp16_spmm if self.is_f16 else capi.lib().b200spmm_tf32_spmm
        capi.check(fn(self._p, B.data_ptr(), B.stride(0), n, C_out.data_ptr(), C_out.stride(0),
                      capi.C_F16 if c_half else capi.C_F32, s), "b200spmm_spmm")
        if sync:
            capi.check(capi.lib().b200spmm_plan_sync(self._p, s), "b200spmm_plan_sync")
        return C_out

    def sync(self, stream=None):
        import torch
        s = (stream or torch.cuda.current_stream()).cuda_stream
        capi.check(capi.lib().b200spmm_plan_sync(self._p, s), "b200spmm_plan_sync")

    def bench(self, B, C_out, warmup: int = WARMUP_RUNS, runs: int = RUNS, c_half: bool = False) -> PERF_RESULT:
        """The reference's timing protocol (src/fp16.cu:255-268) on device tensors."""
        import torch
        ms = C.c_float()
        s = torch.cuda.current_stream(B.device).cuda_stream
        capi.check(capi.lib().b200spmm_bench(self._p, B.data_ptr(), B.stride(0), B.shape[1], C_out.data_ptr(),
                                             C_out.stride(0), capi.C_F16 if c_half else capi.C_F32, warmup, runs, s,
                                             C.byref(ms)), "b200spmm_bench")
        return PERF_RESULT(ms.value, runs)

    # -- host arrays -----------------------------------------------------------------------
    def spmm_host(self, B: np.ndarray, C_out: np.ndarray | None = None, c_half: bool = False) -> np.ndarray:
        """Host-buffer form: copies B in, runs, copies C back (b200spmm_spmm_host)."""
        want = np.float16 if self.is_f16 else np.float32
        B = np.ascontiguousarray(B, dtype=want)
        if B.ndim != 2 or B.shape[0] != self.cols:
            raise ValueError(f"B must have shape [{self.cols}, n]")
        n = B.shape[1]
        cdt = np.float16 if c_half else np.float32
        if C_out is None:
            C_out = np.empty((self.rows, n), cdt)
        elif C_out.dtype != cdt or C_out.shape != (self.rows, n) or not C_out.flags.c_contiguous:
            raise ValueError("C has the wrong shape, dtype or layout")
        capi.check(capi.lib().b200spmm_spmm_host(self._p, B.ctypes.data, n, C_out.ctypes.data,
                                                 capi.C_F16 if c_half else capi.C_F32), "b200spmm_spmm_host")
        return C_out

    def tall_format(self, rows: int = 128):
        """The plan's super-window copy of the matrix as a dict of numpy arrays plus its counts, or None
        when the plan keeps none: rows=128 the one of the 128-row kernel (b200spmm_plan_tall_*), rows=256
        the one of the CTA-pair kernel (b200spmm_plan_pair_*)."""
        if rows not in (128, 256):
            raise ValueError("super-windows have 128 or 256 rows")
        kind = "tall" if rows == 128 else "pair"
        get_info = getattr(capi.lib(), f"b200spmm_plan_{kind}_info")
        copy_out = getattr(capi.lib(), f"b200spmm_plan_{kind}_copy_to_host")
        info = capi.BtcfInfo()
        capi.check(get_info(self._p, C.byref(info)), f"b200spmm_plan_{kind}_info")
        if info.row_window == 0:
            return None
        cw, dt = info.col_window, (np.float16 if self.is_f16 else np.float32)
        out = {"rowOffset": np.zeros(info.eff_row_windows + 1, np.uint32), "tcA2B": np.zeros(info.total_tiles * cw, np.uint32),
               "data": np.zeros(info.total_tiles * info.row_window * cw, dt), "rowIdx": np.zeros(info.eff_row_windows, np.uint32)}
        capi.check(copy_out(self._p, out["rowOffset"].ctypes.data, out["tcA2B"].ctypes.data, out["data"].ctypes.data,
                            out["rowIdx"].ctypes.data), f"b200spmm_plan_{kind}_copy_to_host")
        out.update(row_window=info.row_window, eff_row_windows=info.eff_row_windows, total_tiles=info.total_tiles)
        return out

    def launch_info(self) -> capi.LaunchInfo:
        li = capi.LaunchInfo()
        capi.check(capi.lib().b200spmm_plan_launch_info(self._p, C.byref(li)), "b200spmm_plan_launch_info")
        return li


class ShardedSpmm:
    """The sharded operator of the C ABI (b200spmm_sharded_*): one process, several GPUs, the matrix cut
    into time-balanced row ranges, B replicated, C row-sharded.  Host arrays in, host arrays out, like
    fp16_spmm (src/fp16.cu:221-281); the device-pointer calls are reachable through ``_s``."""

    def __init__(self, csr: CSR_MTX, devices, row_charge: int = 6):
        lib = capi.lib()
        self._s = C.c_void_p()
        devs = (C.c_int * len(devices))(*devices)
        capi.check(lib.b200spmm_sharded_create(csr.rows, csr.cols, csr.nnzs, csr.row_ptr.ctypes.data, csr.col_idx.ctypes.data,
                                               csr.values.ctypes.data, _dtype_code(csr.values.dtype), devs, len(devices),
                                               row_charge, C.byref(self._s)), "b200spmm_sharded_create")
        self.devices = list(devices)
        self.rows, self.cols = csr.rows, csr.cols
        self.dtype = csr.values.dtype
        cuts = np.zeros(len(devices) + 1, np.uint64)
        n = C.c_int()
        capi.check(lib.b200spmm_sharded_info(self._s, C.byref(n), cuts.ctypes.data), "b200spmm_sharded_info")
        self.row_begin = cuts.astype(np.int64)

    def spmm_host(self, B: np.ndarray, c_half: bool = False) -> np.ndarray:
        B = np.ascontiguousarray(B, dtype=self.dtype)
        out = np.empty((self.rows, B.shape[1]), np.float16 if c_half else np.float32)
        capi.check(capi.lib().b200spmm_spmm_sharded_host(self._s, B.ctypes.data, B.shape[1], out.ctypes.data,
                                                         capi.C_F16 if c_half else capi.C_F32), "b200spmm_spmm_sharded_host")
        return out

    def spmm_allgather(self, B_per_device, C_full_per_device):
        """Device tensors: B_per_device[p] is B on devices[p]; C_full_per_device[p] is a [rows, n] fp32 tensor
        there.  Every shard writes its rows in place, then the all-gather completes every copy."""
        n = B_per_device[0].shape[1]
        ptr = lambda xs: (C.c_void_p * len(xs))(*xs)
        dB = ptr([b.data_ptr() for b in B_per_device])
        dC = ptr([c.data_ptr() + int(self.row_begin[p]) * c.stride(0) * c.element_size() for p, c in enumerate(C_full_per_device)])
        full = ptr([c.data_ptr() for c in C_full_per_device])
        lib = capi.lib()
        capi.check(lib.b200spmm_spmm_sharded(self._s, dB, B_per_device[0].stride(0), n, dC, C_full_per_device[0].stride(0),
                                             capi.C_F32), "b200spmm_spmm_sharded")
        capi.check(lib.b200spmm_allgather_c(self._s, full, n, capi.C_F32), "b200spmm_allgather_c")
        capi.check(lib.b200spmm_sharded_sync(self._s), "b200spmm_sharded_sync")

    def close(self):
        if self._s:
            capi.lib().b200spmm_sharded_destroy(self._s)
            self._s = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _operator(btcf: BTCF_MTX_NO_BITMAP, B: DENSE_MTX, C_mtx: DENSE_MTX, want) -> PERF_RESULT:
    if btcf.dtype != want:
        raise TypeError("matrix element type does not match the operator")
    import torch
    plan = SpmmPlan(btcf)
    try:
        c_half = C_mtx.values.dtype == np.float16
        dB = torch.from_numpy(np.ascontiguousarray(B.values, dtype=want)).cuda()
        dC = torch.empty((btcf.rows, B.cols), dtype=torch.float16 if c_half else torch.float32, device="cuda")
        perf = plan.bench(dB, dC, WARMUP_RUNS, RUNS, c_half)
        C_mtx.values[...] = dC.cpu().numpy()  # the reference stops before this step (src/fp16.cu:269)
        return perf
    finally:
        plan.close()


def fp16_spmm(btcf: BTCF_MTX_NO_BITMAP, B: DENSE_MTX, C_mtx: DENSE_MTX) -> PERF_RESULT:
    """PERF_RESULT fp16_spmm(BTCF_MTX_NO_BITMAP&, DENSE_MTX& B, DENSE_MTX& C), src/fp16.cu:221-281:
    upload, 3 warm-ups, 5 timed launches, and C copied back to the host."""
    return _operator(btcf, B, C_mtx, np.float16)


def tf32_spmm(btcf: BTCF_MTX_NO_BITMAP, B: DENSE_MTX, C_mtx: DENSE_MTX) -> PERF_RESULT:
    """The tf32 operator the reference's Makefile names (Makefile:20,37) but never implemented."""
    return _operator(btcf, B, C_mtx, np.float32)
