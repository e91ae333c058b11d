"""ctypes declarations for include/b200_spmm.h and include/b200_spmm_kat.h."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200spmm.so")

OK = 0
ERR_INVALID_ARG, ERR_BAD_CSR, ERR_UNSUPPORTED, ERR_NO_MEMORY, ERR_CUDA, ERR_NO_DEVICE, ERR_DEVICE_TIMEOUT = (
    -1, -2, -3, -4, -5, -6, -7)
F16, TF32 = 0, 1
C_F32, C_F16 = 0, 1

u64, i64, u32, i32, vp = C.c_uint64, C.c_int64, C.c_uint32, C.c_int32, C.c_void_p


class BtcfInfo(C.Structure):
    _fields_ = [("rows", u64), ("cols", u64), ("nnzs", u64), ("total_row_windows", u64), ("eff_row_windows", u64),
                ("total_tiles", u64), ("row_window", i32), ("col_window", i32), ("dtype", i32), ("elt_size", i32)]


class LaunchInfo(C.Structure):
    _fields_ = [("n_ctas", i32), ("threads", i32), ("stages", i32), ("feature_slab", i32), ("n_slabs", i32),
                ("smem_bytes", i64), ("kernel_launches", i64), ("tma_gather", i32), ("bitmap_tiles", i32),
                ("row_window", i32)]


class KatMma(C.Structure):
    _fields_ = [(n, u32) for n in ("a_off", "a_lbo", "a_sbo", "a_swizzle", "b_off", "b_lbo", "b_sbo", "b_swizzle",
                                   "idesc", "d_col", "accumulate", "kind")]


# name -> (restype, argtypes); every symbol the two headers declare
SIGNATURES = {
    "b200spmm_status_string": (C.c_char_p, [C.c_int]),
    "b200spmm_last_cuda_error": (C.c_char_p, []),
    "b200spmm_version": (C.c_int, []),
    "b200spmm_csr2btcf_nobitmap": (C.c_int, [u64, u64, u64, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                              C.POINTER(vp)]),
    "b200spmm_btcf_info": (C.c_int, [vp, C.POINTER(BtcfInfo)]),
    "b200spmm_btcf_rowOffset": (vp, [vp]),
    "b200spmm_btcf_tcA2B": (vp, [vp]),
    "b200spmm_btcf_data": (vp, [vp]),
    "b200spmm_btcf_rowIdx": (vp, [vp]),
    "b200spmm_btcf_destroy": (None, [vp]),
    "b200spmm_btcf_rewindow": (C.c_int, [C.POINTER(BtcfInfo), vp, vp, vp, vp, C.c_int, C.c_int, C.POINTER(vp)]),
    "b200spmm_csr2btcf_nobitmap_device": (C.c_int, [u64, u64, u64, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp,
                                                    C.POINTER(vp)]),
    "b200spmm_dbtcf_info": (C.c_int, [vp, C.POINTER(BtcfInfo)]),
    "b200spmm_dbtcf_rowOffset": (vp, [vp]),
    "b200spmm_dbtcf_tcA2B": (vp, [vp]),
    "b200spmm_dbtcf_data": (vp, [vp]),
    "b200spmm_dbtcf_rowIdx": (vp, [vp]),
    "b200spmm_dbtcf_copy_to_host": (C.c_int, [vp, vp, vp, vp, vp]),
    "b200spmm_dbtcf_destroy": (None, [vp]),
    "b200spmm_csr2btcf": (C.c_int, [u64, u64, u64, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
    "b200spmm_btcfb_info": (C.c_int, [vp, C.POINTER(BtcfInfo), C.POINTER(C.c_int)]),
    "b200spmm_btcfb_rowOffset": (vp, [vp]),
    "b200spmm_btcfb_nnzOffset": (vp, [vp]),
    "b200spmm_btcfb_tcA2B": (vp, [vp]),
    "b200spmm_btcfb_tcBit": (vp, [vp]),
    "b200spmm_btcfb_data": (vp, [vp]),
    "b200spmm_btcfb_rowIdx": (vp, [vp]),
    "b200spmm_btcfb_destroy": (None, [vp]),
    "b200spmm_btcfb_expand": (C.c_int, [vp, C.POINTER(vp)]),
    "b200spmm_btcf2gbtcf": (C.c_int, [vp, vp, u64, C.POINTER(vp)]),
    "b200spmm_gbtcf_info": (C.c_int, [vp, C.POINTER(u64), C.POINTER(u32)]),
    "b200spmm_gbtcf_groupOffset": (vp, [vp]),
    "b200spmm_gbtcf_rowIdx": (vp, [vp]),
    "b200spmm_gbtcf_atomic": (vp, [vp]),
    "b200spmm_gbtcf_destroy": (None, [vp]),
    "b200spmm_gbtcf_validate": (C.c_int, [vp, vp, u64, vp, vp, vp, u64, C.POINTER(u64)]),
    "b200spmm_load_matrix": (C.c_int, [C.c_char_p, C.c_int, C.POINTER(vp)]),
    "b200spmm_csr_info": (C.c_int, [vp, C.POINTER(u64), C.POINTER(u64), C.POINTER(u64), C.POINTER(u64)]),
    "b200spmm_csr_row_ptr": (vp, [vp]),
    "b200spmm_csr_col_idx": (vp, [vp]),
    "b200spmm_csr_values": (vp, [vp]),
    "b200spmm_csr_destroy": (None, [vp]),
    "b200spmm_shard_rows": (C.c_int, [u64, vp, C.c_int, C.c_int, vp]),
    "b200spmm_shard_rows_weighted": (C.c_int, [u64, vp, C.c_int, C.c_int, u64, vp]),
    "b200spmm_sharded_create": (C.c_int, [u64, u64, u64, vp, vp, vp, C.c_int, vp, C.c_int, u64, C.POINTER(vp)]),
    "b200spmm_sharded_info": (C.c_int, [vp, C.POINTER(C.c_int), vp]),
    "b200spmm_sharded_stream": (vp, [vp, C.c_int]),
    "b200spmm_spmm_sharded": (C.c_int, [vp, vp, i64, i64, vp, i64, C.c_int]),
    "b200spmm_sharded_sync": (C.c_int, [vp]),
    "b200spmm_spmm_sharded_host": (C.c_int, [vp, vp, i64, vp, C.c_int]),
    "b200spmm_allgather_c": (C.c_int, [vp, vp, i64, C.c_int]),
    "b200spmm_sharded_destroy": (None, [vp]),
    "b200spmm_build_schedule": (C.c_int, [vp, u64, C.c_int, vp]),
    "b200spmm_build_tile_schedule": (C.c_int, [vp, u64, C.c_int, vp, vp, vp, vp]),
    "b200spmm_build_row_bands": (C.c_int, [vp, vp, u64, u64, C.c_int, C.c_int, vp, vp, C.POINTER(C.c_int)]),
    "b200spmm_plan_create": (C.c_int, [vp, C.c_int, C.c_int, C.POINTER(vp)]),
    "b200spmm_plan_create_device": (C.c_int, [C.POINTER(BtcfInfo), vp, vp, vp, vp, C.c_int, C.c_int, C.POINTER(vp)]),
    "b200spmm_plan_destroy": (None, [vp]),
    "b200spmm_plan_info": (C.c_int, [vp, C.POINTER(BtcfInfo)]),
    "b200spmm_spmm": (C.c_int, [vp, vp, i64, i64, vp, i64, C.c_int, vp]),
    "b200spmm_fp16_spmm": (C.c_int, [vp, vp, i64, i64, vp, i64, C.c_int, vp]),
    "b200spmm_tf32_spmm": (C.c_int, [vp, vp, i64, i64, vp, i64, C.c_int, vp]),
    "b200spmm_plan_sync": (C.c_int, [vp, vp]),
    "b200spmm_spmm_host": (C.c_int, [vp, vp, i64, vp, C.c_int]),
    "b200spmm_bench": (C.c_int, [vp, vp, i64, i64, vp, i64, C.c_int, C.c_int, C.c_int, vp, C.POINTER(C.c_float)]),
    "b200spmm_spmm_noalloc": (C.c_int, [C.POINTER(BtcfInfo), vp, vp, vp, vp, vp, i64, i64, vp, i64, C.c_int, C.c_int,
                                        C.c_int, vp]),
    "b200spmm_spmm_noalloc_status": (C.c_int, [C.c_int, vp]),
    "b200spmm_allgather_plan": (C.c_int, [vp, C.c_int, vp, vp]),
    "b200spmm_btcf_transpose_tiles": (C.c_int, [vp]),
    "b200spmm_btcf_tiles_col_major": (C.c_int, [vp]),
    "b200spmm_plan_tall_info": (C.c_int, [vp, C.POINTER(BtcfInfo)]),
    "b200spmm_plan_tall_copy_to_host": (C.c_int, [vp, vp, vp, vp, vp]),
    "b200spmm_plan_pair_info": (C.c_int, [vp, C.POINTER(BtcfInfo)]),
    "b200spmm_plan_pair_copy_to_host": (C.c_int, [vp, vp, vp, vp, vp]),
    "b200spmm_plan_launch_info": (C.c_int, [vp, C.POINTER(LaunchInfo)]),
    "b200spmm_kat_umma": (C.c_int, [vp, u32, C.POINTER(KatMma), C.c_int, C.c_int, vp, C.c_int]),
    "b200spmm_kat_umma_pair": (C.c_int, [vp, u32, C.POINTER(KatMma), C.c_int, C.c_int, vp, C.c_int]),
    "b200spmm_kat_wait_limit": (C.c_uint64, [C.c_uint64]),
    "b200spmm_kat_spmm_starved": (C.c_int, [vp, vp, i64, i64, vp, i64, C.c_uint64, vp]),
    "b200spmm_kat_instr_desc": (u32, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "b200spmm_kat_tma": (C.c_int, [vp, u64, u64, u64, C.c_int, u32, u32, C.c_int, vp, C.c_int, u32, vp, u32,
                                    C.c_int]),
    "b200spmm_kat_umma_rate": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), C.c_int]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library; there is no fallback when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m hopper_spmm_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


class SpmmError(RuntimeError):
    def __init__(self, status: int, where: str):
        l = lib()
        msg = l.b200spmm_status_string(status).decode()
        if status == ERR_CUDA:
            msg += " - " + l.b200spmm_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} ({status})")
        self.status = status


def check(status: int, where: str) -> None:
    if status != OK:
        raise SpmmError(status, where)
