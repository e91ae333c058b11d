"""B200 (sm_100a) condensed row-window SpMM behind the operator surface of Ritt2020/hopper_spmm.

The computing code is CUDA/C++ in ``csrc/`` behind the C ABI of ``include/b200_spmm.h``;
``spmm`` mirrors the reference's host interface over it, ``synth`` makes the seeded synthetic
benchmark inputs.
"""
from .spmm import (BTCF_MTX_NO_BITMAP, CSR2BTCFNOBITMAP, CSR_MTX, DENSE_MTX, DeviceBtcf, IDX_MAX, PERF_RESULT, ROW_WINDOW, RUNS,
                   WARMUP_RUNS, ShardedSpmm, SpmmPlan, fp16_spmm, rewindow, shard_rows, tf32_spmm, transpose_tiles)

from .formats import BTCF2GBTCF, BTCF_MTX, CSR2BTCF, GBTCF_MTX, load_matrix, validateBTCF2GBTCFConversion

__all__ = ["BTCF2GBTCF", "BTCF_MTX", "CSR2BTCF", "GBTCF_MTX", "load_matrix", "validateBTCF2GBTCFConversion", "BTCF_MTX_NO_BITMAP", "CSR2BTCFNOBITMAP", "CSR_MTX", "DENSE_MTX", "DeviceBtcf", "IDX_MAX", "PERF_RESULT", "ROW_WINDOW",
           "RUNS", "WARMUP_RUNS", "ShardedSpmm", "SpmmPlan", "fp16_spmm", "rewindow", "shard_rows", "tf32_spmm", "transpose_tiles"]
