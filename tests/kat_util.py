"""Shared-memory operand images for the single-tile tcgen05 known-answer tests.

The packers put a logical matrix into the byte layout the SpMM kernel uses:
  * gathered rows of B (UMMA "A" operand, M = features): MN-major, 128-byte swizzle.
    fp16: 64-feature blocks of 8 k-rows x 128 B (1 KiB), block (h, g) at (2h + g) KiB where g is
    the group of 8 k-rows, 16-byte units XORed with the row number; tf32: 32-feature blocks of
    4 k-rows x 128 B (512 B), block (h, g) at (2h + g) * 512 B, 32-byte units XORed with the row
    number (the only MN-major layout tcgen05 takes for 32-bit operands).
  * 16 x CW tile of the sparse matrix (UMMA "B" operand, N = 16 window rows): K-major rows of
    32 bytes with the 32-byte swizzle, i.e. the 16-byte half of a row is flipped on rows 4-7
    and 12-15.
"""
import ctypes as C

import numpy as np

from hopper_spmm_b200 import _capi as capi


def pack_gathered(mat: np.ndarray) -> bytes:
    """mat[m features][k]: fp16 with k = 16, or fp32 with k = 8."""
    m_dim, k_dim = mat.shape
    esz = mat.dtype.itemsize
    per16 = 16 // esz                      # elements per 16-byte piece
    per_block = 128 // esz                 # features per 128-byte block row
    n_blocks = (m_dim + per_block - 1) // per_block
    group_rows = 8 if esz == 2 else 4      # k-rows per swizzle group
    groups = (k_dim + group_rows - 1) // group_rows
    group_bytes = group_rows * 128
    img = np.zeros(n_blocks * groups * group_bytes, np.uint8)
    raw = mat.view(np.uint8).reshape(m_dim, k_dim, esz)
    for m in range(m_dim):
        h, cc, e = m // per_block, (m % per_block) // per16, m % per16
        for k in range(k_dim):
            g, kr = k // group_rows, k % group_rows
            if esz == 2:    # 16-byte units XORed with the row number
                unit = (cc ^ kr) << 4
            else:           # 32-byte units XORed with the row number
                unit = (((cc >> 1) ^ kr) << 5) | ((cc & 1) << 4)
            off = (h * groups + g) * group_bytes + kr * 128 + unit + e * esz
            img[off:off + esz] = raw[m, k]
    return img.tobytes()


def pack_tile(tile: np.ndarray) -> bytes:
    """tile[16 rows][CW]: fp16 with CW = 16 or fp32 with CW = 8 (32-byte rows)."""
    rows, cw = tile.shape
    assert cw * tile.dtype.itemsize == 32
    raw = np.ascontiguousarray(tile).view(np.uint8).reshape(rows, 2, 16)
    img = np.zeros((rows, 2, 16), np.uint8)
    for r in range(rows):
        flip = (r >> 2) & 1
        img[r, 0 ^ flip] = raw[r, 0]
        img[r, 1 ^ flip] = raw[r, 1]
    return img.tobytes()


def run_umma(image: bytes, mmas, n_cols=16, device=0):
    """Returns (status, D[128, n_cols] float32)."""
    lib = capi.lib()
    arr = (capi.KatMma * len(mmas))(*mmas)
    out = np.zeros((128, n_cols), np.float32)
    buf = np.frombuffer(image, np.uint8)
    st = lib.b200spmm_kat_umma(buf.ctypes.data, len(image), arr, len(mmas), n_cols, out.ctypes.data, device)
    return st, out


def spmm_tile_mma(tf32: bool, m: int, a_off: int, b_off: int, d_col=0, accumulate=0):
    """The MMA the SpMM kernel issues for one tile and one feature chunk."""
    idesc = capi.lib().b200spmm_kat_instr_desc(2 if tf32 else 0, m, 16, 1, 0)
    return capi.KatMma(a_off=a_off, a_lbo=1024 if tf32 else 2048, a_sbo=512 if tf32 else 1024,
                       a_swizzle=1 if tf32 else 2, b_off=b_off, b_lbo=16,
                       b_sbo=256, b_swizzle=6, idesc=idesc, d_col=d_col, accumulate=accumulate, kind=1 if tf32 else 0)


def m64_rows(d: np.ndarray) -> np.ndarray:
    """Rows of an M = 64 accumulator: row i sits in TMEM lane (i % 16) + 32 * (i // 16)."""
    lanes = [(i % 16) + 32 * (i // 16) for i in range(64)]
    return d[lanes]


def run_tma(tensor: np.ndarray, box_inner, box_rows, swizzle, loads, expect_bytes, dump_bytes, device=0):
    lib = capi.lib()
    rows, inner = tensor.shape
    t = np.ascontiguousarray(tensor)
    l = np.ascontiguousarray(np.array(loads, np.int32).reshape(-1, 7))
    dump = np.zeros(dump_bytes, np.uint8)
    st = lib.b200spmm_kat_tma(t.ctypes.data, inner, rows, inner * t.dtype.itemsize, t.dtype.itemsize, box_inner,
                              box_rows, swizzle, l.ctypes.data, len(l), expect_bytes, dump.ctypes.data, dump_bytes,
                              device)
    return st, dump
