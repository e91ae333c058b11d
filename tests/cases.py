"""Small seeded matrices shared by the CPU and GPU parity tests."""
import numpy as np


def random_csr(rows, cols, density, seed, dtype=np.float16, empty_rows=(), dense_rows=()):
    """Random CSR with ascending columns per row; `empty_rows` ranges are cleared and
    `dense_rows` hold every column."""
    rng = np.random.default_rng(seed)
    mask = rng.random((rows, cols)) < density
    for lo, hi in empty_rows:
        mask[lo:hi] = False
    for r in dense_rows:
        mask[r] = True
    row_ptr = np.concatenate([[0], np.cumsum(mask.sum(1))]).astype(np.uint32)
    col_idx = np.nonzero(mask)[1].astype(np.uint32)
    vals = rng.uniform(-1, 1, col_idx.size).astype(np.float32).astype(dtype)
    return rows, cols, row_ptr, col_idx, vals


def dense_b(cols, n, seed, dtype=np.float16):
    rng = np.random.default_rng(seed + 1000)
    return rng.uniform(-1, 1, (cols, n)).astype(np.float32).astype(dtype)


FORMAT_FIELDS = ("rowOffset", "tcA2B", "data", "rowIdx")


def same_format(f, g):
    """Bit-for-bit equality of two converted matrices (any objects with the four arrays)."""
    for k in FORMAT_FIELDS:
        a = np.ascontiguousarray(getattr(f, k)).view(np.uint8)
        b = np.ascontiguousarray(getattr(g, k)).view(np.uint8)
        if a.shape != b.shape or not np.array_equal(a, b):
            return False
    return (f.eff_row_windows, f.total_tiles) == (g.eff_row_windows, g.total_tiles)
