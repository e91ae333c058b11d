"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations (uniform-random CSR, 16x8 block-clustered, R-MAT graph adjacency, pruned weight).

They stand in for the public graph / pruned-weight datasets such workloads are usually run on;
no dataset is reproduced.  Everything is derived from one counter-based generator (a
splitmix64-style hash of (seed, stream, index)) written in integer tensor arithmetic, so the
same inputs come out on CPU and on CUDA and do not depend on thread count or chunking.
Normal deviates use Box-Muller in float64 and may differ in the last bit between devices;
uniform deviates are exact.
"""
from __future__ import annotations

import math

import numpy as np
import torch

_M1 = 0xBF58476D1CE4E5B9 - (1 << 64)
_M2 = 0x94D049BB133111EB - (1 << 64)
_GOLD = 0x9E3779B97F4A7C15 - (1 << 64)


def _lsr(x: torch.Tensor, k: int) -> torch.Tensor:
    """Logical right shift of int64 bit patterns."""
    return (x >> k) & ((1 << (64 - k)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    x = (x ^ _lsr(x, 30)) * _M1
    x = (x ^ _lsr(x, 27)) * _M2
    return x ^ _lsr(x, 31)


def _wrap(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _mix_int(x: int) -> int:
    m = (1 << 64) - 1
    x &= m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def rand_bits(seed: int, stream: int, idx: torch.Tensor) -> torch.Tensor:
    """64 random bits (as int64) for every index in ``idx`` (int64 tensor)."""
    key = _wrap(_mix_int(seed * 0x9E3779B97F4A7C15 + stream))
    return _mix(idx * _GOLD + key)


def uniform01_f32(bits: torch.Tensor, part: int = 0) -> torch.Tensor:
    """Exact fp32 uniform on [0,1) with 24-bit resolution from bits [40,64) (part 0) or [8,32) (part 1)."""
    sh = 40 if part == 0 else 8
    return (_lsr(bits, sh) & 0xFFFFFF).to(torch.float32) * (1.0 / (1 << 24))


def uniform01_f64(bits: torch.Tensor) -> torch.Tensor:
    return _lsr(bits, 11).to(torch.float64) * (1.0 / (1 << 53))


def normal_f64(seed: int, stream: int, idx: torch.Tensor) -> torch.Tensor:
    """Standard normal deviates (Box-Muller on two independent uniforms)."""
    u1 = uniform01_f64(rand_bits(seed, stream, idx * 2))
    u2 = uniform01_f64(rand_bits(seed, stream, idx * 2 + 1))
    return torch.sqrt(-2.0 * torch.log1p(-u1)) * torch.cos((2.0 * math.pi) * u2)


def _arange(n: int, device, start: int = 0) -> torch.Tensor:
    return torch.arange(start, start + n, dtype=torch.int64, device=device)


def dense_uniform(rows: int, cols: int, seed: int, stream: int, device="cpu", dtype=torch.float16) -> torch.Tensor:
    """Row-major [rows, cols] with entries U[-1,1): an exact fp32 draw rounded to ``dtype``."""
    out = torch.empty((rows, cols), dtype=dtype, device=device)
    step = max(1, (1 << 24) // max(cols, 1))
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        idx = _arange((r1 - r0) * cols, device, r0 * cols)
        out[r0:r1] = (uniform01_f32(rand_bits(seed, stream, idx)) * 2.0 - 1.0).to(dtype).view(r1 - r0, cols)
    return out


def dense_normal(rows: int, cols: int, seed: int, stream: int, device="cpu", dtype=torch.float16,
                 sigma: float = 1.0) -> torch.Tensor:
    out = torch.empty((rows, cols), dtype=dtype, device=device)
    step = max(1, (1 << 23) // max(cols, 1))
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        idx = _arange((r1 - r0) * cols, device, r0 * cols)
        out[r0:r1] = (normal_f64(seed, stream, idx) * sigma).to(torch.float32).to(dtype).view(r1 - r0, cols)
    return out


class Csr:
    """CSR_MTX fields (reference: src/utils/class.h:30-37) as tensors: row_ptr int64 [rows+1],
    col_idx int32 [nnz] ascending inside each row, values fp16 or fp32 [nnz]."""

    def __init__(self, rows, cols, row_ptr, col_idx, values):
        self.rows, self.cols = int(rows), int(cols)
        self.row_ptr, self.col_idx, self.values = row_ptr, col_idx, values
        self.nnz = int(col_idx.numel())

    def numpy(self):
        """(row_ptr uint32, col_idx uint32, values) as numpy arrays on the host."""
        return (self.row_ptr.cpu().numpy().astype(np.uint32), self.col_idx.cpu().numpy().astype(np.uint32),
                self.values.cpu().numpy())

    def row_slice(self, r0: int, r1: int) -> "Csr":
        lo, hi = int(self.row_ptr[r0]), int(self.row_ptr[r1])
        return Csr(r1 - r0, self.cols, self.row_ptr[r0:r1 + 1] - lo, self.col_idx[lo:hi], self.values[lo:hi])


def _csr_from_sorted_keys(keys: torch.Tensor, rows: int, cols: int):
    """keys = row * cols_pow2 + col ... callers pass (row << 32) | col, sorted and distinct."""
    r = keys >> 32
    c = (keys & 0xFFFFFFFF).to(torch.int32)
    counts = torch.bincount(r, minlength=rows)
    row_ptr = torch.zeros(rows + 1, dtype=torch.int64, device=keys.device)
    row_ptr[1:] = torch.cumsum(counts, 0)
    return row_ptr, c, r


def uniform_random_csr(rows: int, cols: int, density: float, seed: int = 0, device="cpu") -> Csr:
    """Uniform-random sparsity, columns sampled without replacement per row; row r holds
    floor(d*(r+1)) - floor(d*r) entries with d = density*cols (40 or 41 at 4096 x 1 %).
    Values U[-1,1) fp16."""
    d = density * cols
    r = torch.arange(rows + 1, dtype=torch.float64)
    per_row = (torch.floor(d * r[1:]) - torch.floor(d * r[:-1])).to(torch.int64).to(device)
    keys_out = []
    step = max(1, (1 << 24) // cols)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        idx = _arange((r1 - r0) * cols, device, r0 * cols)
        k = _lsr(rand_bits(seed, 1, idx), 1).view(r1 - r0, cols)
        order = torch.argsort(k, dim=1)  # a random permutation of the columns of every row
        take = _arange(cols, device)[None, :] < per_row[r0:r1, None]
        rr = _arange(r1 - r0, device, r0)[:, None].expand(-1, cols)
        keys_out.append((rr[take] << 32) | order[take])
    keys = torch.sort(torch.cat(keys_out)).values
    row_ptr, col_idx, _ = _csr_from_sorted_keys(keys, rows, cols)
    vals = (uniform01_f32(rand_bits(seed, 2, _arange(keys.numel(), device))) * 2.0 - 1.0).to(torch.float16)
    return Csr(rows, cols, row_ptr, col_idx, vals)


def block_clustered_csr(rows: int, cols: int, density: float, seed: int = 0, device="cpu", block_rows: int = 16,
                        block_cols: int = 8) -> Csr:
    """Non-zeros clustered into aligned block_rows x block_cols blocks: round(density * slots)
    distinct slots chosen uniformly, every entry of a chosen block non-zero, values N(0,1) fp32."""
    gr, gc = rows // block_rows, cols // block_cols
    n_slots = gr * gc
    n_pick = int(round(density * n_slots))
    k = _lsr(rand_bits(seed, 1, _arange(n_slots, device)), 1)
    slots = torch.sort(torch.topk(k, n_pick, largest=False, sorted=False).indices).values
    br, bc = slots // gc, slots % gc
    lr = _arange(block_rows, device)[None, :, None]
    lc = _arange(block_cols, device)[None, None, :]
    r = (br[:, None, None] * block_rows + lr).expand(-1, block_rows, block_cols)
    c = (bc[:, None, None] * block_cols + lc).expand(-1, block_rows, block_cols)
    keys = torch.sort(((r << 32) | c).reshape(-1)).values
    row_ptr, col_idx, _ = _csr_from_sorted_keys(keys, rows, cols)
    vals = normal_f64(seed, 2, _arange(keys.numel(), device)).to(torch.float32)
    return Csr(rows, cols, row_ptr, col_idx, vals)


def rmat_edges(scale: int, n_edges: int, seed: int, device, a=0.57, b=0.19, c=0.19, chunk: int = 1 << 25):
    """Sorted distinct (row << 32 | col) keys of an R-MAT graph with 2**scale nodes, no noise."""
    out = []
    ab, abc = a + b, a + b + c
    for e0 in range(0, n_edges, chunk):
        m = min(chunk, n_edges - e0)
        idx = _arange(m, device, e0)
        row = torch.zeros(m, dtype=torch.int64, device=device)
        col = torch.zeros(m, dtype=torch.int64, device=device)
        for lvl in range(scale):
            if lvl % 2 == 0:
                bits = rand_bits(seed, 16 + lvl // 2, idx)
            u = uniform01_f32(bits, lvl % 2)
            down = u >= ab                      # quadrants c, d: lower half of the rows
            right = ((u >= a) & (u < ab)) | (u >= abc)  # quadrants b, d: right half of the columns
            row = (row << 1) | down.to(torch.int64)
            col = (col << 1) | right.to(torch.int64)
        out.append(torch.unique((row << 32) | col))
        del row, col, idx
    keys = torch.cat(out) if len(out) > 1 else out[0]
    return torch.unique(keys) if len(out) > 1 else keys


def rmat_csr(scale: int, avg_degree: int, seed: int = 0, device="cpu", self_loops: bool = False) -> Csr:
    """GNN-style adjacency: R-MAT (0.57, 0.19, 0.19, 0.05), duplicates removed, optional self
    loops, values 1/deg(row) in fp16 where deg counts the stored entries of the row."""
    n = 1 << scale
    keys = rmat_edges(scale, avg_degree * n, seed, device)
    if self_loops:
        diag = _arange(n, device)
        keys = torch.unique(torch.cat([keys, (diag << 32) | diag]))
    row_ptr, col_idx, r = _csr_from_sorted_keys(keys, n, n)
    deg = (row_ptr[1:] - row_ptr[:-1]).to(torch.float32)
    vals = (1.0 / deg)[r].to(torch.float16)
    return Csr(n, n, row_ptr, col_idx, vals)


def pruned_weight_csr(rows: int, cols: int, keep: float = 0.1, sigma: float = 0.02, seed: int = 0,
                      device="cpu") -> Csr:
    """Unstructured pruning: keep-mask Bernoulli(keep) per entry, kept values N(0, sigma) fp16."""
    keys_out = []
    step = max(1, (1 << 24) // cols)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        idx = _arange((r1 - r0) * cols, device, r0 * cols)
        kept = uniform01_f64(rand_bits(seed, 1, idx)) < keep
        lin = idx[kept]
        keys_out.append(((lin // cols) << 32) | (lin % cols))
    keys = torch.cat(keys_out)  # already ordered by (row, col)
    row_ptr, col_idx, r = _csr_from_sorted_keys(keys, rows, cols)
    lin = r * cols + col_idx.to(torch.int64)
    vals = (normal_f64(seed, 2, lin) * sigma).to(torch.float32).to(torch.float16)
    return Csr(rows, cols, row_ptr, col_idx, vals)


# ---------------------------------------------------------------------- the five configurations

CONFIGS = {
    # name: (dtype, N features, description)
    "uniform_4096_fp16": ("f16", 128, "A 4096x4096 uniform 1%, B 4096x128 U[-1,1] fp16"),
    "blocks_16384_tf32": ("tf32", 256, "A 16384x16384 16x8 blocks 0.5%, B 16384x256 N(0,1) fp32"),
    "rmat20_gnn_fp16": ("f16", 64, "R-MAT 2^20 deg 16 + self loops, 1/deg fp16, B 2^20x64 U[-1,1]"),
    "pruned_llm_fp16": ("f16", 2048, "A 28672x8192 keep 10% N(0,0.02), B 8192x2048 N(0,1) fp16"),
    "rmat24_sharded_fp16": ("f16", 128, "R-MAT 2^24 deg 32, 1/deg fp16, B 2^24x128 U[-1,1], row-sharded"),
}


def make_config(name: str, seed: int = 0, device="cpu", scale_down: int = 0):
    """Returns (Csr, B tensor) of a configuration.  ``scale_down`` k shrinks every matrix
    dimension by 2**k (R-MAT: scale - k) for tests; 0 is the full size."""
    k = scale_down
    if name == "uniform_4096_fp16":
        m = 4096 >> k
        return uniform_random_csr(m, m, 0.01, seed, device), dense_uniform(m, 128, seed, 3, device)
    if name == "blocks_16384_tf32":
        m = 16384 >> k
        return (block_clustered_csr(m, m, 0.005, seed, device),
                dense_normal(m, 256, seed, 3, device, torch.float32))
    if name == "rmat20_gnn_fp16":
        s = 20 - k
        return rmat_csr(s, 16, seed, device, self_loops=True), dense_uniform(1 << s, 64, seed, 3, device)
    if name == "pruned_llm_fp16":
        return (pruned_weight_csr(28672 >> k, 8192 >> k, 0.1, 0.02, seed, device),
                dense_normal(8192 >> k, 2048 >> min(k, 3), seed, 3, device))
    if name == "rmat24_sharded_fp16":
        s = 24 - k
        return rmat_csr(s, 32, seed, device, self_loops=False), dense_uniform(1 << s, 128, seed, 3, device)
    raise KeyError(name)
