"""Synthetic-input generators: pinned by checksums, right counts and distributions."""
import hashlib
import json
import os

import numpy as np
import pytest

from hopper_spmm_b200 import synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_matches_committed_checksums():
    sums = json.load(open(os.path.join(GOLDEN, "synth_checksums.json")))
    for key, want in sums.items():
        name, k = key.split("/")
        csr, B = synth.make_config(name, 0, "cpu", int(k))
        rp, ci, v = csr.numpy()
        h = hashlib.sha256()
        for a in (rp, ci):
            h.update(np.ascontiguousarray(a).tobytes())
        assert (csr.rows, csr.cols, csr.nnz) == (want["rows"], want["cols"], want["nnz"])
        assert h.hexdigest() == want["structure_sha256"], key
        assert abs(float(np.asarray(v, np.float64).sum()) - want["values_sum"]) <= 1e-6 * max(1, csr.nnz ** 0.5)


def test_uniform_config_counts():
    csr, B = synth.make_config("uniform_4096_fp16")
    rp, ci, v = csr.numpy()
    assert csr.nnz == 167772 and B.shape == (4096, 128)
    per_row = np.diff(rp.astype(np.int64))
    assert set(per_row.tolist()) == {40, 41}
    for r in (0, 17, 4095):  # without replacement, ascending
        assert np.all(np.diff(ci[rp[r]:rp[r + 1]].astype(np.int64)) > 0)
    assert -1 <= v.astype(np.float32).min() and v.astype(np.float32).max() <= 1  # fp16 rounding can reach 1.0


def test_block_config_counts():
    csr, B = synth.make_config("blocks_16384_tf32")
    rp, ci, v = csr.numpy()
    assert csr.nnz == 1342208 and B.shape == (16384, 256) and v.dtype == np.float32
    per_row = np.diff(rp.astype(np.int64))
    assert np.all(per_row % 8 == 0)
    assert np.all(per_row.reshape(-1, 16) == per_row.reshape(-1, 16)[:, :1])  # 16-row aligned blocks
    assert abs(float(v.std()) - 1.0) < 0.01


def test_rmat_properties():
    csr, B = synth.make_config("rmat20_gnn_fp16", scale_down=7)
    rp, ci, v = csr.numpy()
    n = csr.rows
    assert n == 1 << 13 and B.shape == (n, 64)
    deg = np.diff(rp.astype(np.int64))
    assert deg.min() >= 1  # self loops
    rows = np.repeat(np.arange(n), deg)
    assert np.all(np.isin(np.arange(n) * n + np.arange(n), rows * n + ci))
    assert np.allclose(v.astype(np.float32), (1.0 / deg[rows]).astype(np.float16).astype(np.float32))
    assert deg[: n // 2].sum() > 2.5 * deg[n // 2:].sum()  # a + b = 0.76 of the mass in the upper half


def test_pruned_weight_density():
    csr, B = synth.make_config("pruned_llm_fp16", scale_down=3)
    rp, ci, v = csr.numpy()
    dens = csr.nnz / (csr.rows * csr.cols)
    assert abs(dens - 0.1) < 0.002 and abs(float(v.astype(np.float32).std()) - 0.02) < 0.001


@pytest.mark.gpu
def test_cuda_generation_equals_cpu():
    import torch
    for name, k in (("uniform_4096_fp16", 2), ("rmat24_sharded_fp16", 10), ("blocks_16384_tf32", 3)):
        a, _ = synth.make_config(name, 0, "cpu", k)
        b, _ = synth.make_config(name, 0, "cuda", k)
        assert torch.equal(a.row_ptr, b.row_ptr.cpu()) and torch.equal(a.col_idx, b.col_idx.cpu())
