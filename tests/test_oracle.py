"""The oracle against the reference: golden format vectors produced by the reference's own
converter, the live harness where it is built, and the closed-form answers of the reference's
single-tile tests."""
import os

import numpy as np
import pytest

import oracle
from cases import FORMAT_FIELDS, random_csr, same_format

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("flavour", ["fp16", "tf32"])
@pytest.mark.parametrize("case", ["hand", "rand_a", "rand_b"])
def test_converter_matches_reference_golden(flavour, case):
    g = np.load(os.path.join(GOLDEN, f"format_ref_{flavour}.npz"))
    rows, cols = (int(x) for x in g[f"{case}_shape"])
    rw, cw = (int(x) for x in g[f"{case}_window"])
    assert (rw, cw) == ((8, 16) if flavour == "fp16" else (8, 8))  # src/common.h:17-18,40-41
    f = oracle.csr2btcf_nobitmap(rows, cols, g[f"{case}_row_ptr"], g[f"{case}_col_idx"], g[f"{case}_values"], rw, cw)
    for k in FORMAT_FIELDS:
        assert np.array_equal(getattr(f, k).view(np.uint8), g[f"{case}_{k}"].view(np.uint8)), k


def test_hand_example_values():
    # 20x40 example converted by the reference itself: three windows of one tile each.
    g = np.load(os.path.join(GOLDEN, "format_ref_fp16.npz"))
    M = 0xFFFFFFFF
    assert g["hand_rowOffset"].tolist() == [0, 1, 2, 3]
    assert g["hand_rowIdx"].tolist() == [0, 8, 16]
    assert g["hand_tcA2B"].tolist() == [0, 4, 16, 32] + [M] * 12 + [1, 39] + [M] * 14 + [6, 7] + [M] * 14
    assert g["hand_data"].size == 384


@pytest.mark.parametrize("flavour,dt", [("fp16", np.float16), ("tf32", np.float32)])
def test_converter_matches_live_reference(flavour, dt):
    if not oracle.ref_available(flavour):
        pytest.skip("reference harness not built (needs the reference sources)")
    for seed in range(6):
        rows, cols = [(17, 40), (64, 64), (333, 1000), (8, 5), (1, 1), (250, 77)][seed]
        rows, cols, rp, ci, v = random_csr(rows, cols, [0.05, 0.3, 0.01, 0.5, 1.0, 0.08][seed], seed, dt,
                                           empty_rows=[(8, 24)] if rows > 24 else ())
        ref = oracle.ref_convert(flavour, rows, cols, rp, ci, v)
        mine = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, ref.row_window, ref.col_window)
        assert same_format(mine, ref)


@pytest.mark.parametrize("flavour,dt", [("fp16", np.float16), ("tf32", np.float32)])
def test_live_reference_output_rewindows_to_the_sixteen_row_format(flavour, dt):
    # the reference's converter runs here (8-row windows); its arrays, re-windowed by the library,
    # must equal the restated converter's 16-row output
    if not oracle.ref_available(flavour):
        pytest.skip("reference harness not built (needs the reference sources)")
    import hopper_spmm_b200 as hs
    for seed in range(5):
        rows, cols = [(17, 40), (64, 64), (333, 1000), (9, 5), (250, 77)][seed]
        rows, cols, rp, ci, v = random_csr(rows, cols, [0.05, 0.3, 0.01, 0.5, 0.08][seed], seed, dt,
                                           empty_rows=[(8, 24), (40, 48)] if rows > 48 else ())
        ref = oracle.ref_convert(flavour, rows, cols, rp, ci, v)
        f16 = hs.rewindow(rows, cols, len(ci), ref.rowOffset, ref.tcA2B, ref.data, ref.rowIdx, row_window_in=8)
        assert same_format(f16, oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, 16, ref.col_window))


def test_kat1_fp16_single_tile():
    # src/test_fp16.cu:407-415: A[i] = half(i+1) (64x16, K-major), B = 1 (8x16) -> C[r][c] = 256 r + 136
    A = np.arange(1, 64 * 16 + 1, dtype=np.float32).astype(np.float16).astype(np.float32).reshape(64, 16)
    B = np.ones((8, 16), np.float32)
    C = oracle.tile_accumulate(A, B, 64, 8, 16, 1)
    expect = (256.0 * np.arange(64) + 136.0)[:, None].repeat(8, 1)
    assert np.array_equal(C, expect)


def test_kat2_tf32_single_tile():
    # test/02.tma_and_wgmma/tma_wgmma.cu:340-348: A[i] = i+1 (64x8), B[i] = 1 + 0.01 i (8x8)
    A = np.arange(1, 64 * 8 + 1, dtype=np.float32).reshape(64, 8)
    B = (1.0 + 0.01 * np.arange(64, dtype=np.float32)).astype(np.float32).reshape(8, 8)
    C = oracle.tile_accumulate(A, B, 64, 8, 8, 1)
    expect = A.astype(np.float64) @ B.astype(np.float64).T
    bad, max_rel, _ = oracle.compare(C, expect.astype(np.float32), 1e-6)
    assert bad == 0 and max_rel < 1e-6


def test_kat3_pipeline_accumulate():
    # test/03.warp_specialized/main.cu:235-241: srand(42), A 64 x (8 T), B 8 x (8 T), rand()/RAND_MAX
    T = 16
    stream = oracle.rand_fill(42, 64 * 8 * T + 8 * 8 * T)
    A, B = stream[:64 * 8 * T].reshape(64, 8 * T), stream[64 * 8 * T:].reshape(8, 8 * T)
    assert 0.0 <= stream.min() and stream.max() <= 1.0
    C = oracle.tile_accumulate(A, B, 64, 8, 8, T)
    expect = A.astype(np.float64) @ B.astype(np.float64).T
    assert np.allclose(C, expect, rtol=1e-5)


def test_compare_rule():
    ref = np.array([[1.0, 1e-7, 100.0, 0.0]], np.float32)
    ok = np.array([[1.009, 1e-7 + 9e-6, 100.9, 5e-6]], np.float32)
    assert oracle.compare(ok, ref, 0.01)[0] == 0           # tf32.cu:47-71
    bad = np.array([[1.02, 1e-7 + 2e-5, 100.0, np.nan]], np.float32)
    assert oracle.compare(bad, ref, 0.01)[0] == 3
    assert oracle.compare_abs(np.array([0.0, 2.0]), np.array([0.9, 0.5]), 1.0) == 1  # verify.h:26


def test_csr_and_tile_forms_agree():
    for dt, cw in ((np.float16, 16), (np.float32, 8)):
        rows, cols, rp, ci, v = random_csr(150, 300, 0.05, 3, dt, empty_rows=[(32, 64)])
        B = np.random.default_rng(5).uniform(-1, 1, (cols, 40)).astype(dt)
        f = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, 16, cw)
        c1 = oracle.spmm_csr(rows, rp, ci, v, B)
        c2 = oracle.spmm_btcf(f, B)
        dense = np.zeros((rows, cols))
        dense[np.repeat(np.arange(rows), np.diff(rp.astype(np.int64))), ci] = v.astype(np.float64)
        exact = dense @ B.astype(np.float64)
        assert np.abs(c1 - exact).max() < 1e-4 and np.abs(c2 - exact).max() < 1e-4
        assert np.all(c1[32:64] == 0)


def test_half_conversions_exact():
    h = np.arange(65536, dtype=np.uint16)
    f = oracle.half_to_float(h)
    ref = h.view(np.float16).astype(np.float32)
    keep = ~np.isnan(ref)
    assert np.array_equal(f.view(np.uint32)[keep], ref.view(np.uint32)[keep])
    x = np.random.default_rng(0).standard_normal(100000).astype(np.float32)
    x *= np.random.default_rng(1).choice([1e-8, 1e-5, 1.0, 1e3, 6e4], x.size).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.float_to_half(x), x.astype(np.float16).view(np.uint16))
