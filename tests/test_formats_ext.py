"""The reference's other formats and its file loader: bitmap-compressed BTCF_MTX (CSR2BTCF,
src/utils/convert.h:22-139), group-split GBTCF_MTX (BTCF2GBTCF, convert.h:232-276) and load_matrix
(src/utils/load.h:152-322).  The golden files hold what the reference's own code produced; the
oracle restates it; the library must agree with both, bit for bit."""
import os

import numpy as np
import pytest

import hopper_spmm_b200 as hs
import oracle
from cases import random_csr
from hopper_spmm_b200 import _capi as capi

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
FLAVOURS = [("fp16", np.float16, 16), ("tf32", np.float32, 8)]
CASES = ["hand", "rand_a", "rand_b", "wide"]


def golden_case(g, name):
    rows, cols = (int(x) for x in g[f"{name}_shape"])
    return rows, cols, g[f"{name}_row_ptr"], g[f"{name}_col_idx"], g[f"{name}_values"]


def bits_equal(a, b):
    return a.shape == b.shape and np.array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))


@pytest.mark.parametrize("flavour,dt,cw", FLAVOURS)
@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_the_reference_bitmap_converter(flavour, dt, cw, name):
    g = np.load(os.path.join(GOLDEN, f"format_ref_bitmap_{flavour}.npz"))
    rows, cols, rp, ci, v = golden_case(g, name)
    assert tuple(g[f"{name}_window"]) == (8, cw)
    # the reference's fp16 build addresses bitmap words by tile number: repeated only for this comparison
    o = oracle.csr2btcf_bitmap(rows, rp, ci, v, 8, cw, legacy_word_index=(flavour == "fp16"))
    for field in ("rowOffset", "nnzOffset", "tcA2B", "tcBit", "rowIdx"):
        assert np.array_equal(getattr(o, field), g[f"{name}_{field}"]), field
    assert bits_equal(o.data, g[f"{name}_data"])
    go, gr, at, length = oracle.btcf2gbtcf(o.rowOffset, o.rowIdx)
    assert np.array_equal(go, g[f"{name}_groupOffset"]) and np.array_equal(gr, g[f"{name}_group_rowIdx"])
    assert np.array_equal(at, g[f"{name}_atomic"]) and length >= 32


@pytest.mark.parametrize("flavour,dt,cw", FLAVOURS)
@pytest.mark.parametrize("name", CASES)
def test_library_bitmap_format_matches_the_reference(flavour, dt, cw, name):
    g = np.load(os.path.join(GOLDEN, f"format_ref_bitmap_{flavour}.npz"))
    rows, cols, rp, ci, v = golden_case(g, name)
    f = hs.CSR2BTCF(hs.CSR_MTX(rows, cols, rp, ci, v))  # the reference's 8-row windows
    assert (f.row_window, f.col_window, f.bitmap_words) == (8, cw, 8 * cw // 64)
    for field in ("rowOffset", "nnzOffset", "tcA2B", "rowIdx"):
        assert np.array_equal(getattr(f, field), g[f"{name}_{field}"]), field
    assert bits_equal(np.array(f.data), g[f"{name}_data"])
    if flavour == "tf32":  # one word per tile: the reference's indexing is sound there
        assert np.array_equal(f.tcBit, g[f"{name}_tcBit"])
    else:                  # two words per tile: compare with the restatement that keeps them apart
        assert np.array_equal(f.tcBit, oracle.csr2btcf_bitmap(rows, rp, ci, v, 8, cw).tcBit)
    # every tile: as many bits as stored values
    pop = np.array([bin(int(w)).count("1") for w in f.tcBit]).reshape(-1, f.bitmap_words).sum(1)
    assert np.array_equal(pop, np.diff(f.nnzOffset.astype(np.int64)))


@pytest.mark.parametrize("dt,cw", [(np.float16, 16), (np.float32, 8)])
@pytest.mark.parametrize("rw", [8, 16])
def test_bitmap_format_at_both_window_heights_expands_to_the_dense_format(dt, cw, rw):
    rows, cols, rp, ci, v = random_csr(203, 517, 0.05, 7, dt, empty_rows=[(48, 96)], dense_rows=[7, 200])
    v = v.copy()
    v[::5] = 0  # explicit zeros are stored values of the bitmap format
    f = hs.CSR2BTCF(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=rw)
    o = oracle.csr2btcf_bitmap(rows, rp, ci, v, rw, cw)
    for field in ("rowOffset", "nnzOffset", "tcA2B", "tcBit", "rowIdx"):
        assert np.array_equal(getattr(f, field), getattr(o, field)), field
    assert bits_equal(np.array(f.data), o.data) and f.nnzOffset[-1] == len(ci)
    dense = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=rw)
    back = f.expand()
    assert np.array_equal(back.rowOffset, dense.rowOffset) and np.array_equal(back.tcA2B, dense.tcA2B)
    assert np.array_equal(back.rowIdx, dense.rowIdx) and bits_equal(np.array(back.data), np.array(dense.data))


def test_bitmap_converter_refuses_rows_that_are_not_strictly_ascending():
    rp = np.array([0, 3], np.uint32)
    v = np.ones(3, np.float16)
    for ci in ([4, 2, 9], [2, 2, 9]):
        with pytest.raises(capi.SpmmError) as e:
            hs.CSR2BTCF(hs.CSR_MTX(1, 16, rp, np.array(ci, np.uint32), v))
        assert e.value.status == capi.ERR_BAD_CSR
    empty = hs.CSR2BTCF(hs.CSR_MTX(5, 7, np.zeros(6, np.uint32), np.zeros(0, np.uint32), np.zeros(0, np.float16)))
    assert empty.total_tiles == 0 and list(empty.nnzOffset) == [0] and list(empty.rowOffset) == [0]


@pytest.mark.parametrize("flavour,dt,cw", FLAVOURS)
@pytest.mark.parametrize("name", CASES)
def test_group_split_matches_the_reference_and_validates(flavour, dt, cw, name):
    g = np.load(os.path.join(GOLDEN, f"format_ref_bitmap_{flavour}.npz"))
    rows, cols, rp, ci, v = golden_case(g, name)
    f = hs.CSR2BTCF(hs.CSR_MTX(rows, cols, rp, ci, v))
    gb = hs.BTCF2GBTCF(f)
    assert np.array_equal(gb.groupOffset, g[f"{name}_groupOffset"])
    assert np.array_equal(gb.rowIdx, g[f"{name}_group_rowIdx"]) and np.array_equal(gb.atomic, g[f"{name}_atomic"])
    assert gb.total_groups == len(g[f"{name}_atomic"])
    assert hs.validateBTCF2GBTCFConversion(f, gb)
    if name == "wide":
        assert gb.atomic.any() and gb.total_groups > f.eff_row_windows


def test_group_validator_rejects_broken_lists():
    rng = np.random.default_rng(3)
    tiles = rng.integers(1, 200, 300)
    tiles[:4] = (1, 32, 33, 1000)

    class W:
        rowOffset = np.concatenate([[0], np.cumsum(tiles)]).astype(np.uint32)
        rowIdx = (np.arange(300) * 16).astype(np.uint32)

    gb = hs.BTCF2GBTCF(W)
    go, gr, at, length = oracle.btcf2gbtcf(W.rowOffset, W.rowIdx)
    assert gb.group_len == length == max(32, int(tiles.sum() / 300))
    assert np.array_equal(gb.groupOffset, go) and np.array_equal(gb.rowIdx, gr) and np.array_equal(gb.atomic, at)
    assert hs.validateBTCF2GBTCFConversion(W, gb)
    # every group stays inside its window and the groups of a window cover it
    assert go[0] == 0 and go[-1] == W.rowOffset[-1] and np.all(np.diff(go.astype(np.int64)) > 0)

    class Broken:
        total_groups = gb.total_groups
        groupOffset, rowIdx, atomic = np.array(gb.groupOffset), np.array(gb.rowIdx), np.array(gb.atomic)

    for field, k, val in (("groupOffset", 1, int(gb.groupOffset[1]) + 1), ("rowIdx", 7, 3), ("atomic", 0, 1)):
        b = Broken()
        arr = np.array(getattr(gb, field))
        arr[k] = val
        setattr(b, field, arr)
        assert not hs.validateBTCF2GBTCFConversion(W, b), field


@pytest.mark.parametrize("flavour,dt,cw", FLAVOURS)
@pytest.mark.parametrize("name,declared", [("sample", 14), ("short", 6)])
def test_loader_matches_the_reference_loader(flavour, dt, cw, name, declared):
    g = np.load(os.path.join(GOLDEN, f"mtx_ref_{flavour}.npz"))
    path = os.path.join(GOLDEN, f"{name}.mtx")
    m = hs.load_matrix(path, dt)
    assert (m.rows, m.cols) == tuple(g[f"{name}_shape"]) and m.declared_nnzs == declared
    assert np.array_equal(m.row_ptr, g[f"{name}_row_ptr"]) and np.array_equal(m.col_idx, g[f"{name}_col_idx"])
    assert bits_equal(m.values, g[f"{name}_values"])
    rows, cols, rp, ci, v = oracle.load_matrix_text(open(path).read(), dt)
    assert (rows, cols) == (m.rows, m.cols) and np.array_equal(rp, m.row_ptr) and np.array_equal(ci, m.col_idx)
    assert bits_equal(v, m.values)
    if name == "short":
        assert m.nnzs == 3  # fewer entries than promised: the file simply has fewer (load.h:232-236)


def test_loader_errors(tmp_path):
    with pytest.raises(capi.SpmmError) as e:
        hs.load_matrix(str(tmp_path / "missing.mtx"))
    assert e.value.status == capi.ERR_INVALID_ARG
    bad = tmp_path / "bad.mtx"
    bad.write_text("%%MatrixMarket matrix coordinate real general\n3 3 2\n1 1 1.0\n4 1 2.0\n")
    with pytest.raises(capi.SpmmError) as e:
        hs.load_matrix(str(bad))
    assert e.value.status == capi.ERR_BAD_CSR
    nosize = tmp_path / "nosize.mtx"
    nosize.write_text("% only comments\n")
    with pytest.raises(capi.SpmmError):
        hs.load_matrix(str(nosize))
    pattern = tmp_path / "pattern.mtx"  # no values: no line reads as an entry
    pattern.write_text("%%MatrixMarket matrix coordinate pattern general\n2 2 2\n1 1\n2 2\n")
    m = hs.load_matrix(str(pattern))
    assert m.nnzs == 0 and list(m.row_ptr) == [0, 0, 0]
