"""The shipped converter (through the C ABI) against the oracle and the reference's golden
vectors, bit for bit, plus the host-side planners."""
import ctypes as C
import os

import numpy as np
import pytest

import hopper_spmm_b200 as hs
import oracle
from cases import FORMAT_FIELDS, random_csr, same_format
from hopper_spmm_b200 import _capi as capi

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def convert(rows, cols, rp, ci, v, rw=16, cw=0, threads=0):
    return hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=rw, col_window=cw, n_threads=threads)


@pytest.mark.parametrize("flavour", ["fp16", "tf32"])
@pytest.mark.parametrize("case", ["hand", "rand_a", "rand_b"])
def test_library_matches_reference_golden(flavour, case):
    g = np.load(os.path.join(GOLDEN, f"format_ref_{flavour}.npz"))
    rows, cols = (int(x) for x in g[f"{case}_shape"])
    f = convert(rows, cols, g[f"{case}_row_ptr"], g[f"{case}_col_idx"], g[f"{case}_values"], rw=8)
    for k in FORMAT_FIELDS:
        assert np.array_equal(np.asarray(getattr(f, k)).view(np.uint8), g[f"{case}_{k}"].view(np.uint8)), k
    assert f.total_row_windows == (rows + 7) // 8


@pytest.mark.parametrize("dt,cw", [(np.float16, 16), (np.float32, 8), (np.float32, 4), (np.float16, 8)])
@pytest.mark.parametrize("rw", [8, 16])
def test_library_matches_oracle(dt, cw, rw):
    shapes = [(1, 1, 1.0), (16, 16, 0.5), (17, 33, 0.2), (203, 517, 0.03), (500, 70000, 0.0005), (96, 7, 0.6)]
    for seed, (rows, cols, dens) in enumerate(shapes):
        rows, cols, rp, ci, v = random_csr(rows, cols, dens, seed, dt, empty_rows=[(16, 48)] if rows > 64 else (),
                                           dense_rows=[3] if cols < 1000 and rows > 3 else ())
        a = convert(rows, cols, rp, ci, v, rw, cw, threads=seed % 3)
        b = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, rw, cw)
        assert same_format(a, b)
        assert a.rowOffset[-1] == a.total_tiles and len(a.tcA2B) == a.total_tiles * cw


def test_empty_matrix_and_empty_windows():
    rp = np.zeros(41, np.uint32)
    f = convert(40, 10, rp, np.zeros(0, np.uint32), np.zeros(0, np.float16))
    assert (f.eff_row_windows, f.total_tiles, f.total_row_windows) == (0, 0, 3)
    assert f.rowOffset.tolist() == [0]
    rows, cols, rp, ci, v = random_csr(80, 50, 0.1, 9, empty_rows=[(0, 16), (32, 64)])
    f = convert(rows, cols, rp, ci, v)
    assert f.rowIdx.tolist() == [16, 64]


def test_duplicates_last_wins_and_unsorted_rows():
    # one row holding column 5 twice and columns out of order (convert.h:215 keeps the last write)
    rp = np.array([0, 4], np.uint32)
    ci = np.array([9, 5, 2, 5], np.uint32)
    v = np.array([1, 2, 3, 4], np.float16)
    f = convert(1, 16, rp, ci, v)
    g = oracle.csr2btcf_nobitmap(1, 16, rp, ci, v, 16, 16)
    assert same_format(f, g)
    assert f.tcA2B[:3].tolist() == [2, 5, 9] and f.data[:3].tolist() == [3.0, 4.0, 1.0]


def test_padding_and_zero_fill():
    rows, cols, rp, ci, v = random_csr(37, 100, 0.1, 4)
    f = convert(rows, cols, rp, ci, v)
    a2b = f.tcA2B.reshape(-1, 16)
    for w in range(f.eff_row_windows):
        lst = a2b[f.rowOffset[w]:f.rowOffset[w + 1]].ravel()
        real = lst[lst != hs.IDX_MAX]
        assert np.all(np.diff(real.astype(np.int64)) > 0)            # ascending, distinct
        assert np.all(lst[len(real):] == hs.IDX_MAX)                 # padding only at the end
    # the last window has 5 real rows: rows 5..15 of its tiles are zero
    last = f.data.reshape(-1, 16, 16)[f.rowOffset[-2]:]
    assert np.all(last[:, 5:, :] == 0)
    assert np.count_nonzero(f.data) == np.count_nonzero(v)


def test_bad_csr_is_rejected():
    rows, cols, rp, ci, v = random_csr(20, 20, 0.3, 1)
    for mutate in ("nonmonotone", "col", "nnz"):
        rp2, ci2 = rp.copy(), ci.copy()
        if mutate == "nonmonotone":
            rp2[5], rp2[6] = rp2[6] + 1, rp2[5]
        elif mutate == "col":
            ci2[3] = 20
        else:
            rp2[-1] += 1
        with pytest.raises(capi.SpmmError) as e:
            convert(rows, cols, rp2, ci2, v)
        assert e.value.status == capi.ERR_BAD_CSR
    with pytest.raises(capi.SpmmError) as e:
        convert(rows, cols, rp, ci, v, rw=12)
    assert e.value.status == capi.ERR_INVALID_ARG


def test_shard_rows_is_nnz_balanced():
    rows, cols, rp, ci, v = random_csr(1000, 300, 0.05, 2, dense_rows=list(range(0, 40)))
    for parts in (1, 2, 4, 8):
        cuts = hs.shard_rows(rows, rp, parts)
        assert cuts[0] == 0 and cuts[-1] == rows and np.all(np.diff(cuts.astype(np.int64)) >= 0)
        assert all(c % 16 == 0 or c == rows for c in cuts)
        nnz = np.diff(rp[cuts.astype(np.int64)].astype(np.int64))
        window_max = max(int(rp[min(rows, r + 16)]) - int(rp[r]) for r in range(0, rows, 16))
        assert nnz.sum() == len(ci) and nnz.max() - len(ci) / parts <= window_max


def test_sharded_conversion_concatenates():
    rows, cols, rp, ci, v = random_csr(400, 200, 0.04, 7, empty_rows=[(64, 96)])
    whole = convert(rows, cols, rp, ci, v)
    cuts = hs.shard_rows(rows, rp, 4).astype(np.int64)
    per_window, a2b, data, ridx = [], [], [], []
    for p in range(4):
        r0, r1 = cuts[p], cuts[p + 1]
        lo, hi = int(rp[r0]), int(rp[r1])
        part = convert(r1 - r0, cols, rp[r0:r1 + 1] - lo, ci[lo:hi], v[lo:hi])
        per_window += np.diff(part.rowOffset.astype(np.int64)).tolist()
        a2b.append(np.array(part.tcA2B)); data.append(np.array(part.data)); ridx.append(np.array(part.rowIdx) + r0)
    assert per_window == np.diff(whole.rowOffset.astype(np.int64)).tolist()
    assert np.array_equal(np.concatenate(a2b), whole.tcA2B)
    assert np.array_equal(np.concatenate(data).view(np.uint16), np.array(whole.data).view(np.uint16))
    assert np.array_equal(np.concatenate(ridx), whole.rowIdx)


def test_schedule_covers_every_window_once_and_balances_tiles():
    rng = np.random.default_rng(0)
    for eff, n_ctas in ((0, 4), (1, 148), (50, 148), (5000, 148), (5000, 7)):
        tiles = rng.integers(1, 40, eff)
        if eff > 10:
            tiles[:3] = 2000  # hub windows
        row_offset = np.concatenate([[0], np.cumsum(tiles)]).astype(np.uint32)
        cuts = np.zeros(n_ctas + 1, np.uint32)
        st = capi.lib().b200spmm_build_schedule(row_offset.ctypes.data, eff, n_ctas, cuts.ctypes.data)
        assert st == capi.OK
        assert cuts[0] == 0 and cuts[-1] == eff and np.all(np.diff(cuts.astype(np.int64)) >= 0)
        if eff >= n_ctas * 4:
            charge = 12  # tile-equivalents per window in the schedule's cost model
            load = np.diff(row_offset[cuts].astype(np.int64)) + charge * np.diff(cuts.astype(np.int64))
            assert load.max() <= (row_offset[-1] + charge * eff) / n_ctas + tiles.max() + charge


def test_tile_schedule_covers_every_tile_once_and_accounts_for_every_piece():
    rng = np.random.default_rng(1)
    for eff, n_ctas in ((0, 4), (1, 148), (3, 16), (50, 148), (5000, 148), (5000, 7), (40000, 148)):
        tiles = rng.integers(1, 40, eff)
        if eff > 10:
            tiles[:3] = (30000, 2000, 700)  # hub windows, the first far heavier than one CTA's share
        if eff == 1:
            tiles[:] = 5000
        row_offset = np.concatenate([[0], np.cumsum(tiles)]).astype(np.uint32)
        total = int(row_offset[-1])
        cta_tile = np.zeros(n_ctas + 1, np.uint32)
        wfirst = np.zeros(n_ctas, np.uint32)
        wlast = np.zeros(n_ctas, np.uint32)
        slot_window = np.zeros(2 * n_ctas, np.uint32)
        st = capi.lib().b200spmm_build_tile_schedule(row_offset.ctypes.data, eff, n_ctas, cta_tile.ctypes.data,
                                                     wfirst.ctypes.data, wlast.ctypes.data, slot_window.ctypes.data)
        assert st == capi.OK
        t = cta_tile.astype(np.int64)
        assert t[0] == 0 and t[-1] == total and np.all(np.diff(t) >= 0)
        expect_slot = np.full(2 * n_ctas, 0xFFFFFFFF, np.uint32)
        for c in range(n_ctas):
            if t[c + 1] == t[c]:
                continue
            wf = int(np.searchsorted(row_offset, t[c], side="right")) - 1
            wl = int(np.searchsorted(row_offset, t[c + 1] - 1, side="right")) - 1
            assert (wfirst[c], wlast[c]) == (wf, wl)
            head = row_offset[wf] < t[c]
            tail = row_offset[wl + 1] > t[c + 1]
            if head:
                expect_slot[2 * c] = wf
            if tail and not (head and wf == wl):  # a piece cut on both sides sits in the head slot
                expect_slot[2 * c + 1] = wl
        assert np.array_equal(slot_window, expect_slot)
        if eff:
            charge = 12
            load = np.diff(t) + charge * (wlast.astype(np.int64) - wfirst + 1) * (np.diff(t) > 0)
            share = (total + charge * eff) / n_ctas
            slack = max(32, total // n_ctas // 16) + 3 * charge
            assert load.max() <= share + slack, (eff, n_ctas, load.max(), share)


def test_row_bands_cut_only_between_windows_and_cover_all_rows():
    rng = np.random.default_rng(5)
    for eff, n_parts, want in ((0, 8, 4), (3, 16, 8), (5000, 148 * 16, 8), (5000, 7, 8), (40000, 296 * 16, 8)):
        tiles = rng.integers(1, 40, eff)
        if eff > 10:
            tiles[:3] = (30000, 2000, 700)
        row_offset = np.concatenate([[0], np.cumsum(tiles)]).astype(np.uint32)
        # windows 16 rows apart with some empty windows in between
        row_idx = (np.cumsum(rng.integers(1, 3, eff)) * 16).astype(np.uint32) if eff else np.zeros(0, np.uint32)
        rows = int(row_idx[-1]) + 40 if eff else 100
        band_chunk = np.zeros(want + 1, np.uint32)
        band_row = np.zeros(want + 1, np.uint64)
        n_bands = C.c_int()
        st = capi.lib().b200spmm_build_row_bands(row_offset.ctypes.data, row_idx.ctypes.data, eff, rows, n_parts, want,
                                                 band_chunk.ctypes.data, band_row.ctypes.data, C.byref(n_bands))
        assert st == capi.OK and 1 <= n_bands.value <= want
        nb = n_bands.value
        bc, br = band_chunk[:nb + 1].astype(np.int64), band_row[:nb + 1].astype(np.int64)
        assert bc[0] == 0 and bc[-1] == n_parts and np.all(np.diff(bc) > 0)
        assert br[0] == 0 and br[-1] == rows and np.all(np.diff(br) > 0)
        cta_tile = np.zeros(n_parts + 1, np.uint32)
        wfirst, wlast = np.zeros(n_parts, np.uint32), np.zeros(n_parts, np.uint32)
        slot_window = np.zeros(2 * n_parts, np.uint32)
        capi.lib().b200spmm_build_tile_schedule(row_offset.ctypes.data, eff, n_parts, cta_tile.ctypes.data,
                                                wfirst.ctypes.data, wlast.ctypes.data, slot_window.ctypes.data)
        for k in range(1, nb):
            c = int(bc[k])
            assert cta_tile[c] == row_offset[wfirst[c]], "a band starts at the first tile of a window"
            assert slot_window[2 * c] == 0xFFFFFFFF and br[k] == row_idx[wfirst[c]]
        if eff >= 5000 and n_parts >= 148 * 16:
            assert nb == want


def rewound(f, rw_out=16, rows=None, threads=0):
    return hs.rewindow(f.rows if rows is None else rows, f.cols, f.nnzs, f.rowOffset, f.tcA2B, f.data, f.rowIdx,
                       row_window_in=f.row_window, row_window=rw_out, n_threads=threads)


@pytest.mark.parametrize("flavour", ["fp16", "tf32"])
@pytest.mark.parametrize("case", ["hand", "rand_a", "rand_b"])
def test_reference_built_format_rewindows_to_the_direct_conversion(flavour, case):
    # the arrays the reference's own CSR2BTCFNOBITMAP produced (8-row windows), brought to 16 rows
    g = np.load(os.path.join(GOLDEN, f"format_ref_{flavour}.npz"))
    rows, cols = (int(x) for x in g[f"{case}_shape"])
    rp, ci, v = g[f"{case}_row_ptr"], g[f"{case}_col_idx"], g[f"{case}_values"]
    f16 = hs.rewindow(rows, cols, len(ci), g[f"{case}_rowOffset"], g[f"{case}_tcA2B"], g[f"{case}_data"],
                      g[f"{case}_rowIdx"], row_window_in=8, row_window=16)
    direct = convert(rows, cols, rp, ci, v, rw=16)
    assert same_format(f16, direct)
    assert (f16.row_window, f16.col_window, f16.total_row_windows) == (16, direct.col_window, (rows + 15) // 16)
    assert same_format(f16, oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, 16, direct.col_window))


@pytest.mark.parametrize("dt,cw", [(np.float16, 16), (np.float32, 8), (np.float32, 4)])
def test_rewindow_random_matrices(dt, cw):
    shapes = [(1, 1, 1.0), (9, 40, 0.3), (16, 16, 0.5), (23, 33, 0.2), (203, 517, 0.03), (500, 70000, 0.0005), (96, 7, 0.6)]
    for seed, (rows, cols, dens) in enumerate(shapes):
        rows, cols, rp, ci, v = random_csr(rows, cols, dens, seed, dt,
                                           empty_rows=[(16, 48), (56, 64), (96, 104)] if rows > 104 else (),
                                           dense_rows=[3] if cols < 1000 and rows > 3 else ())
        v = v.copy()
        v[::7] = 0  # stored zeros keep their column
        f8 = convert(rows, cols, rp, ci, v, 8, cw)
        assert same_format(rewound(f8, 16, threads=seed % 3), convert(rows, cols, rp, ci, v, 16, cw))
        assert same_format(rewound(f8, 8), f8)


def test_rewindow_of_an_empty_format_and_bad_input():
    f8 = convert(40, 10, np.zeros(41, np.uint32), np.zeros(0, np.uint32), np.zeros(0, np.float16), rw=8)
    f16 = rewound(f8)
    assert (f16.eff_row_windows, f16.total_tiles, f16.total_row_windows) == (0, 0, 3)
    rows, cols, rp, ci, v = random_csr(64, 50, 0.1, 5)
    f8 = convert(rows, cols, rp, ci, v, rw=8)

    def broken(**kw):
        a = {k: np.array(getattr(f8, k)) for k in FORMAT_FIELDS}
        for k, fn in kw.items():
            fn(a[k])
        with pytest.raises(RuntimeError):
            hs.rewindow(rows, cols, f8.nnzs, a["rowOffset"], a["tcA2B"], a["data"], a["rowIdx"], 8, 16)

    def swap_first_two(x):
        x[[0, 1]] = x[[1, 0]]

    def set_first(value):
        def fn(x):
            x[0] = value
        return fn

    broken(tcA2B=swap_first_two)              # columns of a window must ascend
    broken(tcA2B=set_first(cols))             # column past the matrix
    broken(rowIdx=set_first(3))               # windows start on multiples of the input height
    broken(rowIdx=swap_first_two)             # windows must ascend
    broken(rowOffset=set_first(1))            # rowOffset starts at zero
    with pytest.raises(RuntimeError):         # 16 -> 8 is not a re-windowing
        rewound(convert(rows, cols, rp, ci, v, rw=16), 8)



@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("rw_out", [32, 64, 128])
def test_rewindow_to_taller_windows_equals_a_direct_conversion(dt, rw_out):
    # the merge the plan applies on the device for its 128-row kernel, here on the host: the same arrays as
    # the converter's algorithm (src/utils/convert.h:146-225) at that window height
    rows, cols, rp, ci, v = random_csr(715, 900, 0.02, 5, dt, empty_rows=[(0, 130), (256, 384), (600, 640)], dense_rows=[140, 700])
    cw = 16 if dt == np.float16 else 8
    f16 = convert(rows, cols, rp, ci, v, rw=16)
    tall = hs.rewindow(rows, cols, len(ci), f16.rowOffset, f16.tcA2B, f16.data, f16.rowIdx, row_window_in=16, row_window=rw_out)
    want = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, rw_out, cw)
    assert same_format(tall, want) and tall.row_window == rw_out


@pytest.mark.parametrize("dt,rw", [(np.float16, 8), (np.float16, 16), (np.float32, 8), (np.float32, 16)])
def test_column_major_tiles_of_the_transposed_build(dt, rw):
    # SPARSE_A_TRANSPOSE (src/utils/convert.h:207-213): the same lists and offsets, every tile stored column
    # by column.  The library reaches it by rewriting a converted format in place; doing so twice gives the
    # row-major format back, and a plan refuses column-major tiles whatever the device.
    from cases import random_csr
    import oracle
    rows, cols, rp, ci, v = random_csr(203, 300, 0.04, 3, dt, empty_rows=[(16, 40)], dense_rows=[77])
    cw = 16 if dt == np.float16 else 8
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=rw)
    row_major = np.array(f.data).copy()
    bits = np.uint16 if dt == np.float16 else np.uint32
    want = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, rw, cw, col_major_tiles=True)
    hs.transpose_tiles(f)
    assert f.col_major_tiles
    assert np.array_equal(np.asarray(f.data).view(bits), np.asarray(want.data).view(bits))
    for k in ("rowOffset", "tcA2B", "rowIdx"):
        assert np.array_equal(getattr(f, k), getattr(want, k)), k
    p = C.c_void_p()
    assert capi.lib().b200spmm_plan_create(f._h, 0, 0, C.byref(p)) == capi.ERR_UNSUPPORTED
    hs.transpose_tiles(f)
    assert not f.col_major_tiles and np.array_equal(np.asarray(f.data).view(bits), row_major.view(bits))
