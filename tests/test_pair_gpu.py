"""The CTA-pair path on the device: 256-row super-windows multiplied by clusters of two CTAs that share one
MMA of 256 window rows x 256 features (tcgen05.mma.cta_group::2).  The merged format against a conversion
at 256 rows (the reference's algorithm, src/utils/convert.h:146-225, at ROW_WINDOW = 256) and the kernel
against the CPU oracle.  Small matrices are sent down this path with B200SPMM_WINDOW=256."""
import numpy as np
import pytest

import hopper_spmm_b200 as hs
import oracle
import parity
from cases import dense_b, random_csr

pytestmark = pytest.mark.gpu


@pytest.fixture
def pair(monkeypatch):
    monkeypatch.setenv("B200SPMM_WINDOW", "256")


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_merged_format_equals_a_conversion_at_256_rows(dt, pair):
    rows, cols, rp, ci, v = random_csr(1100, 900, 0.02, 5, dt, empty_rows=[(0, 130), (256, 512), (900, 960)], dense_rows=[140, 700])
    v = v.copy()
    v[::9] = 0  # explicit zeros keep their column
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        got = plan.tall_format(256)
    finally:
        plan.close()
    cw = 16 if dt == np.float16 else 8
    want = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, 256, cw)
    assert got is not None and got["row_window"] == 256
    assert got["eff_row_windows"] == want.eff_row_windows and got["total_tiles"] == want.total_tiles
    for k in ("rowOffset", "tcA2B", "rowIdx"):
        assert np.array_equal(got[k], getattr(want, k)), k
    bits = np.uint16 if dt == np.float16 else np.uint32
    assert np.array_equal(got["data"].view(bits), np.asarray(want.data).view(bits))


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("n", [136, 256, 320, 520])
def test_ragged_matrix_every_slab_width(dt, n, pair):
    import torch
    rows, cols, rp, ci, v = random_csr(1100, 517, 0.03, 11, dt, empty_rows=[(0, 130), (256, 512), (1000, 1100)], dense_rows=[140])
    B = dense_b(cols, n, 3, dt)
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        dC = torch.full((rows, n), float("nan"), device="cuda")  # every row must be written
        plan.spmm(torch.from_numpy(B).cuda(), dC)
        info = plan.launch_info()
        assert info.row_window == 256 and info.feature_slab == 256 and info.kernel_launches == 1
        C_out = dC.cpu().numpy()
        parity.check(C_out, rows, rp, ci, v, B)
        assert np.all(C_out[0:130] == 0) and np.all(C_out[256:512] == 0) and np.all(C_out[1000:] == 0)
        half = plan.spmm_host(B, c_half=True)
        assert half.dtype == np.float16 and np.array_equal(half, C_out.astype(np.float16))
    finally:
        plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_same_bits_as_the_128_row_kernel(dt, monkeypatch):
    # both kernels add a row's products in ascending column order, one tile of CW columns per MMA: merging
    # two 128-row windows moves columns between tiles, so results agree to rounding, and exactly where both
    # window heights give a row the same tiles - a matrix whose windows hold every column
    import torch
    rows, cols = 1024, 640
    rows_, cols_, rp, ci, v = random_csr(rows, cols, 0.05, 31, dt, dense_rows=list(range(3, rows, 128)))
    B = torch.from_numpy(dense_b(cols, 512, 4, dt)).cuda()
    out = {}
    for win in ("128", "256"):
        monkeypatch.setenv("B200SPMM_WINDOW", win)
        plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
        try:
            out[win] = plan.spmm(B).cpu().numpy()
            assert plan.launch_info().row_window == int(win)
        finally:
            plan.close()
    assert np.array_equal(out["128"], out["256"])
    parity.check(out["256"], rows, rp, ci, v, B.cpu().numpy())


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_more_items_than_pairs_and_strided_operands(dt, pair):
    # 40 super-windows x 4 slabs = 160 work items on at most 74 pairs: the run-time hand-out is used (the
    # even CTA writes the item into the odd CTA's list); B and C are views with larger leading dimensions
    import torch
    rows, cols, rp, ci, v = random_csr(10240, 300, 0.04, 17, dt, empty_rows=[(2560, 2830)])
    n = 1024
    Bfull = torch.from_numpy(dense_b(cols, n + 64, 8, dt)).cuda()
    Cfull = torch.zeros((rows, n + 128), device="cuda")
    Bv, Cv = Bfull[:, 32:32 + n], Cfull[:, 64:64 + n]
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        for _ in range(2):  # the hand-out counters must be back at zero for the second launch
            Cv.fill_(float("nan"))
            plan.spmm(Bv, Cv)
            assert plan.launch_info().row_window == 256 and plan.launch_info().n_slabs == 4
            parity.check(Cv.cpu().numpy(), rows, rp, ci, v, Bv.cpu().numpy())
        assert float(Cfull[:, :64].abs().sum()) == 0 and float(Cfull[:, 64 + n:].abs().sum()) == 0
    finally:
        plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_dense_windows_take_packed_rows_of_b(dt, pair):
    # every super-window holds a full row: all tiles but the ragged last one name an aligned group of rows
    # of B and are fed from the per-launch images of B (128-feature blocks, one per CTA of the pair)
    import torch
    n = 328
    rows, cols = 1300, 1000 + (8 if dt == np.float32 else 16) // 2
    rows_, cols_, rp, ci, v = random_csr(rows, cols, 0.01, 23, dt, empty_rows=[(256, 512)], dense_rows=[5, 130, 600, 800, 1030, 1290])
    Bfull = torch.from_numpy(dense_b(cols, n + 72, 9, dt)).cuda()
    Bv = Bfull[:, 8:8 + n]
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        dC = torch.full((rows, n), float("nan"), device="cuda")
        plan.spmm(Bv, dC)
        info = plan.launch_info()
        assert info.row_window == 256 and info.kernel_launches == 2
        parity.check(dC.cpu().numpy(), rows, rp, ci, v, Bv.cpu().numpy())
    finally:
        plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_starved_pipeline_times_out_and_the_plan_recovers(dt, pair):
    # A failure made on the host: every stage expects sixteen bytes more than its loads deliver, so no stage
    # ever fills.  With waits limited to 5 ms every role of the kernel has to leave its loop by itself, tensor
    # memory is released, the status says so, and the next launch of the same plan is a normal, correct product.
    import time
    import torch
    from hopper_spmm_b200 import _capi as capi
    rows, cols, rp, ci, v = random_csr(1100, 517, 0.03, 11, dt, empty_rows=[(256, 512)], dense_rows=[140])
    n = 320
    B = torch.from_numpy(dense_b(cols, n, 3, dt)).cuda()
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        dC = torch.zeros((rows, n), device="cuda")
        s = torch.cuda.current_stream().cuda_stream
        lib = capi.lib()
        assert lib.b200spmm_kat_spmm_starved(plan._p, B.data_ptr(), n, n, dC.data_ptr(), n, 5_000_000, s) == 0
        assert plan.launch_info().row_window == 256
        t0 = time.perf_counter()
        assert lib.b200spmm_plan_sync(plan._p, s) == capi.ERR_DEVICE_TIMEOUT
        assert time.perf_counter() - t0 < 5.0
        for _ in range(2):  # tensor memory was released and the hand-out counters are back at zero
            dC = torch.full((rows, n), float("nan"), device="cuda")
            plan.spmm(B, dC)
            assert plan.launch_info().row_window == 256
            parity.check(dC.cpu().numpy(), rows, rp, ci, v, B.cpu().numpy())
    finally:
        plan.close()


@pytest.mark.parametrize("window", ["128", "256"])
def test_random_shapes_against_the_oracle(window, monkeypatch):
    # twenty seeded shapes per kernel: ragged row and column counts, empty stretches, full rows, feature counts
    # that leave the last slab (and, for the pair kernel, the odd CTA's half of it) partly or wholly empty, both
    # element types, fp32 and fp16 C.  Every row must be written, two launches must give the same bits, fp16 C
    # is the rounded fp32 C.
    import torch
    monkeypatch.setenv("B200SPMM_WINDOW", window)
    rng = np.random.default_rng(int(window))
    ran = set()
    for case in range(20):
        dt = [np.float16, np.float32][rng.integers(2)]
        rows, cols = int(rng.integers(1, 6000)), int(rng.integers(1, 1200))
        dens = float(10 ** rng.uniform(-3, -0.7))
        n = int(rng.choice([64, 128, 136, 192, 256, 264, 320, 520, 776]))
        dense_rows = sorted(set(int(x) for x in rng.integers(0, rows, int(rng.integers(0, 4)))))
        empties = []
        if rows > 600 and rng.random() < 0.6:
            a = int(rng.integers(0, rows - 32))
            empties = [(a, min(rows, a + int(rng.integers(1, 900))))]
        seed = int(rng.integers(1 << 30))
        c_half = bool(rng.integers(2))
        rows_, cols_, rp, ci, v = random_csr(rows, cols, dens, seed, dt, empty_rows=empties, dense_rows=dense_rows)
        B = torch.from_numpy(dense_b(cols, n, seed + 1, dt)).cuda()
        tag = f"case {case}: {dt.__name__} rows={rows} cols={cols} dens={dens:.4g} n={n} dense={dense_rows} empty={empties} c_half={c_half}"
        plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
        try:
            dC = torch.full((rows, n), float("nan"), device="cuda", dtype=torch.float16 if c_half else torch.float32)
            plan.spmm(B, dC, c_half=c_half)
            ran.add(plan.launch_info().row_window)
            out = dC.float().cpu().numpy()
            assert np.isfinite(out).all(), tag
            out32 = plan.spmm(B).cpu().numpy()
            assert np.array_equal(plan.spmm(B).cpu().numpy().view(np.uint32), out32.view(np.uint32)), tag
            if c_half:
                assert np.array_equal(out.astype(np.float16).view(np.uint16), out32.astype(np.float16).view(np.uint16)), tag
            parity.check(out32, rows, rp, ci, v, B.cpu().numpy())
        finally:
            plan.close()
    assert int(window) in ran
