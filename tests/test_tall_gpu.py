"""The 128-row super-window path on the device: the merged format against a conversion at 128 rows
(the reference's algorithm, src/utils/convert.h:146-225, at ROW_WINDOW = 128) and the wide-MMA kernel
against the CPU oracle.  Small matrices are sent down this path with B200SPMM_WINDOW=128; the pruned
weight matrix of the benchmark takes it by itself."""
import numpy as np
import pytest

import hopper_spmm_b200 as hs
import oracle
import parity
from cases import dense_b, random_csr
from hopper_spmm_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture
def tall(monkeypatch):
    monkeypatch.setenv("B200SPMM_WINDOW", "128")


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_merged_format_equals_a_conversion_at_128_rows(dt, tall):
    rows, cols, rp, ci, v = random_csr(715, 900, 0.02, 5, dt, empty_rows=[(0, 130), (256, 384), (600, 640)], dense_rows=[140, 700])
    v = v.copy()
    v[::9] = 0  # explicit zeros keep their column
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        got = plan.tall_format()
    finally:
        plan.close()
    cw = 16 if dt == np.float16 else 8
    want = oracle.csr2btcf_nobitmap(rows, cols, rp, ci, v, 128, cw)
    assert got is not None and got["row_window"] == 128
    assert got["eff_row_windows"] == want.eff_row_windows and got["total_tiles"] == want.total_tiles
    for k in ("rowOffset", "tcA2B", "rowIdx"):
        assert np.array_equal(got[k], getattr(want, k)), k
    bits = np.uint16 if dt == np.float16 else np.uint32
    assert np.array_equal(got["data"].view(bits), np.asarray(want.data).view(bits))


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("n", [64, 128, 192, 256, 320, 520])
def test_ragged_matrix_every_slab_width(dt, n, tall):
    import torch
    rows, cols, rp, ci, v = random_csr(715, 517, 0.03, 11, dt, empty_rows=[(0, 130), (256, 384), (600, 715)], dense_rows=[140])
    B = dense_b(cols, n, 3, dt)
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        dC = torch.full((rows, n), float("nan"), device="cuda")  # every row must be written
        plan.spmm(torch.from_numpy(B).cuda(), dC)
        info = plan.launch_info()
        assert info.row_window == 128 and info.feature_slab == (128 if n <= 128 else 256) and info.kernel_launches == 1
        C_out = dC.cpu().numpy()
        parity.check(C_out, rows, rp, ci, v, B)
        assert np.all(C_out[0:130] == 0) and np.all(C_out[256:384] == 0) and np.all(C_out[600:] == 0)
        half = plan.spmm_host(B, c_half=True)
        assert half.dtype == np.float16 and np.array_equal(half, C_out.astype(np.float16))
    finally:
        plan.close()


def test_narrow_b_and_explicit_cta_counts_stay_with_16_rows(tall):
    rows, cols, rp, ci, v = random_csr(300, 200, 0.05, 2)
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
    for n, n_ctas in ((32, 0), (128, 5)):
        B = dense_b(cols, n, 1)
        plan = hs.SpmmPlan(f, n_ctas=n_ctas)
        try:
            parity.check(plan.spmm_host(B), rows, rp, ci, v, B)
            assert plan.launch_info().row_window == 16
        finally:
            plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("n", [128, 328])
def test_dense_windows_take_packed_rows_of_b(dt, n, tall):
    # every super-window holds a full row, so its column list is 0 .. cols - 1: all tiles but the ragged last
    # one name an aligned group of rows of B and are fed from the per-launch images of B; both element types,
    # one and two feature slabs (the second one partial), B with a larger leading dimension
    import torch
    rows, cols = 700, 1000 + (8 if dt == np.float32 else 16) // 2  # the last tile of every window is ragged
    rows_, cols_, rp, ci, v = random_csr(rows, cols, 0.01, 23, dt, empty_rows=[(256, 384)], dense_rows=[5, 130, 400, 520, 650])
    Bfull = torch.from_numpy(dense_b(cols, n + 72, 9, dt)).cuda()
    Bv = Bfull[:, 8:8 + n]
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        dC = torch.full((rows, n), float("nan"), device="cuda")
        plan.spmm(Bv, dC)
        info = plan.launch_info()
        assert info.row_window == 128 and info.kernel_launches == 2
        parity.check(dC.cpu().numpy(), rows, rp, ci, v, Bv.cpu().numpy())
    finally:
        plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_more_items_than_ctas_and_strided_operands(dt, tall):
    # 40 super-windows x 4 slabs = 160 work items on 148 CTAs: the run-time hand-out is used; B and C are
    # views with larger leading dimensions
    import torch
    rows, cols, rp, ci, v = random_csr(5120, 300, 0.04, 17, dt, empty_rows=[(1280, 1410)])
    n = 1024
    Bfull = torch.from_numpy(dense_b(cols, n + 64, 8, dt)).cuda()
    Cfull = torch.zeros((rows, n + 128), device="cuda")
    Bv, Cv = Bfull[:, 32:32 + n], Cfull[:, 64:64 + n]
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        for _ in range(2):  # the hand-out counters must be back at zero for the second launch
            Cv.fill_(float("nan"))
            plan.spmm(Bv, Cv)
            assert plan.launch_info().row_window == 128 and plan.launch_info().n_slabs == 4
            parity.check(Cv.cpu().numpy(), rows, rp, ci, v, Bv.cpu().numpy())
        assert float(Cfull[:, :64].abs().sum()) == 0 and float(Cfull[:, 64 + n:].abs().sum()) == 0
    finally:
        plan.close()


def test_pruned_weight_matrix_chooses_super_windows_by_itself(monkeypatch):
    # a quarter-size pruned weight matrix: every 16-row window holds 81 % of the columns, eight of them
    # merged hardly more - the plan must pick the 128-row kernel without being told, a graph must not
    import torch
    csr, B = synth.make_config("pruned_llm_fp16", 0, "cuda", 1)
    rp, ci, v = csr.numpy()
    btcf = hs.DeviceBtcf(csr.rows, csr.cols, csr.row_ptr.to(torch.int32), csr.col_idx, csr.values)
    plan = hs.SpmmPlan(btcf)
    try:
        C_dev = plan.spmm(B)
        assert plan.launch_info().row_window == 256  # B is wider than 128 features: the CTA-pair kernel
        # nearly every tile names one aligned group of 16 rows of B: B is re-laid per launch (a second kernel)
        # and such tiles arrive by one bulk copy
        assert plan.launch_info().kernel_launches == 2
        parity.check(C_dev.cpu().numpy(), csr.rows, rp, ci, v, B.cpu().numpy())
    finally:
        plan.close()
    # the same product with B fetched through the tensor maps: where the rows come from changes no bit
    monkeypatch.setenv("B200SPMM_PACK_B", "0")
    plan = hs.SpmmPlan(btcf)
    try:
        C_maps = plan.spmm(B)
        assert plan.launch_info().kernel_launches == 1
        assert torch.equal(C_maps, C_dev)
    finally:
        plan.close()
    monkeypatch.delenv("B200SPMM_PACK_B")
    csr, B = synth.make_config("rmat20_gnn_fp16", 0, "cuda", 4)
    btcf = hs.DeviceBtcf(csr.rows, csr.cols, csr.row_ptr.to(torch.int32), csr.col_idx, csr.values)
    plan = hs.SpmmPlan(btcf)
    try:
        plan.spmm(B)
        assert plan.launch_info().row_window == 16 and plan.tall_format() is None
    finally:
        plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_starved_pipeline_times_out_and_the_plan_recovers(dt, tall):
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
        assert plan.launch_info().row_window == 128
        t0 = time.perf_counter()
        assert lib.b200spmm_plan_sync(plan._p, s) == capi.ERR_DEVICE_TIMEOUT
        assert time.perf_counter() - t0 < 5.0
        for _ in range(2):  # tensor memory was released and the hand-out counters are back at zero
            dC = torch.full((rows, n), float("nan"), device="cuda")
            plan.spmm(B, dC)
            assert plan.launch_info().row_window == 128
            parity.check(dC.cpu().numpy(), rows, rp, ci, v, B.cpu().numpy())
    finally:
        plan.close()
