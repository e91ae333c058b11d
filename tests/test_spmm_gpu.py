"""End-to-end parity on the device, through the C ABI: the converted matrix goes to the GPU,
the sm_100a kernel computes C, and C is compared with the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

import hopper_spmm_b200 as hs
import parity
from cases import dense_b, random_csr
from hopper_spmm_b200 import _capi as capi
from hopper_spmm_b200 import synth

pytestmark = pytest.mark.gpu


def run_host(rows, cols, rp, ci, v, B, c_half=False, n_ctas=0):
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
    plan = hs.SpmmPlan(f, n_ctas=n_ctas)
    try:
        out = plan.spmm_host(B, c_half=c_half)
        return out, plan.launch_info()
    finally:
        plan.close()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("n", [8, 64, 128, 192, 256, 320, 520])
def test_ragged_matrix_every_slab_width(dt, n):
    rows, cols, rp, ci, v = random_csr(203, 517, 0.03, 11, dt, empty_rows=[(48, 96)], dense_rows=[7])
    B = dense_b(cols, n, 3, dt)
    C_out, info = run_host(rows, cols, rp, ci, v, B)
    parity.check(C_out, rows, rp, ci, v, B)
    assert np.all(C_out[48:96] == 0)
    assert info.kernel_launches in (1, 2) and info.feature_slab == min(128, (n + 63) // 64 * 64)


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_single_entry_and_single_tile(dt):
    rp = np.zeros(17, np.uint32)
    rp[6:] = 1
    ci, v = np.array([3], np.uint32), np.array([2.0], dt)
    B = dense_b(9, 128, 0, dt)
    C_out, _ = run_host(16, 9, rp, ci, v, B)
    b_seen = B[3].astype(np.float32)
    if dt == np.float32:  # the tensor core reads fp32 operands as tf32: low 13 mantissa bits dropped
        b_seen = (b_seen.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    expect = np.zeros((16, 128), np.float32)
    expect[5] = 2.0 * b_seen
    assert np.array_equal(C_out, expect)


def test_empty_matrix_gives_zeros():
    rp = np.zeros(41, np.uint32)
    C_out, _ = run_host(40, 10, rp, np.zeros(0, np.uint32), np.zeros(0, np.float16), dense_b(10, 64, 0))
    assert C_out.shape == (40, 64) and np.all(C_out == 0)


def test_leading_and_trailing_empty_windows_are_cleared():
    rows, cols, rp, ci, v = random_csr(400, 64, 0.2, 5, empty_rows=[(0, 64), (350, 400)])
    B = dense_b(cols, 128, 1)
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
    import torch
    plan = hs.SpmmPlan(f)
    dB = torch.from_numpy(B).cuda()
    dC = torch.full((rows, 128), float("nan"), device="cuda")  # poison: every row must be written
    plan.spmm(dB, dC)
    parity.check(dC.cpu().numpy(), rows, rp, ci, v, B)
    plan.close()


def test_long_windows_wrap_the_ring_many_times():
    # 5000 distinct columns in one window = 313 tiles through a 40-stage ring
    rows, cols, rp, ci, v = random_csr(64, 5000, 0.4, 6, dense_rows=[0, 17, 40])
    B = dense_b(cols, 128, 2)
    C_out, _ = run_host(rows, cols, rp, ci, v, B)
    parity.check(C_out, rows, rp, ci, v, B)


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("n,c_half", [(64, False), (320, False), (128, True)])
def test_hub_windows_are_shared_between_ctas(dt, n, c_half):
    # three windows far heavier than one CTA's share (the last one ragged: 203 rows), between light
    # ones and an empty stretch: their pieces go through the partial-result slots and the fix-up kernel
    rows, cols, rp, ci, v = random_csr(203, 6000, 0.004, 21, dt, empty_rows=[(64, 96)], dense_rows=[3, 120, 200])
    B = dense_b(cols, n, 4, dt)
    for n_ctas in (0, 5, 37):
        C_out, info = run_host(rows, cols, rp, ci, v, B, c_half=c_half, n_ctas=n_ctas)
        assert info.kernel_launches == 2
        parity.check(C_out.astype(np.float32), rows, rp, ci, v, B)
        assert np.all(C_out[64:96] == 0)


def test_hub_windows_leave_no_row_unwritten():
    # the same kind of matrix through the device-pointer call into a C full of NaN: the rows of split
    # windows come from the fix-up kernel, the gaps after them from the epilogue's zero fill
    import torch
    rows, cols, rp, ci, v = random_csr(203, 6000, 0.004, 21, empty_rows=[(64, 96), (128, 144)], dense_rows=[3, 120, 200])
    B = dense_b(cols, 128, 4)
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)), n_ctas=37)
    try:
        dC = torch.full((rows, 128), float("nan"), device="cuda")
        plan.spmm(torch.from_numpy(B).cuda(), dC)
        assert plan.launch_info().kernel_launches == 2
        parity.check(dC.cpu().numpy(), rows, rp, ci, v, B)
    finally:
        plan.close()


@pytest.mark.parametrize("case", ["small fp16", "small tf32", "chunks handed out at run time"])
def test_starved_pipeline_times_out_and_the_plan_recovers(case):
    # A failure made on the host: B's tensor map delivers half the bytes every stage barrier expects,
    # so no stage ever completes.  With waits limited to 5 ms the kernel has to unwind by itself (the
    # reference would spin for ever, src/ptx/barrier.h:29-41); the status says so, and the next launch
    # of the same plan is a normal, correct product.
    import time
    import torch
    if case.startswith("small"):
        dt = np.float16 if case.endswith("fp16") else np.float32
        rows, cols, rp, ci, v = random_csr(203, 517, 0.03, 11, dt, dense_rows=[7])
        B = torch.from_numpy(dense_b(cols, 128, 3, dt)).cuda()
    else:
        csr, B = synth.make_config("rmat24_sharded_fp16", 0, "cuda", 6)  # enough tiles for several chunks per CTA
        rows, cols = csr.rows, csr.cols
        rp, ci, v = csr.numpy()
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        n = B.shape[1]
        dC = torch.zeros((rows, n), device="cuda")
        s = torch.cuda.current_stream().cuda_stream
        lib = capi.lib()
        assert lib.b200spmm_kat_spmm_starved(plan._p, B.data_ptr(), n, n, dC.data_ptr(), n, 5_000_000, s) == 0
        t0 = time.perf_counter()
        assert lib.b200spmm_plan_sync(plan._p, s) == capi.ERR_DEVICE_TIMEOUT
        assert time.perf_counter() - t0 < 5.0
        for _ in range(2):  # tensor memory was released and the hand-out counters are back at zero
            dC = torch.full((rows, n), float("nan"), device="cuda")
            plan.spmm(B, dC)
            parity.check(dC.cpu().numpy(), rows, rp, ci, v, B.cpu().numpy())
    finally:
        plan.close()


def test_more_ctas_than_windows_and_one_cta():
    rows, cols, rp, ci, v = random_csr(96, 300, 0.1, 8)
    B = dense_b(cols, 64, 4)
    for n_ctas in (1, 3, 148, 500):
        C_out, info = run_host(rows, cols, rp, ci, v, B, n_ctas=n_ctas)
        parity.check(C_out, rows, rp, ci, v, B)
        assert info.n_ctas == n_ctas


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("n", [64, 128, 320])
def test_compressed_tiles_give_the_same_bits_as_dense_tiles(dt, n, monkeypatch):
    # bitmap + stored values expanded by the producer warps (the shape of the reference's BTCF_MTX,
    # src/utils/class.h:55-67) against the dense 512-byte tiles; explicit zeros, -0.0, a full tile
    # ... and a window whose tiles are all full, rows with 2-3 entries per tile on average
    rows, cols, rp, ci, v = random_csr(331, 4000, 0.01, 33, dt, empty_rows=[(32, 80)], dense_rows=[5, 300] + list(range(160, 176)))
    v = v.copy()
    v[::7] = 0
    v[3::11] = -0.0
    B = dense_b(cols, n, 6, dt)
    # the same CTA count for both: a window that is shared between CTAs is summed from its pieces, and
    # where the cuts fall depends on the number of chunks
    monkeypatch.setenv("B200SPMM_TILES", "dense")
    dense, info_d = run_host(rows, cols, rp, ci, v, B, n_ctas=296)
    monkeypatch.setenv("B200SPMM_TILES", "bitmap")
    packed, info_b = run_host(rows, cols, rp, ci, v, B, n_ctas=296)
    assert info_d.bitmap_tiles == 0 and info_b.bitmap_tiles == 1
    assert np.array_equal(dense.view(np.uint32), packed.view(np.uint32))
    parity.check(packed, rows, rp, ci, v, B)
    # the tiles as records of 32 (position, value) words, expanded by a zero fill and one store per lane; tiles
    # with more than 32 entries still arrive dense (fp16 matrices only: a tf32 plan keeps its dense tiles)
    monkeypatch.setenv("B200SPMM_TILES", "entries")
    listed, info_e = run_host(rows, cols, rp, ci, v, B, n_ctas=296)
    assert info_e.bitmap_tiles == (2 if dt == np.float16 else 0)
    assert np.array_equal(dense.view(np.uint32), listed.view(np.uint32))


def test_fp16_output():
    rows, cols, rp, ci, v = random_csr(130, 200, 0.1, 9)
    B = dense_b(cols, 128, 5)
    c32, _ = run_host(rows, cols, rp, ci, v, B)
    c16, _ = run_host(rows, cols, rp, ci, v, B, c_half=True)
    assert c16.dtype == np.float16 and np.array_equal(c16, c32.astype(np.float16))


def test_strided_device_tensors_and_reference_protocol():
    import torch
    rows, cols, rp, ci, v = random_csr(300, 256, 0.05, 10)
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
    plan = hs.SpmmPlan(f)
    Bfull = torch.from_numpy(dense_b(cols, 256, 6)).cuda()
    Cfull = torch.zeros((rows, 512), device="cuda")
    Bv, Cv = Bfull[:, 64:192], Cfull[:, 128:256]          # ldb = 256, ldc = 512, 16-byte aligned views
    plan.spmm(Bv, Cv)
    parity.check(Cv.cpu().numpy(), rows, rp, ci, v, Bv.cpu().numpy())
    assert float(Cfull[:, :128].abs().sum()) == 0 and float(Cfull[:, 256:].abs().sum()) == 0
    perf = plan.bench(Bv.contiguous(), torch.empty((rows, 128), device="cuda"))
    assert perf.runs == hs.RUNS and perf.time > 0
    plan.close()


def test_unsupported_shapes_are_refused():
    import torch
    rows, cols, rp, ci, v = random_csr(32, 32, 0.2, 1)
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    B = torch.zeros((cols, 12), dtype=torch.float16, device="cuda")
    with pytest.raises(capi.SpmmError) as e:
        plan.spmm(B)
    assert e.value.status == capi.ERR_UNSUPPORTED
    with pytest.raises(capi.SpmmError):
        hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=8))
    plan.close()


def test_reference_operator_names():
    rows, cols, rp, ci, v = random_csr(100, 80, 0.1, 2)
    B = dense_b(cols, 128, 7)
    btcf = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
    Cm = hs.DENSE_MTX(rows, 128)
    perf = hs.fp16_spmm(btcf, hs.DENSE_MTX(cols, 128, B), Cm)
    assert perf.runs == 5
    parity.check(Cm.values, rows, rp, ci, v, B)
    with pytest.raises(TypeError):
        hs.tf32_spmm(btcf, hs.DENSE_MTX(cols, 128, B), Cm)


@pytest.mark.parametrize("name,k", [("uniform_4096_fp16", 0), ("blocks_16384_tf32", 0), ("rmat20_gnn_fp16", 0),
                                    ("pruned_llm_fp16", 0), ("rmat24_sharded_fp16", 5)])
def test_benchmark_configurations(name, k):
    # the first four at their full size, whole result against the CPU oracle; the 2^24-node graph is
    # checked at full size, on a row sample, by the benchmark itself and here at 2^19 nodes
    csr, B = synth.make_config(name, 0, "cuda", k)
    rp, ci, v = csr.numpy()
    Bn = B.cpu().numpy()
    C_out, _ = run_host(csr.rows, csr.cols, rp, ci, v, Bn)
    stats = parity.check(C_out, csr.rows, rp, ci, v, Bn)
    print(name, stats)


def test_rmat_rows_sum_to_one_at_scale(monkeypatch):
    # size-independent property: with values 1/deg(row) and B = ones, every non-empty row of C is 1
    import torch
    csr, _ = synth.make_config("rmat24_sharded_fp16", 0, "cuda", 4)  # 2^20 nodes, ~30M entries
    rp, ci, v = csr.numpy()
    f = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(csr.rows, csr.cols, rp, ci, v))
    plan = hs.SpmmPlan(f)
    B = torch.ones((csr.cols, 128), dtype=torch.float16, device="cuda")
    Cd = plan.spmm(B)
    deg = (csr.row_ptr[1:] - csr.row_ptr[:-1])
    want = (deg > 0).to(torch.float32)[:, None].expand(-1, 128)
    err = (Cd - want).abs().max().item()
    assert err < 2e-3, err  # 1/deg is rounded to fp16: relative 2^-11 per term
    # The host-buffer call of a matrix this large runs band after band and copies each band's rows of
    # C out while the next is computed: same bits as the device-resident call, for fp32 and fp16 C.
    Bn = torch.rand((csr.cols, 128), dtype=torch.float32, device="cuda").sub_(0.5).to(torch.float16)
    for c_half in (False, True):
        want_c = plan.spmm(Bn, c_half=c_half).cpu().numpy()
        got_c = plan.spmm_host(Bn.cpu().numpy(), c_half=c_half)
        assert plan.launch_info().kernel_launches > 2, "expected one launch per band"
        assert np.array_equal(got_c.view(np.uint16 if c_half else np.uint32), want_c.view(np.uint16 if c_half else np.uint32))
    # That call also cuts the features in two halves (the first half of C leaves while the second half of B
    # arrives): twice the launches of the call with the halves switched off, the same bits.
    split_launches = plan.launch_info().kernel_launches
    plan.close()
    monkeypatch.setenv("B200SPMM_HOST_SPLIT", "0")
    plan = hs.SpmmPlan(f)
    try:
        got_c = plan.spmm_host(Bn.cpu().numpy(), c_half=True)
        assert plan.launch_info().kernel_launches * 2 == split_launches
        assert np.array_equal(got_c.view(np.uint16), want_c.view(np.uint16))
    finally:
        plan.close()


def test_bitmap_format_feeds_the_spmm_after_expansion():
    # CSR2BTCF at the kernels' 16-row windows -> dense tiles -> plan -> product
    rows, cols, rp, ci, v = random_csr(300, 900, 0.02, 41, empty_rows=[(16, 48)], dense_rows=[100])
    B = dense_b(cols, 128, 7)
    f = hs.CSR2BTCF(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=16)
    plan = hs.SpmmPlan(f.expand())
    try:
        parity.check(plan.spmm_host(B), rows, rp, ci, v, B)
    finally:
        plan.close()


@pytest.mark.parametrize("flavour", ["fp16", "tf32"])
def test_format_built_by_the_reference_converter_feeds_the_spmm(flavour):
    # The committed arrays are the output of the reference's own CSR2BTCFNOBITMAP (8-row windows);
    # re-windowed to 16 rows they go through the plan like a format converted here, and the product
    # has the bits of the product from the direct conversion.
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", f"format_ref_{flavour}.npz"))
    for case in ("hand", "rand_a", "rand_b"):
        rows, cols = (int(x) for x in g[f"{case}_shape"])
        rp, ci, v = g[f"{case}_row_ptr"], g[f"{case}_col_idx"], g[f"{case}_values"]
        f = hs.rewindow(rows, cols, len(ci), g[f"{case}_rowOffset"], g[f"{case}_tcA2B"], g[f"{case}_data"],
                        g[f"{case}_rowIdx"], row_window_in=8)
        B = dense_b(cols, 72, 13, v.dtype)
        plan = hs.SpmmPlan(f)
        try:
            out = plan.spmm_host(B)
        finally:
            plan.close()
        parity.check(out, rows, rp, ci, v, B)
        direct, _ = run_host(rows, cols, rp, ci, v, B)
        assert np.array_equal(out.view(np.uint8), direct.view(np.uint8))


@pytest.mark.parametrize("kind", ["fp16", "tf32", "fp16 rw8", "tf32 rw8"])
def test_command_line_run_on_a_matrix_market_file(kind, tmp_path):
    # spmm_test <file> <N>: the reference's main (src/fp16.cu:283-319) with a result check added
    import os
    import subprocess
    rows, cols, rp, ci, v = random_csr(500, 400, 0.03, 42, np.float32)
    path = tmp_path / "m.mtx"
    with open(path, "w") as fh:
        fh.write("%%MatrixMarket matrix coordinate real general\n%d %d %d\n" % (rows, cols, len(ci)))
        for r in range(rows):
            for p in range(rp[r], rp[r + 1]):
                fh.write("%d %d %.6f\n" % (r + 1, ci[p] + 1, v[p]))
    exe = os.path.join(os.path.dirname(hs.__file__), "spmm_test")
    out = subprocess.run([exe, str(path), "64"] + kind.split(), capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "nonzeros: %d" % len(ci) in out.stdout and "SPMM mean time" in out.stdout and "(ok," in out.stdout
    assert ("8-row format:" in out.stdout) == kind.endswith("rw8") and "tiles (16x" in out.stdout


@pytest.mark.parametrize("window", ["16", "128", "256"])
def test_tf32_product_against_the_oracle_on_truncated_inputs(window, monkeypatch):
    # The 5e-3 bound of the tf32 configuration has to absorb the rounding of the inputs to tf32.  Against an
    # oracle that sees the inputs as the tensor core does (low 13 mantissa bits dropped; the reference's
    # in-shared-memory conversion is a no-op, src/ptx/ptx_utils.h:32-36) only the order of the fp32 additions
    # differs: the result must agree to 1e-5 of the magnitude sum, for all three kernels.
    import torch
    import oracle
    monkeypatch.setenv("B200SPMM_WINDOW", window)
    rows, cols, rp, ci, v = random_csr(1100, 900, 0.03, 19, np.float32, empty_rows=[(256, 512)], dense_rows=[140, 700])
    B = dense_b(cols, 320, 5, np.float32)
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        got = plan.spmm(torch.from_numpy(B).cuda()).cpu().numpy()
        assert plan.launch_info().row_window == int(window)
    finally:
        plan.close()
    seen = oracle.spmm_csr(rows, rp, ci, v, B, tf32_mode=1)
    mag = oracle.spmm_csr(rows, rp, ci, np.abs(v), np.abs(B))
    live = mag > 0
    tight = float((np.abs(got - seen)[live] / mag[live]).max())
    loose = float((np.abs(got - oracle.spmm_csr(rows, rp, ci, v, B))[live] / mag[live]).max())
    print(f"window {window}: error relative to the magnitude sum {tight:.2e} against truncated inputs, {loose:.2e} against fp32 inputs")
    assert tight < 1e-5 < loose < 5e-3
