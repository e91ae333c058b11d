"""Single-tile known answers on the device: the tcgen05.mma operand layouts, the M = 64 TMEM
layout, accumulation over tiles, and the TMA loads.  Counterparts of the reference's bring-up
programs src/test_fp16.cu (KAT-1), test/02.tma_and_wgmma (KAT-2), test/03.warp_specialized
(accumulation) and test/01.tma_copy_matrix (TMA box layout)."""
import numpy as np
import pytest

import kat_util as ku
import oracle

pytestmark = pytest.mark.gpu


def _image(gathered: bytes, tile: bytes):
    img = gathered + bytes((-len(gathered)) % 4096)
    b_off = len(img)
    return img + tile + bytes(8192), b_off


@pytest.mark.parametrize("tf32", [False, True])
@pytest.mark.parametrize("m", [128, 64])
def test_single_tile_product(tf32, m):
    dt, cw = (np.float32, 8) if tf32 else (np.float16, 16)
    rng = np.random.default_rng(m + tf32)
    feats = rng.integers(-8, 9, (m, cw)).astype(dt)   # gathered rows of B, [feature][k]
    tile = rng.integers(-8, 9, (16, cw)).astype(dt)   # 16 window rows x CW
    img, b_off = _image(ku.pack_gathered(feats), ku.pack_tile(tile))
    st, d = ku.run_umma(img, [ku.spmm_tile_mma(tf32, m, 0, b_off)])
    assert st == 0
    got = d if m == 128 else ku.m64_rows(d)
    assert np.array_equal(got, feats.astype(np.float32) @ tile.astype(np.float32).T)  # small integers: exact


@pytest.mark.parametrize("tf32", [False, True])
@pytest.mark.parametrize("n", [128, 256])
def test_super_window_tile_product(tf32, n):
    # The MMA of the 128-row kernel: the sparse tile (128 window rows x CW, K-major, 32-byte swizzle) is
    # operand A, the gathered rows of B (n features x CW, MN-major, 128-byte swizzle) operand B - the
    # reference's transposition (src/fp16.cu:147) undone.  D[row][feature], row = TMEM lane.
    from hopper_spmm_b200 import _capi as capi
    dt, cw = (np.float32, 8) if tf32 else (np.float16, 16)
    rng = np.random.default_rng(n + tf32)
    tile = rng.integers(-8, 9, (128, cw)).astype(dt)
    feats = rng.integers(-8, 9, (n, cw)).astype(dt)   # gathered rows of B, [feature][k]
    gathered = ku.pack_gathered(feats)
    img = ku.pack_tile(tile) + gathered + bytes(8192)
    idesc = capi.lib().b200spmm_kat_instr_desc(2 if tf32 else 0, 128, n, 0, 1)
    mma = capi.KatMma(a_off=0, a_lbo=16, a_sbo=256, a_swizzle=6, b_off=4096, b_lbo=1024 if tf32 else 2048,
                      b_sbo=512 if tf32 else 1024, b_swizzle=1 if tf32 else 2, idesc=idesc, d_col=0, accumulate=0,
                      kind=1 if tf32 else 0)
    st, d = ku.run_umma(img, [mma], n_cols=n)
    assert st == 0
    assert np.array_equal(d, tile.astype(np.float32) @ feats.astype(np.float32).T)  # small integers: exact


@pytest.mark.parametrize("tf32", [False, True])
def test_cta_pair_tile_product(tf32):
    # One MMA over a pair of CTAs (cta_group::2): M = 256 window rows (128 per CTA), N = 256 features of
    # which every CTA holds 128 in its own shared memory, K = one tile.  D rows 128 r .. come out of CTA r.
    import ctypes as C
    from hopper_spmm_b200 import _capi as capi
    dt, cw = (np.float32, 8) if tf32 else (np.float16, 16)
    rng = np.random.default_rng(7 + tf32)
    tile = rng.integers(-8, 9, (256, cw)).astype(dt)
    feats = rng.integers(-8, 9, (256, cw)).astype(dt)   # gathered rows of B, [feature][k]
    images = b""
    for r in range(2):
        img = ku.pack_tile(tile[128 * r:128 * r + 128]) + ku.pack_gathered(np.ascontiguousarray(feats[128 * r:128 * r + 128]))
        images += img + bytes(16384 - len(img))
    idesc = capi.lib().b200spmm_kat_instr_desc(2 if tf32 else 0, 256, 256, 0, 1)
    mma = capi.KatMma(a_off=0, a_lbo=16, a_sbo=256, a_swizzle=6, b_off=4096, b_lbo=1024 if tf32 else 2048,
                      b_sbo=512 if tf32 else 1024, b_swizzle=1 if tf32 else 2, idesc=idesc, d_col=0, accumulate=0,
                      kind=1 if tf32 else 0)
    out = np.zeros((2, 128, 256), np.float32)
    buf = np.frombuffer(images, np.uint8)
    st = capi.lib().b200spmm_kat_umma_pair(buf.ctypes.data, 16384, (capi.KatMma * 1)(mma), 1, 256, out.ctypes.data, 0)
    assert st == 0
    want = tile.astype(np.float32) @ feats.astype(np.float32).T
    assert np.array_equal(out.reshape(256, 256), want)  # small integers: exact


def test_kat1_fp16_values():
    # src/test_fp16.cu:407-415 re-expressed for the transposed mapping: the 64x16 operand
    # A[i] = half(i+1) plays the feature side (M = 64), the all-ones operand the window side.
    A = np.arange(1, 64 * 16 + 1, dtype=np.float32).astype(np.float16).reshape(64, 16)
    ones = np.ones((16, 16), np.float16)
    img, b_off = _image(ku.pack_gathered(A), ku.pack_tile(ones))
    st, d = ku.run_umma(img, [ku.spmm_tile_mma(False, 64, 0, b_off)])
    assert st == 0
    expect = oracle.tile_accumulate(A.astype(np.float32), ones.astype(np.float32), 64, 16, 16, 1)
    bad, _, _ = oracle.compare(ku.m64_rows(d), expect, 0.01)  # the reference's tolerance, test_fp16.cu:306
    assert bad == 0
    assert np.array_equal(expect[:, 0], A.astype(np.float32).sum(1))


def test_kat2_tf32_values():
    # test/02.tma_and_wgmma/tma_wgmma.cu:340-348: A[i] = i+1 (64x8), B[i] = 1 + 0.01 i
    A = np.arange(1, 64 * 8 + 1, dtype=np.float32).reshape(64, 8)
    Bm = np.zeros((16, 8), np.float32)
    Bm[:8] = (1.0 + 0.01 * np.arange(64, dtype=np.float32)).reshape(8, 8)
    img, b_off = _image(ku.pack_gathered(A), ku.pack_tile(Bm))
    st, d = ku.run_umma(img, [ku.spmm_tile_mma(True, 64, 0, b_off)])
    assert st == 0
    expect = oracle.tile_accumulate(A, Bm, 64, 16, 8, 1)
    bad, _, _ = oracle.compare(ku.m64_rows(d), expect, 0.01)
    assert bad == 0


@pytest.mark.parametrize("tf32", [False, True])
def test_tiles_accumulate_in_tmem(tf32):
    # test/03.warp_specialized/main.cu: T tiles into one accumulator, inputs rand()/RAND_MAX after srand(42)
    dt, cw, T = (np.float32, 8, 6) if tf32 else (np.float16, 16, 6)
    stream = oracle.rand_fill(42, 128 * cw * T + 16 * cw * T)
    A = stream[:128 * cw * T].reshape(128, cw * T).astype(dt)
    Bm = stream[128 * cw * T:].reshape(16, cw * T).astype(dt)
    img, mmas = b"", []
    for t in range(T):
        a_off = len(img)
        img += ku.pack_gathered(np.ascontiguousarray(A[:, t * cw:(t + 1) * cw]))
        img += bytes((-len(img)) % 4096)
        b_off = len(img)
        img += ku.pack_tile(np.ascontiguousarray(Bm[:, t * cw:(t + 1) * cw])) + bytes(512)
        mmas.append(ku.spmm_tile_mma(tf32, 128, a_off, b_off, d_col=16, accumulate=int(t > 0)))
    st, d = ku.run_umma(img + bytes(8192), mmas, n_cols=32)
    assert st == 0
    expect = oracle.tile_accumulate(A.astype(np.float32), Bm.astype(np.float32), 128, 16, cw, T)
    bad, max_rel, _ = oracle.compare(d[:, 16:32], expect, 0.01)  # utils.h:61-85
    assert bad == 0 and max_rel < (2e-3 if tf32 else 1e-5)


def test_tma_tile_load_lands_in_operand_layout():
    data = np.arange(64 * 16, dtype=np.uint16).reshape(64, 16)  # four 16x16 fp16 tiles, 32-byte rows
    loads = [[0, 0, 0, 16, 0, 0, 0], [0, 512, 0, 48, 0, 0, 0]]
    st, dump = ku.run_tma(data, 16, 16, 1, loads, 1024, 1024)
    assert st == 0
    expect = ku.pack_tile(data[16:32].view(np.float16)) + ku.pack_tile(data[48:64].view(np.float16))
    assert dump.tobytes() == expect


def test_tma_tile_load_past_the_end_reads_zero():
    data = np.arange(1, 32 * 16 + 1, dtype=np.uint16).reshape(32, 16)
    st, dump = ku.run_tma(data, 16, 16, 1, [[0, 0, 0, 24, 0, 0, 0]], 512, 512)
    assert st == 0
    tile = np.zeros((16, 16), np.uint16)
    tile[:8] = data[24:32]
    assert dump.tobytes() == ku.pack_tile(tile.view(np.float16))


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_tma_gather4_lands_in_operand_layout(dt):
    # 16 (fp16) / 8 (tf32) rows of B picked by index, 128 features: what one producer warp issues per tile
    cw = 16 if dt == np.float16 else 8
    box = 128 // np.dtype(dt).itemsize
    K, N = 96, 128
    B = (np.arange(K * N) % 2039).astype(np.float32).astype(dt).reshape(K, N)
    rows = [5, 95, 3, 40, 41, 0, 63, 9, 77, 1, 2, 96, 50, 96, 96, 96][:cw]  # 96 = first row past the end
    loads = []
    for h in range(N // box):
        for g in range(cw // 4):
            dst = ((h * 2 + g) * 512) if dt == np.float32 else ((h * 2 + g // 2) * 1024 + (g % 2) * 512)
            loads.append([1, dst, h * box] + rows[4 * g:4 * g + 4])
    total = cw * N * np.dtype(dt).itemsize
    as_bits = B.view(np.uint16 if dt == np.float16 else np.uint32)
    st, dump = ku.run_tma(as_bits, box, 1, 3 if dt == np.float16 else 4, loads, total, total)
    assert st == 0
    gathered = np.zeros((cw, N), dt)
    for k, r in enumerate(rows):
        if r < K:
            gathered[k] = B[r]
    assert dump.tobytes() == ku.pack_gathered(np.ascontiguousarray(gathered.T))


@pytest.mark.parametrize("tf32", [False, True])
def test_mma_issue_rate_of_the_spmm_shape(tf32):
    # One MMA per condensed tile and 128-feature chunk: its cost does not depend on the tile's fill
    # and, up to N = 64, not on N either - the 4 KB operand of gathered rows sets it.  The bounds
    # are loose sanity limits (measured: ~59 SM clocks with one issuing thread, ~78 per thread
    # with two, i.e. ~39 per MMA and SM).
    import ctypes as C
    from hopper_spmm_b200 import _capi as capi
    lib = capi.lib()
    out = (C.c_double * 2)()
    seen = {}
    for n, issuers in ((16, 1), (64, 1), (16, 2)):
        assert lib.b200spmm_kat_umma_rate(int(tf32), 128, n, 512, issuers, out, 0) == 0
        seen[(n, issuers)] = (out[0], out[1])
        assert 4.0 < out[0] <= out[1] < 2000.0, seen
    # two issuing threads together get more MMAs through the SM than one
    assert seen[(16, 2)][1] / 2 < seen[(16, 1)][1] * 1.05, seen
    assert lib.b200spmm_kat_umma_rate(0, 128, 24, 16, 1, out, 0) == capi.ERR_INVALID_ARG
    assert lib.b200spmm_kat_umma_rate(0, 128, 16, 16, 3, out, 0) == capi.ERR_INVALID_ARG


def test_a_wait_that_cannot_complete_runs_out_and_the_device_stays_usable():
    # The reference's mbarrier_wait spins for ever (src/ptx/barrier.h:29-41); every wait here is
    # bounded.  The barrier is told to expect 16 bytes more than the one load delivers, so its phase
    # can never complete: the kernel must come back on its own with the time-out status, the load
    # that was issued must have landed all the same, and the next kernel on the device must work.
    from hopper_spmm_b200 import _capi as capi
    lib = capi.lib()
    data = np.arange(64 * 16, dtype=np.uint16).reshape(64, 16)
    loads = [[0, 0, 0, 16, 0, 0, 0]]
    expect = ku.pack_tile(data[16:32].view(np.float16))
    before = lib.b200spmm_kat_wait_limit(5_000_000)  # 5 ms
    try:
        st, dump = ku.run_tma(data, 16, 16, 1, loads, 512 + 16, 512)
        assert st == capi.ERR_DEVICE_TIMEOUT
        assert dump.tobytes() == expect
    finally:
        assert lib.b200spmm_kat_wait_limit(before) == 5_000_000
    st, dump = ku.run_tma(data, 16, 16, 1, loads, 512, 512)
    assert st == 0 and dump.tobytes() == expect
