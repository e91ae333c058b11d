"""The sharded operator of the C ABI (b200spmm_sharded_*): several GPUs driven by one process.  On a
one-GPU box the one-shard form still runs (no collective is needed); the multi-GPU cases need two devices."""
import numpy as np
import pytest

import hopper_spmm_b200 as hs
import parity
from cases import dense_b, random_csr

pytestmark = pytest.mark.gpu


def _n_devices():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_one_shard_equals_the_plain_operator(dt):
    rows, cols, rp, ci, v = random_csr(700, 300, 0.05, 3, dt, empty_rows=[(100, 140)])
    B = dense_b(cols, 128, 4, dt)
    sh = hs.ShardedSpmm(hs.CSR_MTX(rows, cols, rp, ci, v), [0])
    try:
        assert list(sh.row_begin) == [0, rows]
        got = sh.spmm_host(B)
    finally:
        sh.close()
    parity.check(got, rows, rp, ci, v, B)
    plan = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v)))
    try:
        assert np.array_equal(plan.spmm_host(B).view(np.uint32), got.view(np.uint32))
    finally:
        plan.close()


@pytest.mark.parametrize("n_dev", [2, 4, 8])
def test_shards_on_several_devices_give_the_one_device_result(n_dev):
    if _n_devices() < n_dev:
        pytest.skip(f"needs {n_dev} devices")
    import torch
    from hopper_spmm_b200 import synth
    csr, B = synth.make_config("rmat24_sharded_fp16", 0, "cuda", 7)  # 2^17 nodes: hub rows on shard 0
    rp, ci, v = csr.numpy()
    Bn = B.cpu().numpy()
    one = hs.SpmmPlan(hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(csr.rows, csr.cols, rp, ci, v)))
    try:
        want = one.spmm_host(Bn)
    finally:
        one.close()
    parity.check(want, csr.rows, rp, ci, v, Bn)
    sh = hs.ShardedSpmm(hs.CSR_MTX(csr.rows, csr.cols, rp, ci, v), list(range(n_dev)))
    try:
        cuts = sh.row_begin
        assert cuts[0] == 0 and cuts[-1] == csr.rows and all(c % 16 == 0 for c in cuts[:-1]) and np.all(np.diff(cuts) > 0)
        got = sh.spmm_host(Bn)  # 1/N of B per device + all-gather, products, rows of C back
        # a row's additions do not depend on how the rows were cut, except in windows that a GPU shares
        # between CTAs: those are summed from pieces, and which windows are shared depends on the shard.
        # So: the parity rule, and agreement with the one-GPU result to fp32 reassociation noise
        parity.check(got, csr.rows, rp, ci, v, Bn)
        assert np.allclose(got, want, rtol=1e-4, atol=1e-6)
        assert (got.view(np.uint32) == want.view(np.uint32)).mean() > 0.5
        # device-resident products written in place + the all-gather of C
        Bs = [B.to(f"cuda:{d}") for d in range(n_dev)]
        Cs = [torch.full((csr.rows, Bn.shape[1]), float("nan"), device=f"cuda:{d}") for d in range(n_dev)]
        for d in range(n_dev):  # the shards run on streams of their own: what fills B and C must be done first
            torch.cuda.synchronize(d)
        sh.spmm_allgather(Bs, Cs)
        for d in range(n_dev):
            assert np.array_equal(Cs[d].cpu().numpy().view(np.uint32), got.view(np.uint32)), d
    finally:
        sh.close()


@pytest.mark.parametrize("n_dev", [4, 8])
def test_allgather_of_skewed_ranges_runs_in_two_steps(n_dev):
    # Rows whose weight decays fast: the shards are cut for equal work, so the last one holds most of the rows and
    # the all-gather of C must take its two-step form (misplaced bytes to the holder of their even share, then the
    # in-place all-gather of the even shares).  Every device must end up with the whole product.
    if _n_devices() < n_dev:
        pytest.skip(f"needs {n_dev} devices")
    import ctypes as C
    import torch
    from hopper_spmm_b200 import _capi as capi
    rows, cols, n = 40000, 2000, 256
    rng = np.random.default_rng(0)
    deg = np.maximum(1, (1500 * np.exp(-np.arange(rows) / 1200.0)).astype(np.int64))
    rp = np.concatenate([[0], np.cumsum(deg)]).astype(np.uint32)
    ci = np.concatenate([np.sort(rng.choice(cols, d, replace=False)) for d in deg]).astype(np.uint32)
    v = rng.uniform(-1, 1, ci.size).astype(np.float32).astype(np.float16)
    B = dense_b(cols, n, 1)
    sh = hs.ShardedSpmm(hs.CSR_MTX(rows, cols, rp, ci, v), list(range(n_dev)), row_charge=0)
    try:
        cut = np.asarray(sh.row_begin, np.uint64) * np.uint64(n * 4)
        part = C.c_uint64()
        pieces = np.zeros((n_dev, n_dev - 1, 10), np.uint64)
        assert capi.lib().b200spmm_allgather_plan(cut.ctypes.data, n_dev, C.byref(part), pieces.ctypes.data) == capi.OK
        assert part.value > 0, f"expected the two-step exchange for row ranges {list(sh.row_begin)}"
        Bs = [torch.from_numpy(B).to(f"cuda:{d}") for d in range(n_dev)]
        Cs = [torch.full((rows, n), float("nan"), device=f"cuda:{d}") for d in range(n_dev)]
        for d in range(n_dev):
            torch.cuda.synchronize(d)
        sh.spmm_allgather(Bs, Cs)
        first = Cs[0].cpu().numpy()
        parity.check(first, rows, rp, ci, v, B)
        for d in range(1, n_dev):
            assert np.array_equal(Cs[d].cpu().numpy().view(np.uint32), first.view(np.uint32)), d
    finally:
        sh.close()
