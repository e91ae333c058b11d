"""The device-side converter against the host converter (and so the reference algorithm), bit for
bit, and a product computed from a matrix that never left the GPU."""
import numpy as np
import pytest

import hopper_spmm_b200 as hs
import parity
from cases import FORMAT_FIELDS, dense_b, random_csr
from hopper_spmm_b200 import _capi as capi
from hopper_spmm_b200 import synth

pytestmark = pytest.mark.gpu


def device_convert(rows, cols, rp, ci, v, rw=16, cw=0):
    import torch
    d = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).view(dt).copy()).cuda()
    vals = torch.from_numpy(np.ascontiguousarray(v)).cuda()
    return hs.DeviceBtcf(rows, cols, d(rp, np.int32), d(ci, np.int32), vals, row_window=rw, col_window=cw)


def assert_same(dev, host):
    got = dev.to_host()
    assert (dev.eff_row_windows, dev.total_tiles) == (host.eff_row_windows, host.total_tiles)
    for k in FORMAT_FIELDS:
        assert np.array_equal(got[k].view(np.uint8), np.ascontiguousarray(getattr(host, k)).view(np.uint8)), k


@pytest.mark.parametrize("dt,cw", [(np.float16, 16), (np.float32, 8), (np.float32, 4)])
@pytest.mark.parametrize("rw", [8, 16])
def test_matches_host_converter(dt, cw, rw):
    shapes = [(1, 1, 1.0), (16, 16, 0.5), (17, 33, 0.2), (203, 517, 0.03), (500, 70000, 0.0005), (96, 7, 0.6)]
    for seed, (rows, cols, dens) in enumerate(shapes):
        rows, cols, rp, ci, v = random_csr(rows, cols, dens, seed, dt, empty_rows=[(16, 48)] if rows > 64 else (),
                                           dense_rows=[3] if cols < 1000 and rows > 3 else ())
        host = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v), row_window=rw, col_window=cw)
        dev = device_convert(rows, cols, rp, ci, v, rw, cw)
        assert_same(dev, host)
        dev.close()


@pytest.mark.parametrize("name,k", [("uniform_4096_fp16", 0), ("blocks_16384_tf32", 1), ("rmat24_sharded_fp16", 6)])
def test_benchmark_matrices(name, k):
    csr, _ = synth.make_config(name, 0, "cpu", k)
    rp, ci, v = csr.numpy()
    host = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(csr.rows, csr.cols, rp, ci, v))
    dev = device_convert(csr.rows, csr.cols, rp, ci, v)
    assert_same(dev, host)


def test_empty_matrix():
    rp = np.zeros(41, np.uint32)
    dev = device_convert(40, 10, rp, np.zeros(0, np.uint32), np.zeros(0, np.float16))
    assert (dev.eff_row_windows, dev.total_tiles, dev.total_row_windows) == (0, 0, 3)


def test_unsorted_or_repeated_columns_are_refused():
    rp = np.array([0, 3], np.uint32)
    for ci in ([5, 2, 9], [2, 5, 5], [2, 5, 99]):
        with pytest.raises(capi.SpmmError) as e:
            device_convert(1, 16, rp, np.array(ci, np.uint32), np.ones(3, np.float16))
        assert e.value.status == capi.ERR_BAD_CSR


def test_product_from_a_matrix_that_stayed_on_the_gpu():
    import torch
    csr, B = synth.make_config("rmat24_sharded_fp16", 0, "cuda", 8)  # generated on the device
    dev = hs.DeviceBtcf(csr.rows, csr.cols, csr.row_ptr.to(torch.int32), csr.col_idx, csr.values)
    plan = hs.SpmmPlan(dev)
    C_dev = plan.spmm(B)
    rp, ci, v = csr.numpy()
    parity.check(C_dev.cpu().numpy(), csr.rows, rp, ci, v, B.cpu().numpy())
    plan.close()
