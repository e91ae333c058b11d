"""The allocation-free entry point against the plan-based one.

Some users of this library cannot call cudaMalloc when they need a product - their process has
already given all free device memory to its own pool, or it runs under a latency budget that
rules out an allocating call.  b200spmm_spmm_noalloc serves them: it takes the converted matrix
as arrays the caller already holds on the device and keeps its own working memory (schedule
table, status word) in a fixed array inside the library.  Because that array is shared by all
calls and keeps the last call's contents, the check is made on two calls in a row, on matrices
of different size.  Each result must pass the parity rule of the other device tests, and equal
the plan-based entry point bit for bit whenever that one computed every window in one piece (it
may share a heavy window between CTAs, which changes the order of the fp32 additions; the
allocation-free path never does, having no memory for the pieces).

Collected last on purpose: a run that stops at the first failure has then seen every other test.
"""
import ctypes as C

import numpy as np
import pytest

import hopper_spmm_b200 as hs
import parity
from cases import dense_b, random_csr
from hopper_spmm_b200 import _capi as capi

pytestmark = pytest.mark.gpu


def _device_format(btcf, torch):
    """The four format arrays in device memory the caller owns (torch tensors here)."""
    def up(a, dt):
        return torch.from_numpy(np.ascontiguousarray(a).view(dt).copy()).cuda()
    info = capi.BtcfInfo()
    capi.check(capi.lib().b200spmm_btcf_info(btcf._h, C.byref(info)), "b200spmm_btcf_info")
    data_dt = np.int16 if btcf.dtype == np.float16 else np.int32
    return info, up(btcf.rowOffset, np.int32), up(btcf.tcA2B, np.int32), up(btcf.data, data_dt), up(btcf.rowIdx, np.int32)


def _noalloc(info, d_ro, d_a2b, d_data, d_ridx, dB, dC, n_ctas, torch):
    st = capi.lib().b200spmm_spmm_noalloc(C.byref(info), d_ro.data_ptr(), d_a2b.data_ptr(), d_data.data_ptr(),
                                          d_ridx.data_ptr(), dB.data_ptr(), dB.stride(0), dB.shape[1], dC.data_ptr(),
                                          dC.stride(0), capi.C_F32, 0, n_ctas, torch.cuda.current_stream().cuda_stream)
    capi.check(st, "b200spmm_spmm_noalloc")
    # the kernel's own verdict (a bounded wait that gave up would show here), read back without allocating
    capi.check(capi.lib().b200spmm_spmm_noalloc_status(0, torch.cuda.current_stream().cuda_stream), "b200spmm_spmm_noalloc_status")


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_two_calls_in_a_row_match_the_plan_based_entry_point(dt):
    import torch
    cases = [random_csr(900, 700, 0.03, 21, dt, empty_rows=[(0, 32), (400, 480)], dense_rows=[50]),
             random_csr(203, 517, 0.05, 22, dt)]  # the second call sees the first call's table
    for k, (rows, cols, rp, ci, v) in enumerate(cases):
        n = 128 if k == 0 else 320
        btcf = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
        dB = torch.from_numpy(dense_b(cols, n, 30 + k, dt)).cuda()
        plan = hs.SpmmPlan(btcf)
        want = plan.spmm(dB)
        whole_windows = plan.launch_info().kernel_launches == 1
        plan.close()
        info, d_ro, d_a2b, d_data, d_ridx = _device_format(btcf, torch)
        for n_ctas in (0, 37):
            got = torch.full((rows, n), float("nan"), device="cuda")  # every row must be written
            _noalloc(info, d_ro, d_a2b, d_data, d_ridx, dB, got, n_ctas, torch)
            parity.check(got.cpu().numpy(), rows, rp, ci, v, dB.cpu().numpy())
            if whole_windows:
                assert torch.equal(got, want), f"case {k}, n_ctas {n_ctas}"
            else:
                assert torch.allclose(got, want, rtol=1e-4, atol=1e-4), f"case {k}, n_ctas {n_ctas}"


def test_sizes_beyond_the_built_in_table_are_refused():
    import torch
    rows, cols, rp, ci, v = random_csr(64, 64, 0.2, 3)
    btcf = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(rows, cols, rp, ci, v))
    info, d_ro, d_a2b, d_data, d_ridx = _device_format(btcf, torch)
    dB = torch.from_numpy(dense_b(cols, 64, 1)).cuda()
    dC = torch.zeros((rows, 64), device="cuda")
    st = capi.lib().b200spmm_spmm_noalloc(C.byref(info), d_ro.data_ptr(), d_a2b.data_ptr(), d_data.data_ptr(),
                                          d_ridx.data_ptr(), dB.data_ptr(), 64, 64, dC.data_ptr(), 64, capi.C_F32, 0,
                                          1025, None)
    assert st == capi.ERR_UNSUPPORTED
    assert b"1024" in capi.lib().b200spmm_last_cuda_error()
