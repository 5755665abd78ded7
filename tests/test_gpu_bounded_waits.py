"""The give-up path of the kernels' bounded waits, exercised without any fault: one warp waits, through the
kernels' own wait helpers and with a short limit, on a barrier nothing will ever complete.  The wait runs out, the
sticky status word is set, the launch returns, and the device goes on serving the regular entry points."""
import ctypes
import time

import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu


def _gemv_ok(ext):
    tr, suh, svh, x = R.make_layer(5, 256, 256, 4, 2)
    y = torch.empty((2, 256), dtype=torch.half, device="cuda")
    ext.gemv_grouped(x.cuda(), [dict(trellis=tr.cuda(), suh=suh.cuda(), svh=svh.cuda(), mcg=False, mul1=False)], y)
    torch.cuda.synchronize()
    return bool(torch.isfinite(y.float()).all())


def test_gemv_wait_runs_out_and_reports(ext):
    L = ext.lib()
    L.exl3_gemv_selftest_wait.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    word = torch.zeros(64, dtype=torch.int32, device="cuda")            # a status word of its own
    assert L.exl3_gemv_selftest_wait(word.data_ptr(), 5000, None) == 0
    t0 = time.perf_counter()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0                               # it came back
    assert int(word[0].item()) != 0                                     # and said why
    assert _gemv_ok(ext) and ext.workspace_status(torch.device("cuda", 0)) == 0    # the regular path is untouched
    assert L.exl3_gemv_selftest_wait(None, 10, None) == -6
    assert L.exl3_gemv_selftest_wait(word.data_ptr(), 0, None) == -1


@pytest.mark.parametrize("which", [0, 1])
def test_tcgen05_wait_runs_out_and_reports(ext, which):
    L = ext.lib()
    L.exl3_gemm_tc_selftest_wait.argtypes = [ctypes.c_int, ctypes.c_uint, ctypes.c_void_p]
    torch.cuda.synchronize()
    assert ext.gemm_tc_status() == 0
    try:
        assert L.exl3_gemm_tc_selftest_wait(which, 3000, None) == 0     # three milliseconds
        t0 = time.perf_counter()
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 5.0
        assert ext.gemm_tc_status() != 0
    finally:
        assert L.exl3_gemm_tc_status_reset() == 0
    assert ext.gemm_tc_status() == 0
    # the many-row path still works afterwards and leaves the word clear
    tr, suh, svh, x = R.make_layer(9, 256, 256, 4, 40)
    y = torch.empty((40, 256), dtype=torch.half, device="cuda")
    ext.gemm_tc(x.cuda(), tr.cuda(), y, suh.cuda(), svh.cuda())
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and ext.gemm_tc_status() == 0
    assert L.exl3_gemm_tc_selftest_wait(2, 100, None) == -1
