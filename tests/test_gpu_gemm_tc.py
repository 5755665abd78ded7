"""GPU parity of the many-row path (in-kernel decode feeding tcgen05.mma) against the CPU oracle
and against the library's own reconstruct -> dense route, through the C ABI."""
import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu
MAX_REL_ERR, MIN_COSINE = 1e-2, 0.9999


def _run(ext, ic, oc, K, rows, seed, dtype=torch.float16):
    tr, suh, svh, x = R.make_layer(seed, ic, oc, K, rows, act_dtype=dtype)
    y = torch.full((rows, oc), float("nan"), dtype=torch.half, device="cuda")
    ext.gemm_tc(x.cuda(), tr.cuda(), y, suh.cuda(), svh.cuda())
    torch.cuda.synchronize()
    assert ext.gemm_tc_status() == 0
    return tr, suh, svh, x, y


@pytest.mark.parametrize("K", [2, 3, 4, 5, 6])
@pytest.mark.parametrize("rows,ic,oc", [(17, 128, 128), (64, 256, 256), (144, 384, 128), (300, 256, 384), (512, 128, 256), (777, 192 * 2, 128)])
def test_gemm_tc_vs_oracle(ext, coracle, K, rows, ic, oc):
    tr, suh, svh, x, y = _run(ext, ic, oc, K, rows, 17 * K + rows)
    w = coracle.reconstruct(tr.numpy())
    ref = coracle.layer(x.numpy(), w, suh.numpy(), svh.numpy())
    got = y.float().cpu().numpy().astype(np.float64)
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    cos = float((got * ref).sum() / np.linalg.norm(got) / np.linalg.norm(ref))
    assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, (rel, cos)


@pytest.mark.parametrize("K", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("rows,ic,oc", [(1, 128, 256), (17, 256, 256), (32, 512, 512), (100, 384, 256), (128, 1024, 768)])
def test_gemm_tmem_operand_path_vs_oracle(ext, coracle, K, rows, ic, oc):
    """Up to 128 rows and a multiple of 256 output channels: the kernel that stores the decoded
    codewords into tensor memory and reads them as the A operand of tcgen05.mma."""
    tr, suh, svh, x, y = _run(ext, ic, oc, K, rows, 31 * K + rows)
    w = coracle.reconstruct(tr.numpy())
    ref = coracle.layer(x.numpy(), w, suh.numpy(), svh.numpy())
    got = y.float().cpu().numpy().astype(np.float64)
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    cos = float((got * ref).sum() / np.linalg.norm(got) / np.linalg.norm(ref))
    assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, (rel, cos)


@pytest.mark.parametrize("rows,ic,oc,K,dtype", [
    (32, 5120, 1024, 3, torch.float16), (64, 17408, 512, 4, torch.bfloat16), (128, 2048, 5120, 5, torch.float16),
    (512, 5120, 1024, 3, torch.bfloat16), (700, 2048, 5120, 4, torch.float16), (2048, 1024, 2048, 4, torch.bfloat16),
])
def test_gemm_tc_vs_reconstruct_route(ext, rows, ic, oc, K, dtype):
    """Larger shapes against reconstruct + dense matmul on the GPU (the reference's own route)."""
    tr, suh, svh, x, y = _run(ext, ic, oc, K, rows, 5 + rows, dtype)
    xg = x.cuda().half()
    xh = torch.empty_like(xg)
    ext.had_r_128(xg, xh, suh.cuda(), None, 1.0)
    w = torch.empty((ic, oc), dtype=torch.half, device="cuda")
    ext.reconstruct(w, tr.cuda(), K, False, False)
    y2 = (xh.float() @ w.float()).half()
    ext.had_r_128(y2, y2, None, svh.cuda(), 1.0)
    rel = float((y.float() - y2.float()).abs().max() / y2.float().abs().max())
    assert rel < 5e-3, rel
    # run-to-run identical bytes
    y3 = torch.empty_like(y)
    ext.gemm_tc(x.cuda(), tr.cuda(), y3, suh.cuda(), svh.cuda())
    assert torch.equal(y, y3)
