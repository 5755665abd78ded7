"""The plugin's custom ops on the GPU: every branch of the row-count dispatch (fused GEMV, tcgen05
GEMM, reconstruct + dense GEMM) gives the oracle's layer, for single shards and fused layers."""
import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(ext):
    from orcasaq2 import ops
    return ops


def _check(y, ref, tol=1e-2):
    got = y.float().cpu().numpy().astype(np.float64)
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    cos = float((got * ref).sum() / np.linalg.norm(got) / np.linalg.norm(ref))
    assert rel <= tol and cos >= 0.9999, (rel, cos)


@pytest.mark.parametrize("rows", [1, 16, 17, 150, 1030])
def test_shard_gemm_dispatch(ops, coracle, rows):
    ic, oc, K = 256, 384, 4
    tr, suh, svh, x = R.make_layer(rows, ic, oc, K, rows)
    y = torch.ops.orcasaq2.shard_gemm(x.cuda(), tr.cuda(), suh.cuda(), svh.cuda(), oc, float(K), False, False)
    assert y.shape == (rows, oc) and y.dtype == torch.half
    ref = coracle.layer(x.numpy(), coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy())
    _check(y, ref)


@pytest.mark.parametrize("rows", [3, 40, 1100])
def test_layer_gemm_fused(ops, coracle, rows):
    ic, spec = 256, [(256, 4), (128, 5), (128, 6)]
    x = torch.randn((rows, ic), generator=torch.Generator().manual_seed(rows)).half()
    trs, suhs, svhs, refs = [], [], [], []
    for i, (oc, K) in enumerate(spec):
        tr, suh, svh, _ = R.make_layer(200 + i, ic, oc, K, 1)
        trs.append(tr.cuda()); suhs.append(suh.cuda()); svhs.append(svh.cuda())
        refs.append(coracle.layer(x.numpy(), coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy()))
    y = torch.ops.orcasaq2.layer_gemm(x.cuda(), trs, suhs, svhs, [oc for oc, _ in spec],
                                      [float(K) for _, K in spec], [False] * 3, [False] * 3)
    assert y.shape == (rows, 512)
    _check(y, np.concatenate(refs, 1))


@pytest.mark.parametrize("rows", [1030, 4100])
def test_many_rows_take_the_pair_kernel(ops, coracle, rows):
    """From 1024 rows with an even number of 128-channel output blocks: decode once + dense tcgen05 GEMM on CTA pairs,
    as a single shard and as a fused layer (every shard writes its column block of the result: pitched output);
    the GEMM's epilogue rotates and scales the output rows in registers."""
    ic, oc, K = 256, 512, 3
    tr, suh, svh, x = R.make_layer(rows, ic, oc, K, rows)
    y = torch.ops.orcasaq2.shard_gemm(x.cuda(), tr.cuda(), suh.cuda(), svh.cuda(), oc, float(K), False, False)
    _check(y, coracle.layer(x.numpy(), coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy()))
    spec = [(256, 4), (512, 5), (256, 6)]
    trs, suhs, svhs, refs = [], [], [], []
    for i, (o, k) in enumerate(spec):
        t, su, sv, _ = R.make_layer(300 + i, ic, o, k, 1)
        trs.append(t.cuda()); suhs.append(su.cuda()); svhs.append(sv.cuda())
        refs.append(coracle.layer(x.numpy(), coracle.reconstruct(t.numpy()), su.numpy(), sv.numpy()))
    yl = torch.ops.orcasaq2.layer_gemm(x.cuda(), trs, suhs, svhs, [o for o, _ in spec], [float(k) for _, k in spec],
                                       [False] * 3, [False] * 3)
    _check(yl, np.concatenate(refs, 1))
    from orcasaq2 import _ext
    assert _ext.gemm_tc_status() == 0


def test_empty_batch(ops):
    tr, suh, svh, _ = R.make_layer(1, 128, 128, 4, 1)
    x = torch.empty((0, 128), dtype=torch.half, device="cuda")
    y = torch.ops.orcasaq2.shard_gemm(x, tr.cuda(), suh.cuda(), svh.cuda(), 128, 4.0, False, False)
    assert y.shape == (0, 128)


def test_reconstruct_weight_matches_reference_fixture(ext):
    """orcasaq2.reconstruct_weight on the GPU against the deploy weight the reference's own
    function produced (fixture), same trellis / suh / svh."""
    import os
    import orcasaq2
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))
    tr = torch.from_numpy(gold["dw_trellis"]).cuda()
    suh = torch.from_numpy(gold["dw_suh"]).cuda()
    svh = torch.from_numpy(gold["dw_svh"]).cuda()
    w = orcasaq2.reconstruct_weight(tr, suh, svh, None, None)
    ref = gold["dw_out"].astype(np.float32)
    got = w.float().cpu().numpy()
    assert w.shape == ref.shape
    ulp = np.maximum(np.abs(ref), 2.0 ** -14) * 2.0 ** -10
    assert np.all(np.abs(got - ref) <= 2 * ulp + 1e-4)
