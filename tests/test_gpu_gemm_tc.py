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
@pytest.mark.parametrize("rows,ic,oc", [(1, 128, 256), (17, 256, 256), (32, 512, 512), (100, 384, 256), (128, 1024, 768),
                                        (64, 256, 384), (100, 512, 128)])
def test_gemm_tmem_operand_path_vs_oracle(ext, coracle, K, rows, ic, oc):
    """Up to 128 rows (widths that are even and odd multiples of 128): the kernel that stores the decoded
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
    # from 1024 rows CTA pairs (tcgen05.mma.cta_group::2) when the number of 128-channel output blocks is even:
    # full tiles, a last tile of one ragged half (the second CTA's token rows all out of range), a last tile with a
    # ragged second half, split input dimension; and an odd number of output blocks, which stays on single CTAs
    (1024, 512, 256, 3, torch.float16), (1100, 256, 512, 5, torch.float16), (1500, 384, 256, 2, torch.bfloat16),
    (1024, 4096, 256, 4, torch.float16), (1300, 256, 384, 6, torch.float16), (4096, 512, 1024, 3, torch.float16),
    (1200, 2048, 512, 5, torch.bfloat16),
    # more tiles than the 74 CTA pairs of a B200 hold at once: the tiles beyond the last full round are cut into
    # quarter- (80 and 90 tiles) or half-width (110 tiles) work items; 2100 rows leave a ragged last token tile
    (2048, 256, 2560, 3, torch.float16), (2100, 256, 2560, 4, torch.bfloat16), (2816, 384, 2560, 2, torch.float16),      # many input channels per row: the output is rotated in place afterwards, not folded
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


def _dense_ref(ext, x, tr, suh, svh, K):
    """reconstruct + dense matmul on the GPU (the reference's own route) for fp16 activations x."""
    xh = torch.empty_like(x)
    ext.had_r_128(x, xh, suh, None, 1.0)
    w = torch.empty((x.shape[1], svh.numel()), dtype=torch.half, device="cuda")
    ext.reconstruct(w, tr, K, False, False)
    y = (xh.float() @ w.float()).half()
    ext.had_r_128(y, y, None, svh, 1.0)
    return y


@pytest.mark.parametrize("rows,ic,oc,K,layout", [
    (1100, 512, 256, 3, "pitched"),        # rotation folded into the rebuilt weight by the tcgen05 kernel
    (1100, 384, 256, 4, "pitched"),        # input dimension not a multiple of 256: folded on the legacy tensor path
    (1100, 512, 512, 5, "offset"),         # contiguous rows: folding is cheaper than a pass over the output
    (1024, 4096, 256, 2, "offset"),        # many input channels per row: plain weight, output rotated in place afterwards
])
def test_many_rows_output_not_16_byte_aligned(ext, rows, ic, oc, K, layout):
    """The pair kernel rotates the output in its epilogue only when the output rows are 16-byte aligned; an output
    that is only 8-byte aligned takes the older routes (rotation folded into the weight, or a pass over the result)."""
    tr, suh, svh, x = R.make_layer(900 + rows + ic, ic, oc, K, rows)
    xg, trg, sug, svg = x.half().cuda(), tr.cuda(), suh.cuda(), svh.cuda()
    ref = _dense_ref(ext, xg, trg, sug, svg, K).float()
    if layout == "offset":                 # activations that are only 8-byte aligned too: the pre-pass with 8 bytes per lane
        xflat = torch.empty(rows * ic + 4, dtype=torch.half, device="cuda")
        xflat[4:].view(rows, ic).copy_(xg)
        xg = xflat[4:].view(rows, ic)
        assert xg.data_ptr() % 16 == 8
    if layout == "pitched":
        wide = torch.full((rows, oc + 12), 7.0, dtype=torch.half, device="cuda")
        out = wide[:, 4:4 + oc]
    else:
        flat = torch.full((rows * oc + 8,), 7.0, dtype=torch.half, device="cuda")
        out = flat[4:4 + rows * oc].view(rows, oc)
    assert out.data_ptr() % 16 == 8
    ext.gemm_tc(xg, trg, out, sug, svg)
    torch.cuda.synchronize()
    assert ext.gemm_tc_status() == 0
    assert (out.float() - ref).abs().max() / ref.abs().max() < 5e-3
    if layout == "pitched":
        assert bool((wide[:, :4] == 7.0).all()) and bool((wide[:, 4 + oc:] == 7.0).all())
    else:
        assert bool((flat[:4] == 7.0).all()) and bool((flat[4 + rows * oc:] == 7.0).all())


@pytest.mark.parametrize("rows,ic,oc,K", [(24, 1024, 512, 4), (128, 512, 256, 3), (300, 512, 384, 5), (600, 256, 128, 4)])
def test_gemm_tc_fused_rmsnorm_residual_and_pitch(ext, rows, ic, oc, K):
    """RMSNorm in the activation pre-pass, residual add and a wider output matrix in the post-pass equal
    the separate operations -- on the tensor-memory kernel (<= 128 rows), on the split
    shared-memory kernel, and through the binding's own completion where the kernel runs unsplit."""
    tr, suh, svh, x = R.make_layer(700 + rows, ic, oc, K, rows)
    g = torch.Generator().manual_seed(5)
    gamma = (1.0 + 0.1 * torch.randn(ic, generator=g)).half().cuda()
    wide = torch.randn((rows, oc + 256), generator=g).half().cuda()          # residual lives in the wide matrix
    res = wide[:, 128:128 + oc]
    xg, trg, sug, svg = (x * 3.0).half().cuda(), tr.cuda(), suh.cuda(), svh.cuda()
    xf = xg.float()
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()).half()
    ref = _dense_ref(ext, xn, trg, sug, svg, K).float() + res.float()
    out = wide.clone()
    ext.gemm_tc(xg, trg, out[:, 128:128 + oc], sug, svg, in_mode=ext.IN_RMSNORM, norm_weight=gamma, eps=1e-5,
                residual=out[:, 128:128 + oc])
    torch.cuda.synchronize()
    assert ext.gemm_tc_status() == 0
    assert (out[:, 128:128 + oc].float() - ref).abs().max() / ref.abs().max() < 5e-3
    # the columns beside the block are untouched
    assert torch.equal(out[:, :128], wide[:, :128]) and torch.equal(out[:, 128 + oc:], wide[:, 128 + oc:])


@pytest.mark.parametrize("rows,ic,oc,K", [(40, 768, 256, 3), (200, 256, 128, 6)])
def test_gemm_tc_fused_silu_mul(ext, rows, ic, oc, K):
    tr, suh, svh, _ = R.make_layer(800 + rows, ic, oc, K, 1)
    gu = torch.randn((rows, 2 * ic), generator=torch.Generator().manual_seed(rows)).half().cuda()
    trg, sug, svg = tr.cuda(), suh.cuda(), svh.cuda()
    y = torch.empty((rows, oc), dtype=torch.half, device="cuda")
    ext.gemm_tc(gu, trg, y, sug, svg, in_mode=ext.IN_SILU_MUL)
    act = (torch.nn.functional.silu(gu[:, :ic].float()) * gu[:, ic:].float()).half()
    ref = _dense_ref(ext, act, trg, sug, svg, K).float()
    assert ext.gemm_tc_status() == 0
    assert (y.float() - ref).abs().max() / ref.abs().max() < 5e-3


@pytest.mark.parametrize("rows", [17, 64, 128])
def test_gemm_tc_grouped_fused_layer(ext, coracle, rows):
    """Three shards with different bitrates in one grouped launch (the mid-batch form of a fused
    qkv_proj), plain and with RMSNorm + residual, against the oracle and the single-shard calls."""
    ic, spec = 512, [(768, 4), (128, 5), (384, 6)]          # even and odd multiples of 128
    shards, refs, col = [], [], 0
    x = None
    for i, (oc, K) in enumerate(spec):
        tr, suh, svh, xi = R.make_layer(40 * rows + i, ic, oc, K, rows)
        x = xi if x is None else x
        shards.append(dict(trellis=tr.cuda(), suh=suh.cuda(), svh=svh.cuda(), mcg=False, mul1=False, out_col=col))
        refs.append((tr, suh, svh))
        col += oc
    xg = x.half().cuda()
    y = torch.full((rows, col), float("nan"), dtype=torch.half, device="cuda")
    assert ext.gemm_tc_grouped(xg, shards, y)
    torch.cuda.synchronize()
    assert ext.gemm_tc_status() == 0
    xf = x.half().numpy()
    ref = np.concatenate([coracle.layer(xf, coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy()) for tr, suh, svh in refs], 1)
    got = y.float().cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= MAX_REL_ERR
    # identical to the single-shard kernel, shard by shard
    y1 = torch.empty_like(y)
    for s, (oc, K) in zip(shards, spec):
        ext.gemm_tc(xg, s["trellis"], y1[:, s["out_col"]:s["out_col"] + oc], s["suh"], s["svh"])
    assert torch.equal(y, y1)
    # fused RMSNorm and in-place residual
    g = torch.Generator().manual_seed(9)
    gamma = (1.0 + 0.1 * torch.randn(ic, generator=g)).half().cuda()
    acc = torch.randn((rows, col), generator=g).half().cuda()
    acc1 = acc.clone()
    assert ext.gemm_tc_grouped(xg, shards, acc, in_mode=ext.IN_RMSNORM, norm_weight=gamma, eps=1e-5, residual=acc)
    for s, (oc, K) in zip(shards, spec):
        blk = acc1[:, s["out_col"]:s["out_col"] + oc]
        ext.gemm_tc(xg, s["trellis"], blk, s["suh"], s["svh"], in_mode=ext.IN_RMSNORM, norm_weight=gamma, eps=1e-5, residual=blk)
    assert torch.equal(acc, acc1)


def test_gemm_tc_grouped_declines_other_shapes(ext):
    tr, suh, svh, x = R.make_layer(8, 256, 256, 4, 200)
    sh = [dict(trellis=tr.cuda(), suh=suh.cuda(), svh=svh.cuda(), mcg=False, mul1=False)]
    y = torch.zeros((200, 256), dtype=torch.half, device="cuda")
    assert ext.gemm_tc_grouped(x.half().cuda(), sh, y) is False          # more than 128 rows
    assert float(y.abs().max()) == 0.0
