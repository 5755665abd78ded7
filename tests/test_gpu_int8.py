"""GPU parity of the int8 embedding gather (bit-exact) and the int8 head (tolerance) against
the CPU oracle and the reference-generated fixtures, through the C ABI."""
import os

import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))
DT = {"f16": torch.float16, "bf16": torch.bfloat16}


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("name", ["f16", "bf16"])
def test_embed_matches_reference_fixture(ext, name):
    q = torch.from_numpy(GOLD[f"i8_{name}_q"]).cuda()
    s = torch.from_numpy(GOLD[f"i8_{name}_s"].copy()).view(DT[name]).cuda()
    ids = torch.from_numpy(GOLD[f"i8_{name}_ids"]).cuda()
    out = ext.int8_embed(q, s, ids)
    assert out.shape == (*ids.shape, q.shape[1]) and out.dtype == DT[name]
    assert np.array_equal(_bits(out), GOLD[f"i8_{name}_emb"].view(np.uint16))


@pytest.mark.parametrize("name", ["f16", "bf16"])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_embed_bit_exact_large(ext, coracle, name, idt):
    vocab, hidden = 4099, 5120
    q, s = R.make_int8_table(7, vocab, hidden, DT[name])
    ids = torch.randint(0, vocab, (37,), generator=torch.Generator().manual_seed(2))
    ids[0], ids[1] = 0, vocab - 1
    out = ext.int8_embed(q.cuda(), s.cuda(), ids.to(idt).cuda())
    ref = coracle.int8_embed(q.numpy(), _bits(s), ids.numpy(), name == "bf16")
    assert np.array_equal(_bits(out), ref)


def test_embed_edge_cases(ext):
    q, s = R.make_int8_table(1, 64, 128)
    empty = ext.int8_embed(q.cuda(), s.cuda(), torch.empty((0,), dtype=torch.int64, device="cuda"))
    assert empty.shape == (0, 128)
    bad = ext.int8_embed(q.cuda(), s.cuda(), torch.tensor([3, 64, -1], device="cuda"))
    assert torch.all(bad[1:] == 0) and torch.any(bad[0] != 0)      # out-of-range ids give zero rows
    with pytest.raises(RuntimeError):
        ext.int8_embed(q.cuda(), s.cuda(), torch.tensor([1.0], device="cuda"))


@pytest.mark.parametrize("name", ["f16", "bf16"])
@pytest.mark.parametrize("rows,vocab,hidden", [(1, 1000, 256), (4, 96, 128), (9, 2049, 1024), (16, 512, 5120), (35, 300, 192)])
def test_head_vs_oracle(ext, coracle, name, rows, vocab, hidden):
    q, s = R.make_int8_table(rows + vocab, vocab, hidden, DT[name])
    x = torch.randn((rows, hidden), generator=torch.Generator().manual_seed(rows)).to(DT[name])
    out = ext.int8_head(q.cuda(), s.cuda(), x.cuda())
    assert out.shape == (rows, vocab) and out.dtype == DT[name]
    ref = coracle.int8_head(q.numpy(), _bits(s), _bits(x), name == "bf16")
    got = out.float().cpu().numpy()
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    cos = float((got * ref).sum() / np.linalg.norm(got) / np.linalg.norm(ref))
    assert rel <= (2e-3 if name == "f16" else 1e-2) and cos >= 0.9999, (rel, cos)


@pytest.mark.parametrize("name", ["f16", "bf16"])
@pytest.mark.parametrize("rows,vocab,hidden", [(17, 1000, 256), (32, 515, 512), (33, 4099, 1024), (64, 2048 + 7, 5120), (300, 300, 768)])
def test_head_many_rows_one_pass_over_the_table(ext, coracle, name, rows, vocab, hidden):
    """17..64 rows are served by ONE pass over the int8 table (the staged kernel); more rows in passes of 64."""
    q, s = R.make_int8_table(rows + vocab, vocab, hidden, DT[name])
    x = torch.randn((rows, hidden), generator=torch.Generator().manual_seed(rows)).to(DT[name])
    out = ext.int8_head(q.cuda(), s.cuda(), x.cuda())
    assert out.shape == (rows, vocab) and out.dtype == DT[name]
    ref = coracle.int8_head(q.numpy(), _bits(s), _bits(x), name == "bf16")
    got = out.float().cpu().numpy()
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    cos = float((got * ref).sum() / np.linalg.norm(got) / np.linalg.norm(ref))
    assert rel <= (2e-3 if name == "f16" else 1e-2) and cos >= 0.9999, (rel, cos)
    # the rows do not depend on how many others ride along: the first 5 rows alone (resident kernel) agree closely
    few = ext.int8_head(q.cuda(), s.cuda(), x[:5].cuda()).float().cpu().numpy()
    assert np.abs(few - got[:5]).max() / np.abs(ref).max() <= (2e-3 if name == "f16" else 1e-2)


def test_head_many_rows_bf16_large_activations_and_direct_call_limits(ext, coracle):
    q, s = R.make_int8_table(6, 512, 256, torch.bfloat16)
    x = (torch.randn((40, 256), generator=torch.Generator().manual_seed(4)) * 3.0e5).to(torch.bfloat16)
    out = ext.int8_head(q.cuda(), s.cuda(), x.cuda()).float().cpu().numpy()
    ref = coracle.int8_head(q.numpy(), _bits(s), _bits(x), True)
    assert np.isfinite(out).all() and np.abs(out - ref).max() / np.abs(ref).max() <= 1e-2
    L = ext.lib()
    lg = torch.empty((65, 512), dtype=torch.bfloat16, device="cuda")
    xx = torch.zeros((65, 256), dtype=torch.bfloat16, device="cuda")
    args = lambda r, h: (q.cuda().data_ptr(), s.cuda().data_ptr(), xx.data_ptr(), lg.data_ptr(), r, 512, h, 512, 1, None)  # noqa: E731
    assert L.exl3_int8_head(*args(65, 256)) == -1        # more rows than one call takes
    assert L.exl3_int8_head(*args(20, 192)) == -1        # above 16 rows the hidden size must be a multiple of 256


def test_head_bf16_large_activations(ext, coracle):
    """bf16 rows beyond the fp16 range are rescaled inside the kernel, not clipped."""
    q, s = R.make_int8_table(5, 256, 128, torch.bfloat16)
    x = (torch.randn((2, 128), generator=torch.Generator().manual_seed(4)) * 3.0e5).to(torch.bfloat16)
    out = ext.int8_head(q.cuda(), s.cuda(), x.cuda()).float().cpu().numpy()
    ref = coracle.int8_head(q.numpy(), _bits(s), _bits(x), True)
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() / np.abs(ref).max() <= 1e-2


@pytest.mark.parametrize("name", ["f16", "bf16"])
def test_head_matches_reference_fixture(ext, name):
    q = torch.from_numpy(GOLD[f"i8_{name}_q"]).cuda()
    s = torch.from_numpy(GOLD[f"i8_{name}_s"].copy()).view(DT[name]).cuda()
    x = torch.from_numpy(GOLD[f"i8_{name}_x"].copy()).view(DT[name]).cuda()
    out = ext.int8_head(q, s, x).float().cpu().numpy()
    ref = torch.from_numpy(GOLD[f"i8_{name}_logits"].copy()).view(DT[name]).float().numpy()
    assert np.abs(out - ref).max() / np.abs(ref).max() <= (2e-3 if name == "f16" else 1.5e-2)
