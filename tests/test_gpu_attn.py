"""Decode attention kernel (exl3_decode_attn, through the C ABI) against an fp32 PyTorch restatement of
softmax(q K^T / sqrt(d)) V on the same fp16 inputs.  Tolerance: fp16 output rounding plus fp16
probabilities, max abs error <= 2e-3 * max|ref| + 1e-3 and cosine >= 0.9999."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, kc, vc, seq_len):
    B, qh, hd = q.shape
    kvh = kc.shape[1]
    G = qh // kvh
    k = kc[:, :, :seq_len].float().repeat_interleave(G, dim=1)      # query head h -> KV head h // G
    v = vc[:, :, :seq_len].float().repeat_interleave(G, dim=1)
    s = torch.einsum("bhd,bhtd->bht", q.float(), k) * hd ** -0.5
    return torch.einsum("bht,bhtd->bhd", torch.softmax(s, dim=-1), v)


def _check(out, ref):
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-3 * ref.abs().max().item() + 1e-3, err
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), ref.flatten(), dim=0).item()
    assert cos >= 0.9999, cos


@pytest.mark.parametrize("B,qh,kvh,seq_len,cap", [
    (1, 24, 4, 4097, 4100),      # the 27B decoder at batch 1: many splits
    (2, 24, 4, 1, 64),           # a single token
    (3, 6, 1, 15, 16),           # less than one tile
    (2, 12, 2, 17, 40),          # one tile and one token
    (4, 3, 1, 1000, 1024),       # three query heads per KV head (tensor-parallel slice), ragged tail
    (32, 24, 4, 513, 520),       # batch 32: few splits
    (2, 8, 1, 333, 400),         # eight query heads on one KV head
    (2, 4, 4, 200, 200),         # no grouping
])
def test_decode_attn_matches_fp32(ext, B, qh, kvh, seq_len, cap):
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + seq_len)
    q = torch.randn(B, qh, 256, device="cuda", generator=g).half()
    kc = torch.randn(B, kvh, cap, 256, device="cuda", generator=g).half()
    vc = torch.randn(B, kvh, cap, 256, device="cuda", generator=g).half()
    # rows beyond seq_len must not matter, whatever they hold
    kc[:, :, seq_len:] = float("nan")
    vc[:, :, seq_len:] = float("nan")
    out = ext.decode_attn(q, kc, vc, seq_len)
    _check(out, _ref(q, kc, vc, seq_len))
    again = ext.decode_attn(q, kc, vc, seq_len)
    assert torch.equal(out, again)                                   # fixed summation order


def test_decode_attn_peaked_scores_and_views(ext):
    """Large score spread (the running maximum moves often) and q / out given as views of wider rows."""
    g = torch.Generator(device="cuda").manual_seed(7)
    B, qh, kvh, L = 2, 24, 4, 700
    wide = torch.randn(B, (qh + 2 * kvh) * 256, device="cuda", generator=g).half()
    q = wide[:, :qh * 256].view(B, qh, 256) * 4.0
    q = torch.as_strided(wide, (B, qh, 256), (wide.stride(0), 256, 1))
    kc = (torch.randn(B, kvh, L, 256, device="cuda", generator=g) * 2.0).half()
    vc = torch.randn(B, kvh, L, 256, device="cuda", generator=g).half()
    buf = torch.zeros(B, qh * 256 + 64, device="cuda", dtype=torch.half)
    out = torch.as_strided(buf, (B, qh, 256), (buf.stride(0), 256, 1))
    ext.decode_attn(q, kc, vc, L, out=out)
    _check(out, _ref(q, kc, vc, L))
    assert torch.count_nonzero(buf[:, qh * 256:]) == 0


def test_decode_attn_rejects_bad_arguments(ext):
    q = torch.zeros(1, 24, 128, device="cuda", dtype=torch.half)
    kc = torch.zeros(1, 4, 16, 128, device="cuda", dtype=torch.half)
    with pytest.raises(RuntimeError):
        ext.decode_attn(q, kc, kc, 16)                               # head size 128 is not built
    q = torch.zeros(1, 36, 256, device="cuda", dtype=torch.half)
    kc = torch.zeros(1, 4, 16, 256, device="cuda", dtype=torch.half)
    with pytest.raises(RuntimeError):
        ext.decode_attn(q, kc, kc, 16)                               # nine query heads per KV head
    with pytest.raises(RuntimeError):
        ext.decode_attn(q[:, :24], kc, kc, 17)                       # longer than the cache
    with pytest.raises(RuntimeError):
        ext.decode_attn(q[:, :24].cpu(), kc, kc, 16)                 # no CPU path


@pytest.mark.parametrize("B,qh,kvh,per_seq", [(1, 24, 4, False), (5, 3, 1, True), (32, 12, 2, False)])
def test_rope_append_matches_fp32(ext, B, qh, kvh, per_seq):
    """Rotary + cache append against the rotate-half formula in fp32 (within 2e-3 of the largest value:
    one fp16 rounding), untouched cache rows stay as they were."""
    g = torch.Generator(device="cuda").manual_seed(11 + B)
    cap, pos = 40, 17
    qkv = torch.randn(B, (qh + 2 * kvh) * 256 + 128, device="cuda", generator=g).half()   # wider rows than needed
    ang = torch.rand((B, 128) if per_seq else (128,), device="cuda", generator=g) * 6.28
    cos, sin = torch.cos(ang).half(), torch.sin(ang).half()
    kc = torch.randn(B, kvh, cap, 256, device="cuda", generator=g).half()
    vc = torch.randn(B, kvh, cap, 256, device="cuda", generator=g).half()
    kc0, vc0, src = kc.clone(), vc.clone(), qkv.clone()
    ext.rope_append(qkv, cos, sin, kc, vc, pos, qh)

    t = src[:, :(qh + kvh) * 256].float().view(B, qh + kvh, 256)
    c = cos.float().view(-1, 1, 128) if per_seq else cos.float()
    s = sin.float().view(-1, 1, 128) if per_seq else sin.float()
    lo, hi = t[..., :128], t[..., 128:]
    want = torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)
    got_q = qkv[:, :qh * 256].view(B, qh, 256)
    assert (got_q.float() - want[:, :qh]).abs().max().item() <= 2e-3 * want.abs().max().item()
    assert (kc[:, :, pos].float() - want[:, qh:]).abs().max().item() <= 2e-3 * want.abs().max().item()
    assert torch.equal(vc[:, :, pos], src[:, (qh + kvh) * 256:(qh + 2 * kvh) * 256].view(B, kvh, 256))
    assert torch.equal(qkv[:, qh * 256:], src[:, qh * 256:])          # k, v and the padding of qkv are not modified
    mask = torch.ones(cap, dtype=torch.bool, device="cuda")
    mask[pos] = False
    assert torch.equal(kc[:, :, mask], kc0[:, :, mask]) and torch.equal(vc[:, :, mask], vc0[:, :, mask])
    with pytest.raises(RuntimeError):
        ext.rope_append(qkv, cos, sin, kc, vc, cap, qh)               # position outside the cache


def _paginate(kc, vc, page, layout, gen):
    """Scatter contiguous caches [B, kvh, cap, 256] into page pools in a shuffled page order."""
    B, kvh, cap, hd = kc.shape
    per_seq = cap // page
    n = B * per_seq
    perm = torch.randperm(n + 3, device="cuda", generator=gen)[:n].to(torch.int32)     # three pages stay unused
    table = perm.view(B, per_seq).contiguous()
    shape = (n + 3, kvh, page, hd) if layout == "HND" else (n + 3, page, kvh, hd)
    kp = torch.full(shape, float("nan"), device="cuda", dtype=torch.half)
    vp = torch.full(shape, float("nan"), device="cuda", dtype=torch.half)
    for b in range(B):
        for i in range(per_seq):
            ks, vs = kc[b, :, i * page:(i + 1) * page], vc[b, :, i * page:(i + 1) * page]   # [kvh, page, hd]
            pg = int(table[b, i])
            kp[pg] = ks if layout == "HND" else ks.transpose(0, 1)
            vp[pg] = vs if layout == "HND" else vs.transpose(0, 1)
    return kp, vp, table


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("B,qh,kvh,page,cap", [(1, 24, 4, 16, 2048), (3, 6, 1, 64, 512), (32, 12, 2, 32, 256)])
def test_decode_attn_paged(ext, layout, B, qh, kvh, page, cap):
    """Paged form: same bytes as the contiguous kernel when all sequences are full, fp32 parity with
    ragged per-sequence lengths (including a sequence of one token), unused pages and table entries ignored."""
    g = torch.Generator(device="cuda").manual_seed(B * 7 + page)
    q = torch.randn(B, qh, 256, device="cuda", generator=g).half()
    kc = torch.randn(B, kvh, cap, 256, device="cuda", generator=g).half()
    vc = torch.randn(B, kvh, cap, 256, device="cuda", generator=g).half()
    kp, vp, table = _paginate(kc, vc, page, layout, g)
    full = ext.decode_attn_paged(q, kp, vp, table, None, cap, layout=layout)
    assert torch.equal(full, ext.decode_attn(q, kc, vc, cap))
    lens = torch.randint(1, cap + 1, (B,), device="cuda", generator=g).to(torch.int32)
    lens[0] = 1
    lens[-1] = cap - 5 if B > 1 else 1
    table2 = table.clone()
    for b in range(B):                                   # entries past a sequence's length must not be read:
        table2[b, (int(lens[b]) + page - 1) // page:] = kp.shape[0] - 1      # they point at a page of NaNs
    out = ext.decode_attn_paged(q, kp, vp, table2, lens, cap, layout=layout)
    for b in range(B):
        n = int(lens[b])
        _check(out[b:b + 1], _ref(q[b:b + 1], kc[b:b + 1], vc[b:b + 1], n))


def test_decode_attn_paged_rejects_bad_arguments(ext):
    q = torch.zeros(2, 8, 256, device="cuda", dtype=torch.half)
    kp = torch.zeros(8, 2, 24, 256, device="cuda", dtype=torch.half)      # 24 tokens per page: not a multiple of 16
    table = torch.zeros(2, 4, device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError):
        ext.decode_attn_paged(q, kp, kp, table, None, 48)
    kp = torch.zeros(8, 2, 32, 256, device="cuda", dtype=torch.half)
    with pytest.raises(RuntimeError):
        ext.decode_attn_paged(q, kp, kp, table, None, 32 * 5)             # the table is too short for 160 tokens
    with pytest.raises(RuntimeError):
        ext.decode_attn_paged(q, kp, kp, table.long(), None, 64)
    with pytest.raises(RuntimeError):
        ext.decode_attn_paged(q, kp, kp, table, torch.zeros(3, device="cuda", dtype=torch.int32), 64)
