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


# --------------------------------------------------------------------------- fp8 (e4m3) caches
def _quant(t, scale):
    """What an fp8 cache holds for the values `t`: value / scale rounded to e4m3."""
    return (t.float() / scale).to(torch.float8_e4m3fn)


def _deq(t8, scale):
    return (t8.float() * scale).half()          # exact: an e4m3 value times a power of two fits fp16


@pytest.mark.parametrize("B,qh,kvh,seq_len,cap", [
    (1, 24, 4, 4097, 4112),      # the 27B decoder at batch 1: many splits
    (2, 24, 4, 1, 64),           # a single token
    (3, 6, 1, 15, 16),           # less than one tile
    (2, 12, 2, 17, 48),          # one tile and one token
    (4, 3, 1, 1000, 1024),       # three query heads per KV head, ragged tail
    (32, 24, 4, 513, 528),       # batch 32: few splits
    (2, 8, 1, 333, 400),         # eight query heads on one KV head
])
def test_decode_attn_fp8_cache(ext, B, qh, kvh, seq_len, cap):
    """fp8 cache against fp32 attention over the dequantised bytes (same tolerance as the fp16 kernel: the only
    roundings are the fp16 probabilities and the fp16 output), and against the fp16 kernel on the dequantised
    cache (same arithmetic, other summation order)."""
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + seq_len + 1)
    ks, vs = 0.5, 2.0
    q = torch.randn(B, qh, 256, device="cuda", generator=g).half()
    k8 = _quant(torch.randn(B, kvh, cap, 256, device="cuda", generator=g), ks)
    v8 = _quant(torch.randn(B, kvh, cap, 256, device="cuda", generator=g), vs)
    k8.view(torch.uint8)[:, :, seq_len:] = 0x7F                       # NaN bytes beyond seq_len must not matter
    v8.view(torch.uint8)[:, :, seq_len:] = 0x7F
    out = ext.decode_attn(q, k8, v8, seq_len, k_scale=ks, v_scale=vs)
    kd, vd = _deq(k8, ks), _deq(v8, vs)
    _check(out, _ref(q, kd, vd, seq_len))
    _check(out, ext.decode_attn(q, kd, vd, seq_len).float())
    assert torch.equal(out, ext.decode_attn(q, k8, v8, seq_len, k_scale=ks, v_scale=vs))   # fixed summation order


def test_decode_attn_fp8_every_dimension_lands_in_its_place(ext):
    """One token, V = the dimension index pattern: the output must reproduce V exactly (softmax weight 1), which
    pins the permuted accumulator -> dimension mapping; and a one-hot query picks single K dimensions."""
    B, qh, kvh = 1, 8, 2
    v = (torch.arange(256, device="cuda").float() % 15 - 7).view(1, 1, 1, 256).expand(B, kvh, 16, 256).contiguous()
    v[:, 1] *= -1
    k = torch.zeros(B, kvh, 16, 256, device="cuda")
    q = torch.zeros(B, qh, 256, device="cuda").half()
    out = ext.decode_attn(q, _quant(k, 1.0), _quant(v, 1.0), 1)
    assert torch.equal(out[:, :4].float(), v[:, 0, 0].expand(B, 4, 256))
    assert torch.equal(out[:, 4:].float(), v[:, 1, 0].expand(B, 4, 256))
    # two tokens; K of token 1 is large in dimension d only; a query that is one-hot in d must pick token 1
    for d in (0, 1, 2, 3, 5, 16, 17, 31, 100, 255):
        k = torch.zeros(B, kvh, 16, 256, device="cuda")
        k[:, :, 1, d] = 8.0
        vv = torch.zeros(B, kvh, 16, 256, device="cuda")
        vv[:, :, 1] = 1.0
        q = torch.zeros(B, qh, 256, device="cuda")
        q[:, :, d] = 16.0 * 16.0                                      # score 8 * 256 / 16 = 128: weight ~ 1
        o = ext.decode_attn(q.half(), _quant(k, 1.0), _quant(vv, 1.0), 2)
        assert torch.allclose(o.float(), torch.ones_like(o.float()), atol=1e-3), d
        q = torch.zeros(B, qh, 256, device="cuda")
        q[:, :, (d + 1) % 256] = 256.0                                # any other dimension: both tokens weigh 1/2
        o = ext.decode_attn(q.half(), _quant(k, 1.0), _quant(vv, 1.0), 2)
        assert torch.allclose(o.float(), torch.full_like(o.float(), 0.5), atol=1e-3), d


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("B,qh,kvh,page,cap", [(1, 24, 4, 16, 2048), (3, 6, 1, 64, 512), (32, 12, 2, 32, 256)])
def test_decode_attn_paged_fp8(ext, layout, B, qh, kvh, page, cap):
    g = torch.Generator(device="cuda").manual_seed(B * 7 + page + 1)
    ks, vs = 0.25, 1.0
    q = torch.randn(B, qh, 256, device="cuda", generator=g).half()
    kc = _deq(_quant(torch.randn(B, kvh, cap, 256, device="cuda", generator=g), ks), ks)
    vc = _deq(_quant(torch.randn(B, kvh, cap, 256, device="cuda", generator=g), vs), vs)
    kp, vp, table = _paginate(kc, vc, page, layout, g)               # fp16 pools with NaN in the unused pages
    kp8, vp8 = _quant(kp, ks), _quant(vp, vs)
    full = ext.decode_attn_paged(q, kp8, vp8, table, None, cap, layout=layout, k_scale=ks, v_scale=vs)
    assert torch.equal(full, ext.decode_attn(q, _quant(kc, ks), _quant(vc, vs), cap, k_scale=ks, v_scale=vs))
    lens = torch.randint(1, cap + 1, (B,), device="cuda", generator=g).to(torch.int32)
    lens[0] = 1
    table2 = table.clone()
    for b in range(B):
        table2[b, (int(lens[b]) + page - 1) // page:] = kp.shape[0] - 1
    out = ext.decode_attn_paged(q, kp8, vp8, table2, lens, cap, layout=layout, k_scale=ks, v_scale=vs)
    for b in range(B):
        n = int(lens[b])
        _check(out[b:b + 1], _ref(q[b:b + 1], kc[b:b + 1], vc[b:b + 1], n))


@pytest.mark.parametrize("B,qh,kvh,per_seq", [(1, 24, 4, False), (5, 3, 1, True)])
def test_rope_append_fp8(ext, B, qh, kvh, per_seq):
    """fp8 append = the fp16 append's values divided by the scale and rounded to e4m3; the query is the same."""
    g = torch.Generator(device="cuda").manual_seed(21 + B)
    cap, pos, ks, vs = 48, 17, 0.5, 2.0
    qkv = torch.randn(B, (qh + 2 * kvh) * 256, device="cuda", generator=g).half()
    ang = torch.rand((B, 128) if per_seq else (128,), device="cuda", generator=g) * 6.28
    cos, sin = torch.cos(ang).half(), torch.sin(ang).half()
    k16 = torch.zeros(B, kvh, cap, 256, device="cuda", dtype=torch.half)
    v16 = torch.zeros_like(k16)
    q16 = qkv.clone()
    ext.rope_append(q16, cos, sin, k16, v16, pos, qh)
    k8 = torch.zeros(B, kvh, cap, 256, device="cuda", dtype=torch.uint8).view(torch.float8_e4m3fn)
    v8 = torch.zeros(B, kvh, cap, 256, device="cuda", dtype=torch.uint8).view(torch.float8_e4m3fn)
    q8 = qkv.clone()
    ext.rope_append(q8, cos, sin, k8, v8, pos, qh, k_scale=ks, v_scale=vs)
    assert torch.equal(q8, q16)
    assert torch.equal(k8.view(torch.uint8), _quant(k16, ks).view(torch.uint8))
    assert torch.equal(v8.view(torch.uint8), _quant(v16, vs).view(torch.uint8))
    # a value beyond the e4m3 range saturates to +-448 instead of turning into NaN
    big = torch.full_like(qkv, 1000.0)
    ext.rope_append(big, torch.ones_like(cos), torch.zeros_like(sin), k8, v8, pos + 1, qh, k_scale=1.0, v_scale=1.0)
    assert torch.all(v8[:, :, pos + 1].float() == 448.0) and torch.all(k8[:, :, pos + 1].float() == 448.0)
