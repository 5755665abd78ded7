"""The decoder harness behind the tokens-per-second half of the headline metric (bench_model.py), checked end to
end: a two-layer decoder at small width is built by the SAME code that builds the 27B model, one decode step is
run at batch 1 and 9 with both attention choices, and the logits are compared with an oracle step made of the CPU
oracle's trellis decode, float64 layer algebra and float64 attention.  What this covers that the per-kernel tests
do not: the rotary / cache-append offsets, which tensor is the residual of which layer, the fused RMSNorm and
SiLU-mul inputs, the grouped outputs' column order and the head on the final norm."""
import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu

DIMS = dict(hidden=256, ffn=384, qh=3, kvh=1, hd=256, vocab=300)
LAYERS, CTX = 2, 40
# two layers of fp16 roundings (and fp16 probabilities in the attention kernel) on top of the layer tolerance
MAX_REL_ERR = 2e-2      # max |logits - ref| / max |ref|
MIN_COSINE = 0.999


def _f16(a):
    return np.asarray(a, np.float64).astype(np.float32).astype(np.float16).astype(np.float64)


def _rms(h, eps=1e-6):
    return _f16(h * (1.0 / np.sqrt((h * h).mean(-1, keepdims=True) + eps)))


def _layer(co, x, shard):
    w = co.reconstruct(shard["trellis"].cpu().numpy())
    return R.layer_np(x.astype(np.float16), w, shard["suh"].cpu().numpy(), shard["svh"].cpu().numpy())


def _e4m3(a):
    return torch.from_numpy(np.asarray(a, np.float32)).to(torch.float8_e4m3fn).float().numpy().astype(np.float64)


def _oracle_step(co, model_cpu, table, scales, ids, ctx, kv="fp16"):
    hd, qh, kvh = DIMS["hd"], DIMS["qh"], DIMS["kvh"]
    h = _f16(table[ids].astype(np.float64) * scales[ids][:, None])
    half = hd // 2
    ang = ctx / (10000.0 ** (np.arange(half, dtype=np.float32) / half))
    cos = np.cos(ang).astype(np.float16).astype(np.float64)
    sin = np.sin(ang).astype(np.float16).astype(np.float64)

    def rope(t):                                                    # [B, heads, hd], rotate-half form
        a, b = t[..., :half], t[..., half:]
        return _f16(np.concatenate([a * cos - b * sin, b * cos + a * sin], -1))

    for (qkv, o, gu, down, kc, vc) in model_cpu:
        x = _rms(h)
        y = _f16(np.concatenate([_layer(co, x, s) for s in qkv], 1))
        B = y.shape[0]
        q = rope(y[:, :qh * hd].reshape(B, qh, hd))
        k = rope(y[:, qh * hd:(qh + kvh) * hd].reshape(B, kvh, hd))
        v = y[:, (qh + kvh) * hd:].reshape(B, kvh, hd)
        if kv == "fp8":                                             # what an e4m3 cache (scale 1) keeps of the new token
            k, v = _e4m3(k), _e4m3(v)
        K = np.concatenate([kc[:, :, :ctx], k[:, :, None]], 2)      # [B, kvh, ctx + 1, hd]
        V = np.concatenate([vc[:, :, :ctx], v[:, :, None]], 2)
        att = np.zeros((B, qh, hd))
        for hq in range(qh):
            hk = hq // (qh // kvh)
            s = np.einsum("bd,btd->bt", q[:, hq], K[:, hk]) * hd ** -0.5
            p = np.exp(s - s.max(-1, keepdims=True))
            p /= p.sum(-1, keepdims=True)
            att[:, hq] = np.einsum("bt,btd->bd", p, V[:, hk])
        att = _f16(att).reshape(B, qh * hd)
        h = _f16(_layer(co, att, o[0]) + h)
        g = _f16(np.concatenate([_layer(co, _rms(h), s) for s in gu], 1))
        ffn = DIMS["ffn"]
        act = _f16(g[:, :ffn] / (1.0 + np.exp(-g[:, :ffn])) * g[:, ffn:])
        h = _f16(_layer(co, act, down[0]) + h)
    x = _rms(h)
    return (x @ table.astype(np.float64).T) * scales[None, :]


@pytest.mark.parametrize("attn,kv", [("own", "fp16"), ("sdpa", "fp16"), ("own", "fp8")])
@pytest.mark.parametrize("batch", [1, 9])
def test_decoder_step_matches_oracle(ext, coracle, batch, attn, kv):
    import bench_model as BM
    dev = torch.device("cuda", 0)
    model, table, scales, _, _, qh, kvh = BM.build(0, 1, batch, CTX, dev, LAYERS, DIMS, kv=kv)
    assert model[0][4].dtype == (torch.float8_e4m3fn if kv == "fp8" else torch.float16)
    assert (qh, kvh) == (DIMS["qh"], DIMS["kvh"]) and len(model) == LAYERS
    ids = torch.randint(0, DIMS["vocab"], (batch,), generator=torch.Generator().manual_seed(11)).to(dev)
    # the oracle's copy of the model, taken before the step appends to the caches
    model_cpu = [([dict(s) for s in qkv.shards], [dict(s) for s in o.shards], [dict(s) for s in gu.shards],
                  [dict(s) for s in down.shards], kc.float().cpu().numpy().astype(np.float64),
                  vc.float().cpu().numpy().astype(np.float64)) for qkv, o, gu, down, kc, vc in model]
    step = BM.make_step(model, table, scales, ids, batch, CTX, qh, kvh, 1, attn, DIMS)
    tok, logits = step()
    torch.cuda.synchronize()
    assert ext.workspace_status(dev) == 0
    ref = _oracle_step(coracle, model_cpu, table.cpu().numpy(), scales.float().cpu().numpy().astype(np.float64),
                       ids.cpu().numpy(), CTX, kv)
    got = logits.float().cpu().numpy().astype(np.float64)
    assert got.shape == ref.shape == (batch, DIMS["vocab"])
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    cos = float((got * ref).sum() / (np.linalg.norm(got) * np.linalg.norm(ref)))
    assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, (rel, cos)
    # the step appended the rotated key and the value of the new token at position CTX of every layer's cache
    for (_, _, _, _, kc, vc), (_, _, _, _, kc0, vc0) in zip(model, model_cpu):
        assert np.array_equal(kc[:, :, :CTX].float().cpu().numpy(), kc0[:, :, :CTX].astype(np.float32))
        assert not np.array_equal(kc[:, :, CTX].float().cpu().numpy(), kc0[:, :, CTX].astype(np.float32))
    # a second step from the same state gives the same tokens (the caches' new slot is rewritten with the same values)
    tok2, _ = step()
    assert torch.equal(tok, tok2)
