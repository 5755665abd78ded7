"""The CPU oracle against the fixtures produced by the reference's own Python
(tests/golden/make_golden.py) and against itself (numpy vs PyTorch vs C forms)."""
import os

import numpy as np
import pytest
import torch

import exl3_ref as R

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))


def test_hadamard_matrix_matches_reference():
    h = R.had128_matrix()
    assert np.array_equal(np.sign(h).astype(np.int8), GOLD["had_sign"])
    # the reference builds the matrix in fp32 before casting, so its scale carries fp32 rounding
    assert abs(abs(h[0, 0]) - GOLD["had_scale"][0]) < 1e-8
    assert np.allclose(h @ h.T, np.eye(128), atol=1e-12) and np.array_equal(h, h.T)


def test_t128_matches_reference():
    assert np.allclose(R.t128_np(GOLD["t128_in"]), GOLD["t128_out"], atol=1e-6)


def test_deploy_weight_matches_reference(coracle):
    w = coracle.reconstruct(GOLD["dw_trellis"])
    dw = R.deploy_weight_np(w, GOLD["dw_suh"], GOLD["dw_svh"])
    ref = GOLD["dw_out"].astype(np.float64)           # reference: fp32 algebra, rounded to fp16
    ulp = np.maximum(np.abs(ref), 2.0 ** -14) * 2.0 ** -10
    assert np.all(np.abs(dw - ref) <= ulp + 1e-5)


def test_exl3_k_matches_reference():
    for wd, v, is_int in zip(GOLD["k_widths"], GOLD["k_values"], GOLD["k_is_int"]):
        k = R.exl3_K(torch.empty((1, 1, int(wd))))
        assert float(k) == v and isinstance(k, int) == bool(is_int)


@pytest.mark.parametrize("tag", ["small", "large"])
def test_layer_matches_reference_shard_gemm(coracle, tag):
    """y of the reference's orcasaq2::shard_gemm (both dispatch branches) vs the oracle layer."""
    w = coracle.reconstruct(GOLD[f"sg_{tag}_trellis"])
    y = coracle.layer(GOLD[f"sg_{tag}_x"], w, GOLD[f"sg_{tag}_suh"], GOLD[f"sg_{tag}_svh"])
    ref = GOLD[f"sg_{tag}_y"].astype(np.float64)
    assert np.abs(y - ref).max() / np.abs(ref).max() < 2e-3
    calls = [c.split(",")[0].strip("('") for c in GOLD[f"sg_{tag}_calls"]]
    expect = ["exl3_gemm"] if tag == "small" else ["had_r_128", "reconstruct", "hgemm_recon", "had_r_128"]
    assert calls == expect


@pytest.mark.parametrize("name", ["f16", "bf16"])
def test_int8_paths_match_reference(coracle, name):
    q, ids, s = GOLD[f"i8_{name}_q"], GOLD[f"i8_{name}_ids"], GOLD[f"i8_{name}_s"].view(np.uint16)
    emb = coracle.int8_embed(q, s, ids, name == "bf16").reshape(*ids.shape, -1)
    assert np.array_equal(emb, GOLD[f"i8_{name}_emb"].view(np.uint16))
    assert np.array_equal(emb, GOLD[f"i8_{name}_tab"].view(np.uint16))
    logits = coracle.int8_head(q, s, GOLD[f"i8_{name}_x"].view(np.uint16), name == "bf16")
    # reference run with fp32 activations: its weight stays q*s in fp32 (no rounding to dt)
    ref = GOLD[f"i8_{name}_logits32"]
    assert np.abs(logits - ref).max() / np.abs(ref).max() < (1e-3 if name == "f16" else 8e-3)
    # reference run in dt end to end: weight rounded to dt, result rounded to dt
    bits = torch.from_numpy(GOLD[f"i8_{name}_logits"].copy())
    ref_dt = bits.view(torch.float16 if name == "f16" else torch.bfloat16).float().numpy()
    assert np.abs(logits - ref_dt).max() / np.abs(ref_dt).max() < (2e-3 if name == "f16" else 1.5e-2)


def test_codebook_known_answers(coracle):
    # spot values of the 3INST map, worked by hand from its definition
    def by_hand(s):
        z = (s * 89226354 + 64248484) & 0xFFFFFFFF
        z = (z & 0x8FFF8FFF) ^ 0x3B603B60
        lo = np.array([z & 0xFFFF], np.uint16).view(np.float16)[0]
        hi = np.array([z >> 16], np.uint16).view(np.float16)[0]
        return np.float16(np.float32(lo) + np.float32(hi))
    for s in (0, 1, 2, 255, 256, 4660, 32768, 65535):
        assert coracle.decode_state(s) == by_hand(s) == R.decode_state_np(np.array([s]))[0]
    v = R.decode_state_np(np.arange(65536)).astype(np.float64)
    assert abs(v.mean()) < 1e-3 and abs(v.std() - 1.2437) < 1e-3 and len(np.unique(v)) == 10598
    assert np.isfinite(v).all() and np.abs(v).max() < 4.0


def test_three_forms_agree(coracle):
    for K in (1, 2, 3, 4, 5, 6, 7, 8):
        tr, suh, svh, x = R.make_layer(K, 128, 256, K, 2)
        a = R.reconstruct_np(tr.numpy()).view(np.uint16)
        b = coracle.reconstruct(tr.numpy()).view(np.uint16)
        c = R.torch_reconstruct(tr).numpy().view(np.uint16)
        assert np.array_equal(a, b) and np.array_equal(a, c)
        y1 = R.layer_np(x.numpy(), a.view(np.float16), suh.numpy(), svh.numpy())
        y2 = coracle.layer(x.numpy(), a.view(np.float16), suh.numpy(), svh.numpy())
        assert np.allclose(y1, y2, rtol=1e-5, atol=1e-4)
        y3 = R.torch_layer(x, tr, suh, svh).float().numpy()
        assert np.abs(y1 - y3).max() / np.abs(y1).max() < 2e-3


def test_tile_format_properties(coracle):
    r, c = R.tile_perm()
    assert sorted(zip(r.tolist(), c.tolist())) == [(a, b) for a in range(16) for b in range(16)]
    cr, cc = coracle.tile_perm()
    assert np.array_equal(r, cr) and np.array_equal(c, cc)
    rng = np.random.default_rng(3)
    for K in (2, 3, 5, 8):
        tile = rng.integers(0, 65536, 16 * K, dtype=np.uint16)
        st = R.tile_states_np(tile, K)
        assert np.array_equal(st, coracle.tile_states(tile, K))
        # bitshift trellis: the next state keeps the upper 16-K bits of the previous one...
        for t in range(256):
            nxt = st[(t + 1) % 256]
            assert (int(st[t]) >> K) == (int(nxt) & ((1 << (16 - K)) - 1))
        # ...and is tail-biting: rotating the bit string by K bits rotates the state sequence
        bits = np.unpackbits(tile.view(np.uint8), bitorder="little")
        rot = np.packbits(np.roll(bits, -K), bitorder="little").view(np.uint16)
        assert np.array_equal(R.tile_states_np(rot, K), np.roll(st, -1))


def test_deploy_identity(coracle):
    """x @ W_deploy^T equals the staged pipeline (the algebra of reconstruct_weight)."""
    tr, suh, svh, x = R.make_layer(8, 256, 128, 4, 3)
    w = coracle.reconstruct(tr.numpy())
    dw = R.deploy_weight_np(w, suh.numpy(), svh.numpy())
    y = coracle.layer(x.numpy(), w, suh.numpy(), svh.numpy())
    assert np.allclose(x.numpy().astype(np.float64) @ dw.T, y, atol=1e-3)


def test_sharding_algebra(coracle):
    """Any 128-aligned sub-block is itself a valid layer: column slices concatenate, row slices
    sum (what tensor parallelism relies on)."""
    ic, oc, K = 512, 384, 3
    tr, suh, svh, x = R.make_layer(9, ic, oc, K, 2)
    trn = tr.numpy()
    full = coracle.layer(x.numpy(), coracle.reconstruct(trn), suh.numpy(), svh.numpy())
    cols = [coracle.layer(x.numpy(), coracle.reconstruct(np.ascontiguousarray(trn[:, o // 16:(o + 128) // 16])),
                          suh.numpy(), svh.numpy()[o:o + 128]) for o in range(0, oc, 128)]
    assert np.allclose(np.concatenate(cols, 1), full, atol=1e-3)
    parts = [coracle.layer(np.ascontiguousarray(x.numpy()[:, i:i + 256]),
                           coracle.reconstruct(np.ascontiguousarray(trn[i // 16:(i + 256) // 16])),
                           suh.numpy()[i:i + 256], svh.numpy()) for i in range(0, ic, 256)]
    assert np.allclose(sum(parts), full, atol=1e-3)


def test_edge_inputs(coracle):
    with pytest.raises(RuntimeError):
        coracle.reconstruct(np.zeros((1, 1, 16 * 9), np.int16))          # K out of range
    z = coracle.reconstruct(np.zeros((1, 1, 32), np.int16))
    assert np.all(z == coracle.decode_state(0))
    assert coracle.had_r_128(np.zeros((0, 128), np.float16)).shape == (0, 128)
    with pytest.raises(RuntimeError):
        coracle.int8_embed(np.zeros((4, 16), np.int8), np.zeros(4, np.uint16), np.array([4]), False)
