"""Host-side logic of the plugin mirror on CPU: API surface, fixtures from the reference's own
Python, shard capture and slot mapping, tensor-parallel slicing, custom-op fake kernels, and the
loud failure when the CUDA library or a CUDA tensor is missing."""
import os
import types

import numpy as np
import pytest
import torch

import exl3_ref as R

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))


def test_hadamard_and_t128_match_reference():
    import orcasaq2
    assert orcasaq2.BLOCK == 128
    h = orcasaq2._had("cpu", torch.float64).numpy()
    assert np.array_equal(np.sign(h).astype(np.int8), GOLD["had_sign"])
    assert abs(abs(h[0, 0]) - GOLD["had_scale"][0]) < 1e-8
    y = orcasaq2._t128(torch.from_numpy(GOLD["t128_in"])).numpy()
    assert np.allclose(y, GOLD["t128_out"], atol=1e-6)
    assert orcasaq2._had("cpu", torch.float64) is orcasaq2._had("cpu", torch.float64)     # cached


def test_exl3_k_and_dispatch_threshold():
    from orcasaq2 import ops
    for wd, v, is_int in zip(GOLD["k_widths"], GOLD["k_values"], GOLD["k_is_int"]):
        k = ops.exl3_K(torch.empty((1, 1, int(wd))))
        assert float(k) == v and isinstance(k, int) == bool(is_int)
    assert ops.GEMM_MAX_ROWS == int(GOLD["gemm_max_rows"][0]) == 144


def test_custom_op_schemas_and_fake_kernels():
    from orcasaq2 import ops  # noqa: F401
    schema = str(torch.ops.orcasaq2.shard_gemm.default._schema)
    assert "(Tensor x, Tensor trellis, Tensor suh, Tensor svh, SymInt oc, float k, bool mcg, bool mul1) -> Tensor" in schema
    x = torch.empty((5, 256), dtype=torch.half, device="meta")
    tr = torch.empty((16, 8, 64), dtype=torch.int16, device="meta")
    v = torch.empty((256,), dtype=torch.half, device="meta")
    y = torch.ops.orcasaq2.shard_gemm(x, tr, v, v, 128, 4.0, False, False)
    assert y.shape == (5, 128) and y.dtype == torch.half and y.device.type == "meta"
    y = torch.ops.orcasaq2.layer_gemm(x, [tr, tr], [v, v], [v, v], [128, 128], [4.0, 4.0], [False] * 2, [False] * 2)
    assert y.shape == (5, 256) and y.dtype == torch.half


def test_no_cpu_fallback():
    from orcasaq2 import _ext
    x = torch.zeros((1, 128), dtype=torch.half)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _ext.had_r_128(x, x, None, None, 1.0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _ext.reconstruct(torch.zeros((16, 16), dtype=torch.half), torch.zeros((1, 1, 64), dtype=torch.int16), 4, False, False)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _ext.int8_embed(torch.zeros((4, 16), dtype=torch.int8), torch.zeros(4, dtype=torch.half), torch.zeros(1, dtype=torch.long))


def test_missing_library_is_loud(monkeypatch):
    from orcasaq2 import _ext
    monkeypatch.setattr(_ext, "_lib", None)
    monkeypatch.setattr(_ext, "_LIB_PATH", "/nonexistent/libexl3_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _ext.lib()


# ----------------------------------------------------------------------------- vLLM-facing classes
@pytest.fixture(scope="module")
def cfgmod():
    import vllm.model_executor.parameter as vp
    vp.get_tensor_model_parallel_rank = lambda: 0
    vp.get_tensor_model_parallel_world_size = lambda: 1
    from orcasaq2 import config
    return config


def test_shard_param_slots_match_reference(cfgmod):
    p = cfgmod.Exl3ShardParam(suffix="trellis")
    probes = [None, 0, 1, 3, (0, 1, 2), (2, 3), "q", "k", "v"]
    assert [repr(s) for s in probes] == list(GOLD["slot_probes"])
    assert [p.slot(s) for s in probes] == list(GOLD["slot_values"])
    assert repr(cfgmod.SHARD_IDS) == GOLD["shard_ids"][0]
    with pytest.raises(ValueError):
        p.slot("nope")
    t = torch.arange(6)
    p.weight_loader(p, t, "k")
    p.load_qkv_weight(t + 1, shard_id="v")
    p.load_merged_column_weight(t + 2, shard_id=0)
    assert set(p.shards) == {0, 1, 2} and p.shards[1] is t and p.numel() == 0


def test_quant_config(cfgmod):
    raw = {"bits": 4.0, "head_bits": 6, "tensor_storage": {
        "model.layers.0.self_attn.q_proj": {"stored_tensors": {"model.layers.0.self_attn.q_proj.trellis": {}}},
        "model.layers.0.mlp.gate": {"stored_tensors": {"model.layers.0.mlp.gate.weight": {}}}}}
    c = cfgmod.Exl3Config.from_config(raw)
    assert (c.bits, c.codebook, c.head_bits) == (4.0, "mul1", 6.0)
    assert c.quantized_prefixes == {"model.layers.0.self_attn.q_proj"}
    assert c.get_name() == "exl3" and c.get_config_filenames() == ["quantization_config.json"]
    assert torch.half in c.get_supported_act_dtypes() and torch.bfloat16 in c.get_supported_act_dtypes()
    assert cfgmod._expand("m.layers.0.self_attn.qkv_proj", "qkv_proj") == [
        "m.layers.0.self_attn.q_proj", "m.layers.0.self_attn.k_proj", "m.layers.0.self_attn.v_proj"]
    assert cfgmod._expand("m.mlp.down_proj", "down_proj") == ["m.mlp.down_proj"]
    assert c.get_quant_method(torch.nn.Linear(2, 2), "x") is None
    assert "Exl3Config(bits=4.0" in repr(c)


def test_create_weights_registers_placeholders(cfgmod):
    m = cfgmod.Exl3LinearMethod(cfgmod.Exl3Config.from_config({}), "l.qkv_proj")
    layer = torch.nn.Module()
    m.create_weights(layer, 256, [256, 128, 128], 256, 512, torch.half)
    for name in ("trellis", "suh", "svh", "mcg", "mul1", "weight"):
        assert isinstance(getattr(layer, name), cfgmod.Exl3ShardParam)
    assert layer.exl3_out_total == 512


def test_slice_shard_rejects_unaligned(cfgmod):
    tr, suh, svh, _ = R.make_layer(1, 256, 256, 2, 1)
    with pytest.raises(RuntimeError, match="128-aligned"):
        cfgmod.slice_shard(tr, suh, svh, 0, 256, 64, 192)
    t, a, b = cfgmod.slice_shard(tr, suh, svh, 128, 256, 0, 128)
    assert t.shape == (8, 8, 32) and a.numel() == 128 and b.numel() == 128 and t.is_contiguous()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_slicing_rules(cfgmod, coracle, monkeypatch, world):
    """Column-parallel qkv with replicated KV heads and row-parallel down_proj: every rank's
    slice, run through the oracle, reassembles the unsharded layer."""
    ic, rows = 256, 2
    x = torch.randn((rows, ic), generator=torch.Generator().manual_seed(3)).half()
    # q: 8 blocks of 128 ("heads"), k/v: 2 blocks each -> replicated when world > 2
    spec = [(1024, 3), (256, 4), (256, 5)]
    full = [R.make_layer(60 + i, ic, oc, K, 1)[:3] for i, (oc, K) in enumerate(spec)]
    ref = [coracle.layer(x.numpy(), coracle.reconstruct(t.numpy()), a.numpy(), b.numpy()) for t, a, b in full]
    m = cfgmod.Exl3LinearMethod(cfgmod.Exl3Config.from_config({}), "l.qkv_proj")
    kv_part = max(128, 256 // world)
    layer = types.SimpleNamespace(exl3_tp=dict(in_part=ic, in_full=ic, out_parts=[1024 // world, kv_part, kv_part],
                                               out_full=1536))
    got = [[None] * world for _ in spec]
    for rank in range(world):
        monkeypatch.setattr(cfgmod, "_tp_info", lambda r=rank: (r, world))
        for pos, (t, a, b) in enumerate(full):
            ts, as_, bs = m._slice_for_rank(layer, pos, 3, t, a, b)
            assert bs.numel() == layer.exl3_tp["out_parts"][pos]
            got[pos][rank] = coracle.layer(x.numpy(), coracle.reconstruct(ts.numpy()), as_.numpy(), bs.numpy())
    assert np.allclose(np.concatenate(got[0], 1), ref[0], atol=1e-3)
    rep = max(1, world // (256 // kv_part))
    for pos in (1, 2):
        uniq = [got[pos][r] for r in range(0, world, rep)]
        assert np.allclose(np.concatenate(uniq, 1), ref[pos], atol=1e-3)
        for r in range(world):
            assert np.array_equal(got[pos][r], got[pos][(r // rep) * rep])
    # row-parallel: partial sums add up
    ic2, oc2 = 128 * world, 256
    t, a, b = R.make_layer(70, ic2, oc2, 4, 1)[:3]
    x2 = torch.randn((rows, ic2), generator=torch.Generator().manual_seed(5)).half()
    ref2 = coracle.layer(x2.numpy(), coracle.reconstruct(t.numpy()), a.numpy(), b.numpy())
    layer2 = types.SimpleNamespace(exl3_tp=dict(in_part=128, in_full=ic2, out_parts=[oc2], out_full=oc2))
    acc = 0
    for rank in range(world):
        monkeypatch.setattr(cfgmod, "_tp_info", lambda r=rank: (r, world))
        ts, as_, bs = m._slice_for_rank(layer2, 0, 1, t, a, b)
        xs = np.ascontiguousarray(x2.numpy()[:, rank * 128:(rank + 1) * 128])
        acc = acc + coracle.layer(xs, coracle.reconstruct(ts.numpy()), as_.numpy(), bs.numpy())
    assert np.allclose(acc, ref2, atol=1e-3)


def test_custom_ops_trace_with_fake_tensors(cfgmod):
    """Every kernel the model's forward reaches is an opaque custom op with a registered fake (meta) implementation,
    so Dynamo can trace through the plugin under torch.compile without touching ctypes (reference ops.py:3-16,
    ops.py:63-66 for shard_gemm; the int8 gather sits inside the compiled forward too)."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty((5, 256), dtype=torch.half)
        tr = torch.empty((16, 24, 64), dtype=torch.int16)
        suh, svh = torch.empty((256,), dtype=torch.half), torch.empty((384,), dtype=torch.half)
        y = torch.ops.orcasaq2.shard_gemm(x, tr, suh, svh, 384, 4.0, False, False)
        assert y.shape == (5, 384) and y.dtype == torch.half
        yl = torch.ops.orcasaq2.layer_gemm(x, [tr, tr], [suh, suh], [svh, svh], [384, 384], [4.0, 4.0], [False] * 2, [False] * 2)
        assert yl.shape == (5, 768) and yl.dtype == torch.half
        q, s = torch.empty((300, 256), dtype=torch.int8), torch.empty((300,), dtype=torch.bfloat16)
        ids = torch.empty((2, 7), dtype=torch.int64)
        e = torch.ops.orcasaq2.int8_embed(q, s, ids)
        assert e.shape == (2, 7, 256) and e.dtype == torch.bfloat16
        lg = torch.ops.orcasaq2.int8_head(q, s, x)
        assert lg.shape == (5, 300) and lg.dtype == torch.half


def test_int8_embedding_table_api():
    from orcasaq2.patches.int8_embedding import Int8EmbeddingTable, apply
    q, s = R.make_int8_table(2, 8, 16)
    tab = Int8EmbeddingTable(q, s, torch.half)
    assert tab.scales.shape == (8, 1) and tab.weight.shape == (8, 16) and tab.weight.dtype == torch.half
    assert torch.equal(tab.weight, q.half() * s.reshape(-1, 1))
    with pytest.raises(RuntimeError, match="exllamav3"):
        apply()


def test_int8_embedding_apply_hooks_a_stand_in_engine(monkeypatch):
    """`apply()` (reference patches/int8_embedding.py:46-86) against a stand-in for the engine module it patches:
    an Embedding whose store holds `<key>.qweight` / `<key>.scales` gets an Int8EmbeddingTable from eager reads,
    one without them goes to the stock loader, and a second apply() is a no-op."""
    import sys
    import types
    from orcasaq2.patches import int8_embedding as P

    calls = []

    class Store:
        def __init__(self, tensors):
            self.t = tensors

        def has_tensor(self, key):
            return key in self.t

        def get_tensor(self, key, device, **kw):
            calls.append((key, kw))
            return self.t[key]

    class Embedding:
        def __init__(self, key, store):
            self.key, self.out_dtype, self.embedding = key, torch.half, None
            self.config = types.SimpleNamespace(stc=store)

        def load(self, device, **kwargs):
            self.embedding = "stock"
            return "stock"

    eng = types.ModuleType("exllamav3")
    mods = types.ModuleType("exllamav3.modules")
    emb = types.ModuleType("exllamav3.modules.embedding")
    emb.Embedding = Embedding
    eng.modules, mods.embedding = mods, emb
    for name, m in (("exllamav3", eng), ("exllamav3.modules", mods), ("exllamav3.modules.embedding", emb)):
        monkeypatch.setitem(sys.modules, name, m)

    assert P.apply() is True and P.apply() is False
    q, s = R.make_int8_table(3, 8, 16)
    e = Embedding("model.embed_tokens", Store({"model.embed_tokens.qweight": q, "model.embed_tokens.scales": s}))
    assert e.load("cpu") is None
    assert isinstance(e.embedding, P.Int8EmbeddingTable) and e._numel == q.numel() and e.device == "cpu"
    assert torch.equal(e.embedding.qweight, q) and e.embedding.scales.shape == (8, 1)
    assert all(kw.get("no_defer") for _, kw in calls[-2:]) and calls[-1][1].get("allow_bf16")
    plain = Embedding("model.embed_tokens", Store({"model.embed_tokens.weight": q}))
    assert plain.load("cpu") == "stock" and plain.embedding == "stock"


def _loaded_layer(cfgmod, K=4, flag=None, width=None):
    """A one-shard layer with its tensors captured, ready for process_weights_after_loading."""
    m = cfgmod.Exl3LinearMethod(cfgmod.Exl3Config.from_config({}), "l.o_proj")
    layer = torch.nn.Module()
    m.create_weights(layer, 128, [128], 128, 128, torch.half)
    tr, suh, svh, _ = R.make_layer(5, 128, 128, K, 1)
    if width is not None:
        tr = tr[..., :width].contiguous()
    layer.trellis.weight_loader(layer.trellis, tr, None)
    layer.suh.weight_loader(layer.suh, suh, None)
    layer.svh.weight_loader(layer.svh, svh, None)
    if flag:
        getattr(layer, flag).weight_loader(getattr(layer, flag), torch.zeros(1), None)
    return m, layer


@pytest.mark.parametrize("flag,width,what", [("mcg", None, "mcg"), ("mul1", None, "mul1"), (None, 56, "K=3.5")])
def test_undefined_decoders_are_refused_at_load(cfgmod, flag, width, what):
    """The alternative codebooks and the half bitrates are flagged per tensor in the reference
    (orcasaq2/config.py:218, ops.py:28-34) but defined nowhere in its tree: such a shard is refused when the
    layer is loaded, with the reason, not at the first forward."""
    m, layer = _loaded_layer(cfgmod, 4, flag, width)
    with pytest.raises(RuntimeError, match=what.replace(".", r"\.")):
        m.process_weights_after_loading(layer)


def test_pack_layout_mark(cfgmod, caplog):
    """A pack without this build's layout mark loads, with a loud warning; the synthetic checkpoints carry it."""
    import logging
    from orcasaq2 import checkpoint, ops
    records = []
    h = logging.Handler()
    h.emit = lambda r: records.append(r.getMessage())
    cfgmod.logger.addHandler(h)
    try:
        cfgmod.Exl3Config.from_config({"bits": 4.0})
        assert any("exl3_layout" in r and "NOT known to be compatible" in r for r in records)
        records.clear()
        c = cfgmod.Exl3Config.from_config({"bits": 4.0, "exl3_layout": ops.PACK_LAYOUT})
        assert not records and c.layout == ops.PACK_LAYOUT == checkpoint.PACK_LAYOUT
    finally:
        cfgmod.logger.removeHandler(h)
