"""The vLLM-facing classes on the GPU, driven the way vLLM drives them (create_weights -> the
parameter's weight_loader per shard -> process_weights_after_loading -> apply / embedding), against
the CPU oracle.  No engine is started; the tensor-parallel group lookups are patched to one rank."""
import types

import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cfg(ext):
    import vllm.model_executor.parameter as vp
    vp.get_tensor_model_parallel_rank = lambda: 0
    vp.get_tensor_model_parallel_world_size = lambda: 1
    from orcasaq2 import config
    config._tp_info = lambda: (0, 1)
    return config


def _close(y, ref, tol=1e-2):
    got = y.float().cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= tol


@pytest.mark.parametrize("rows", [1, 6, 40])
def test_linear_method_fused_qkv(cfg, coracle, rows):
    ic, spec = 256, [("q", 384, 4), ("k", 128, 5), ("v", 128, 6)]
    method = cfg.Exl3LinearMethod(cfg.Exl3Config.from_config({}), "model.layers.0.self_attn.qkv_proj")
    layer = torch.nn.Module()
    method.create_weights(layer, ic, [384, 128, 128], ic, 640, torch.bfloat16)
    refs = []
    x = torch.randn((2, rows // 2 if rows > 1 else 1, ic), generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    if rows == 1:
        x = x[:1]
    for i, (sid, oc, K) in enumerate(spec):
        tr, suh, svh, _ = R.make_layer(500 + i, ic, oc, K, 1)
        # loaders hand tensors over on the CPU, keyed by vLLM's shard ids
        layer.trellis.weight_loader(layer.trellis, tr, sid)
        layer.suh.weight_loader(layer.suh, suh, sid)
        layer.svh.weight_loader(layer.svh, svh, sid)
        xf = x.reshape(-1, ic).half()
        refs.append(coracle.layer(xf.numpy(), coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy()))
    method.process_weights_after_loading(layer)
    assert not hasattr(layer, "trellis") and layer.exl3_dense is None
    assert [s["K"] for s in layer.exl3_shards] == [4, 5, 6] and [s["oc"] for s in layer.exl3_shards] == [384, 128, 128]
    assert all(s["trellis"].is_cuda for s in layer.exl3_shards)
    bias = torch.randn(640, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    y = method.apply(layer, x.cuda(), bias)
    assert y.shape == (*x.shape[:-1], 640) and y.dtype == torch.bfloat16
    ref = np.concatenate(refs, 1) + bias.float().cpu().numpy()[None, :]
    _close(y.reshape(-1, 640), ref, tol=2e-2)          # bf16 output rounding on top of the layer tolerance


def test_linear_method_dense_fallback_and_errors(cfg):
    method = cfg.Exl3LinearMethod(cfg.Exl3Config.from_config({}), "model.layers.0.mlp.gate")
    layer = torch.nn.Module()
    method.create_weights(layer, 64, [32], 64, 32, torch.half)
    w = torch.randn(32, 64).half()
    layer.weight.weight_loader(layer.weight, w)
    method.process_weights_after_loading(layer)
    assert layer.exl3_shards is None and layer.exl3_dense.is_cuda
    x = torch.randn(3, 64).half().cuda()
    assert torch.allclose(method.apply(layer, x), x @ w.cuda().t(), atol=1e-2)
    empty = torch.nn.Module()
    method.create_weights(empty, 64, [32], 64, 32, torch.half)
    with pytest.raises(RuntimeError, match="no trellis and no dense"):
        method.process_weights_after_loading(empty)
    bad = torch.nn.Module()
    method.create_weights(bad, 128, [256], 128, 256, torch.half)
    tr, suh, svh, _ = R.make_layer(1, 128, 128, 4, 1)
    for name, t in (("trellis", tr), ("suh", suh), ("svh", svh)):
        getattr(bad, name).weight_loader(getattr(bad, name), t)
    with pytest.raises(RuntimeError, match="outputs, layer wants"):
        method.process_weights_after_loading(bad)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_embedding_method(ext, coracle, dtype):
    from orcasaq2.heads import Exl3EmbeddingMethod
    m = Exl3EmbeddingMethod()
    layer = torch.nn.Module()
    m.create_weights(layer, 128, [300], 128, 300, dtype)
    q, s = R.make_int8_table(9, 300, 128, dtype)
    layer.qweight.weight_loader(layer.qweight, q)
    layer.scales.weight_loader(layer.scales, s)
    m.process_weights_after_loading(layer)
    assert layer.exl3_embed is None and layer.exl3_embed_q.dtype == torch.int8 and layer.exl3_embed_s.shape == (300, 1)
    ids = torch.tensor([[0, 299], [17, 5]]).cuda()
    out = m.embedding(layer, ids)
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)   # noqa: E731
    ref = coracle.int8_embed(q.numpy(), bits(s), ids.cpu().numpy(), dtype == torch.bfloat16)
    assert np.array_equal(bits(out).reshape(-1, 128), ref)
    x = torch.randn((2, 3, 128), generator=torch.Generator().manual_seed(2)).to(dtype)
    logits = m.apply(layer, x.cuda())
    assert logits.shape == (2, 3, 300) and logits.dtype == dtype
    lref = coracle.int8_head(q.numpy(), bits(s), bits(x).reshape(6, 128), dtype == torch.bfloat16)
    _close(logits.reshape(6, 300), lref, tol=1e-2)
    with pytest.raises(RuntimeError, match="qweight without scales"):
        lay2 = torch.nn.Module()
        m.create_weights(lay2, 128, [300], 128, 300, dtype)
        lay2.qweight.weight_loader(lay2.qweight, q)
        m.process_weights_after_loading(lay2)


def test_int8_embedding_table_module(ext, coracle):
    from orcasaq2.patches.int8_embedding import Int8EmbeddingTable
    q, s = R.make_int8_table(4, 64, 128, torch.float16)
    tab = Int8EmbeddingTable(q.cuda(), s.cuda(), torch.float16)
    ids = torch.tensor([3, 63, 0]).cuda()
    out = tab(ids)
    ref = coracle.int8_embed(q.numpy(), s.view(torch.int16).numpy().view(np.uint16), ids.cpu().numpy(), False)
    assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), ref)


# ---- the same flow on vLLM's own layer classes (reference callers: vllm linear.py:585, 1556) ----------
@pytest.fixture(scope="module")
def vllm_layers(cfg):
    """A vLLM config context and a one-rank model-parallel state, so that vLLM's own linear layers
    can be constructed with this plugin's quantization config.  Anything vLLM refuses to set up
    outside an engine skips these tests instead of failing them."""
    import socket
    ctx = None
    try:
        from vllm.config import VllmConfig, set_current_vllm_config
        from vllm.distributed import parallel_state as ps
        ctx = set_current_vllm_config(VllmConfig())
        ctx.__enter__()
        if not ps.model_parallel_is_initialized():
            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                port = s.getsockname()[1]
            ps.init_distributed_environment(world_size=1, rank=0, local_rank=0, backend="gloo",
                                            distributed_init_method=f"tcp://127.0.0.1:{port}")
            ps.initialize_model_parallel(1, 1)
        from vllm.model_executor.layers import linear
    except Exception as e:                                            # noqa: BLE001
        if ctx is not None:
            ctx.__exit__(None, None, None)
        pytest.skip(f"vLLM layers cannot be constructed outside an engine here: {type(e).__name__}: {e}")
    yield linear
    ctx.__exit__(None, None, None)


def _load(layer, specs, ic, seed):
    """Hand every shard to the parameters' own weight_loader, as vLLM's model loaders do."""
    refs = []
    for i, (sid, oc, K) in enumerate(specs):
        tr, suh, svh, _ = R.make_layer(seed + i, ic, oc, K, 1)
        for name, t in (("trellis", tr), ("suh", suh), ("svh", svh)):
            p = getattr(layer, name)
            p.weight_loader(p, t, sid)
        refs.append((tr, suh, svh))
    return refs


@pytest.mark.parametrize("rows", [1, 24])
def test_vllm_qkv_merged_and_row_parallel_layers(vllm_layers, cfg, coracle, rows):
    L = vllm_layers
    qc = cfg.Exl3Config.from_config({})
    hidden, head, ffn = 256, 128, 384
    qkv = L.QKVParallelLinear(hidden, head, 3, 1, bias=False, quant_config=qc, params_dtype=torch.bfloat16,
                              prefix="model.layers.0.self_attn.qkv_proj")
    gate_up = L.MergedColumnParallelLinear(hidden, [ffn, ffn], bias=False, quant_config=qc, params_dtype=torch.bfloat16,
                                           prefix="model.layers.0.mlp.gate_up_proj")
    down = L.RowParallelLinear(ffn, hidden, bias=False, quant_config=qc, params_dtype=torch.bfloat16,
                               prefix="model.layers.0.mlp.down_proj")
    for layer in (qkv, gate_up, down):
        assert isinstance(layer.quant_method, cfg.Exl3LinearMethod)
    cases = [(qkv, [("q", 3 * head, 4), ("k", head, 5), ("v", head, 6)], hidden),
             (gate_up, [(0, ffn, 3), (1, ffn, 3)], hidden),
             (down, [(None, hidden, 4)], ffn)]
    for li, (layer, specs, ic) in enumerate(cases):
        refs = _load(layer, specs, ic, 900 + 10 * li)
        layer.quant_method.process_weights_after_loading(layer)
        x = torch.randn((rows, ic), generator=torch.Generator().manual_seed(li + rows)).to(torch.bfloat16)
        out = layer(x.cuda())
        y = out[0] if isinstance(out, tuple) else out
        xf = x.half().numpy()
        ref = np.concatenate([coracle.layer(xf, coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy())
                              for tr, suh, svh in refs], 1)
        assert y.shape == (rows, sum(oc for _, oc, _ in specs)) and y.dtype == torch.bfloat16
        _close(y, ref, tol=2e-2)


def test_vllm_layers_loaded_from_a_checkpoint_on_disk(vllm_layers, cfg, coracle, tmp_path):
    """A synthetic checkpoint (safetensors + quantization_config.json with its manifest) is read back from
    disk and delivered through the parameters' own weight loaders under vLLM's stacked renaming; the
    manifest decides which layers are EXL3 and which stay dense; every layer's output matches the oracle."""
    from orcasaq2 import checkpoint as C
    L = vllm_layers
    dims = dict(layers=2, hidden=256, ffn=384, q_heads=3, kv_heads=1, head_dim=128, vocab=300)
    dense = "model.layers.1.self_attn.o_proj"
    C.write_synthetic_checkpoint(str(tmp_path), seed=21, dense=[dense], max_file_bytes=200_000, **dims)
    qc = cfg.Exl3Config.from_config(C.read_quantization_config(str(tmp_path)))
    H, F, QH, KVH, HD = (dims[k] for k in ("hidden", "ffn", "q_heads", "kv_heads", "head_dim"))
    modules = {}
    for li in range(dims["layers"]):
        p = f"model.layers.{li}."
        kw = dict(bias=False, quant_config=qc, params_dtype=torch.float16)
        modules[p + "self_attn.qkv_proj"] = L.QKVParallelLinear(H, HD, QH, KVH, prefix=p + "self_attn.qkv_proj", **kw)
        modules[p + "self_attn.o_proj"] = L.RowParallelLinear(QH * HD, H, prefix=p + "self_attn.o_proj", **kw)
        modules[p + "mlp.gate_up_proj"] = L.MergedColumnParallelLinear(H, [F, F], prefix=p + "mlp.gate_up_proj", **kw)
        modules[p + "mlp.down_proj"] = L.RowParallelLinear(F, H, prefix=p + "mlp.down_proj", **kw)
    for name, m in modules.items():
        want = cfg.Exl3LinearMethod if name != dense else L.UnquantizedLinearMethod
        assert isinstance(m.quant_method, want), name
    unused = C.load_into(modules, C.iter_checkpoint_tensors(str(tmp_path)))
    assert all(n.endswith("norm.weight") or n.startswith("model.embed_tokens") for n in unused)
    tensors, storage = C.synthetic_tensors(seed=21, dense=[dense], **dims)
    hf = {"self_attn.qkv_proj": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
          "mlp.gate_up_proj": ["mlp.gate_proj", "mlp.up_proj"]}
    for name, m in modules.items():
        m.cuda()
        m.quant_method.process_weights_after_loading(m)
        ic = m.input_size
        x = torch.randn((3, ic), generator=torch.Generator().manual_seed(len(name))).half()
        out = m(x.cuda())
        y = out[0] if isinstance(out, tuple) else out
        li, suffix = name.split(".")[2], name.split(".", 3)[3]
        parts = [f"model.layers.{li}.{s}" for s in hf.get(suffix, [suffix])]
        if name == dense:
            ref = x.double().numpy() @ tensors[dense + ".weight"].double().numpy().T
        else:
            assert [s["K"] for s in m.exl3_shards] == [storage[p]["bits_per_weight"] for p in parts]
            ref = np.concatenate([coracle.layer(x.numpy(), coracle.reconstruct(tensors[p + ".trellis"].numpy()),
                                                tensors[p + ".suh"].numpy(), tensors[p + ".svh"].numpy())
                                  for p in parts], 1)
        assert y.dtype == torch.float16 and y.shape == ref.shape
        _close(y, ref, tol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_untied_int8_lm_head_on_vllm_layer(vllm_layers, cfg, ext, coracle, dtype):
    """An untied `ParallelLMHead` whose checkpoint carries `lm_head.qweight` / `lm_head.scales`: the reference has
    no slot for them (orcasaq2/config.py:128-132,183); here the head loads and runs on the int8 kernel."""
    from vllm.model_executor.layers.vocab_parallel_embedding import ParallelLMHead
    from orcasaq2.heads import Exl3LMHeadMethod
    qc = cfg.Exl3Config.from_config({"head_bits": 8})
    head = ParallelLMHead(300, 128, params_dtype=dtype, quant_config=qc, prefix="lm_head")
    assert isinstance(head.quant_method, Exl3LMHeadMethod)
    q, s = R.make_int8_table(31, 300, 128, dtype)
    head.qweight.weight_loader(head.qweight, q)
    head.scales.weight_loader(head.scales, s)
    head.quant_method.process_weights_after_loading(head)
    assert head.exl3_embed_q.dtype == torch.int8 and head.exl3_embed_q.is_cuda and head.exl3_shards is None
    x = torch.randn((5, 128), generator=torch.Generator().manual_seed(4)).to(dtype)
    logits = head.quant_method.apply(head, x.cuda())
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)   # noqa: E731
    lref = coracle.int8_head(q.numpy(), bits(s), bits(x), dtype == torch.bfloat16)
    assert logits.shape[0] == 5 and logits.dtype == dtype
    _close(logits[:, :300], lref, tol=1e-2)


def test_lm_head_method_other_forms_and_errors(cfg, ext, coracle):
    """The same method still serves a trellis head (the reference's only untied form) and refuses half a table."""
    from orcasaq2.heads import Exl3LMHeadMethod
    m = Exl3LMHeadMethod(cfg.Exl3Config.from_config({}), "lm_head")
    layer = torch.nn.Module()
    m.create_weights(layer, 128, [256], 128, 256, torch.half)
    tr, suh, svh, x = R.make_layer(77, 128, 256, 4, 3)
    for name, t in (("trellis", tr), ("suh", suh), ("svh", svh)):
        getattr(layer, name).weight_loader(getattr(layer, name), t)
    m.process_weights_after_loading(layer)
    assert layer.exl3_embed_q is None and layer.exl3_shards[0]["K"] == 4
    y = m.apply(layer, x.cuda())
    _close(y, coracle.layer(x.numpy(), coracle.reconstruct(tr.numpy()), suh.numpy(), svh.numpy()))
    half = torch.nn.Module()
    m.create_weights(half, 128, [300], 128, 300, torch.half)
    q, s = R.make_int8_table(3, 300, 128)
    half.scales.weight_loader(half.scales, s)
    with pytest.raises(RuntimeError, match="scales without qweight"):
        m.process_weights_after_loading(half)
    both = torch.nn.Module()
    m.create_weights(both, 128, [300], 128, 300, torch.half)
    both.qweight.weight_loader(both.qweight, q)
    both.scales.weight_loader(both.scales, s)
    both.weight.weight_loader(both.weight, torch.zeros(300, 128).half())
    with pytest.raises(RuntimeError, match="another form"):
        m.process_weights_after_loading(both)
