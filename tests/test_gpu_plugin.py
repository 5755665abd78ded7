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
