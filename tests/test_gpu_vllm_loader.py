"""vLLM's OWN model loader on a synthetic EXL3 checkpoint: `DefaultModelLoader.load_model` builds vLLM's
`Qwen3ForCausalLM`, runs that model's `load_weights` (the HF -> fused renaming q/k/v -> qkv_proj, gate/up ->
gate_up_proj and the shard ids are vLLM's code, vllm/model_executor/models/qwen2.py), and calls every quant
method's `process_weights_after_loading` (vllm/model_executor/model_loader/utils.py).  The plugin is registered the
way vLLM registers it (`orcasaq2.register()`: quantization config "exl3" plus the constructor patch that hands the
config to `embed_tokens` / the tied `lm_head`, reference orcasaq2/__init__.py:64-153).  Then every projection of the
loaded model, the embedding and the logits are compared with the oracle on the tensors read back from disk.
No engine is started and no attention runs (that needs the engine's KV-cache set-up)."""
import socket

import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu

DIMS = dict(layers=2, hidden=256, ffn=384, q_heads=2, kv_heads=1, head_dim=128, vocab=512)


def _close(y, ref, tol=1e-2):
    got = y.float().cpu().numpy().astype(np.float64)
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() / np.abs(ref).max() <= tol


@pytest.fixture(scope="module")
def loaded(ext, tmp_path_factory):
    import orcasaq2
    from orcasaq2 import checkpoint as C
    orcasaq2.register()
    path = str(tmp_path_factory.mktemp("ckpt"))
    dense = "model.layers.1.mlp.down_proj"
    C.write_synthetic_checkpoint(path, seed=33, dense=[dense], max_file_bytes=300_000, **DIMS)
    try:
        from vllm.config import LoadConfig, ModelConfig, VllmConfig, set_current_vllm_config
        from vllm.distributed import parallel_state as ps
        from vllm.model_executor.model_loader import get_model_loader
        mc = ModelConfig(model=path, tokenizer=path, skip_tokenizer_init=True, dtype="float16", max_model_len=128,
                         quantization="exl3")
        vc = VllmConfig(model_config=mc, load_config=LoadConfig())
        with set_current_vllm_config(vc):
            if not ps.model_parallel_is_initialized():
                with socket.socket() as s:
                    s.bind(("127.0.0.1", 0))
                    port = s.getsockname()[1]
                ps.init_distributed_environment(world_size=1, rank=0, local_rank=0, backend="gloo",
                                                distributed_init_method=f"tcp://127.0.0.1:{port}")
                ps.initialize_model_parallel(1, 1)
            model = get_model_loader(vc.load_config).load_model(vllm_config=vc, model_config=mc)
    except Exception as e:                                              # noqa: BLE001
        pytest.skip(f"vLLM's loader cannot run outside an engine here: {type(e).__name__}: {str(e)[:300]}")
    tensors, storage = C.synthetic_tensors(seed=33, dense=[dense], **DIMS)
    return model, tensors, storage, dense


def test_vllm_load_weights_fills_the_plugin_layers(loaded, coracle):
    from orcasaq2 import config as cfg
    from orcasaq2.heads import Exl3EmbeddingMethod
    model, tensors, storage, dense = loaded
    hf = {"self_attn.qkv_proj": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
          "mlp.gate_up_proj": ["mlp.gate_proj", "mlp.up_proj"]}
    checked = 0
    for li, layer in enumerate(model.model.layers):
        for suffix, mod in (("self_attn.qkv_proj", layer.self_attn.qkv_proj), ("self_attn.o_proj", layer.self_attn.o_proj),
                            ("mlp.gate_up_proj", layer.mlp.gate_up_proj), ("mlp.down_proj", layer.mlp.down_proj)):
            name = f"model.layers.{li}.{suffix}"
            parts = [f"model.layers.{li}.{s}" for s in hf.get(suffix, [suffix])]
            x = torch.randn((3, mod.input_size), generator=torch.Generator().manual_seed(len(name) + li)).half()
            out = mod(x.cuda())
            y = out[0] if isinstance(out, tuple) else out
            if name == dense:
                # vLLM hands from_config the `quantization_config` of config.json, which has no `tensor_storage`
                # manifest (vllm/model_executor/model_loader/weight_utils.py, get_quant_config), so the layer gets
                # the EXL3 method and falls back to the dense weight it was given (reference orcasaq2/config.py:202-210,228-231);
                # with the manifest present it would get vLLM's unquantized method.  Either way: no trellis.
                assert not getattr(mod, "exl3_shards", None)
                ref = x.double().numpy() @ tensors[dense + ".weight"].double().numpy().T
            else:
                assert isinstance(mod.quant_method, cfg.Exl3LinearMethod) and not hasattr(mod, "trellis")
                assert [s["K"] for s in mod.exl3_shards] == [storage[p]["bits_per_weight"] for p in parts]
                ref = np.concatenate([coracle.layer(x.numpy(), coracle.reconstruct(tensors[p + ".trellis"].numpy()),
                                                    tensors[p + ".suh"].numpy(), tensors[p + ".svh"].numpy())
                                      for p in parts], 1)
            _close(y, ref)
            checked += 1
    assert checked == 4 * DIMS["layers"]
    # the constructor patch gave the embedding the plugin's method; the tied head is the same module
    emb = model.model.embed_tokens
    assert isinstance(emb.quant_method, Exl3EmbeddingMethod) and emb.exl3_embed_q.dtype == torch.int8
    q, s = tensors["model.embed_tokens.qweight"], tensors["model.embed_tokens.scales"]
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)   # noqa: E731
    ids = torch.tensor([0, 5, DIMS["vocab"] - 1]).cuda()
    got = emb(ids)
    assert np.array_equal(bits(got), coracle.int8_embed(q.numpy(), bits(s.half()), ids.cpu().numpy(), False))
    h = torch.randn((4, DIMS["hidden"]), generator=torch.Generator().manual_seed(9)).half()
    logits = model.compute_logits(h.cuda())
    lref = coracle.int8_head(q.numpy(), bits(s.half()), bits(h), False)
    _close(logits[:, :DIMS["vocab"]], lref)
