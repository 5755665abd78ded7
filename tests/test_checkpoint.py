"""Synthetic EXL3 checkpoint: the file set, the manifest the quantization config reads, and delivery of
the tensors to the plugin's placeholder parameters under vLLM's stacked-parameter renaming (CPU only;
the GPU leg is in test_gpu_plugin.py)."""
import json
import os

import pytest
import torch

DIMS = dict(layers=2, hidden=256, ffn=384, q_heads=3, kv_heads=1, head_dim=128, vocab=500)
DENSE = "model.layers.1.self_attn.o_proj"


@pytest.fixture(scope="module")
def cfgmod():
    import vllm.model_executor.parameter as vp
    vp.get_tensor_model_parallel_rank = lambda: 0
    vp.get_tensor_model_parallel_world_size = lambda: 1
    from orcasaq2 import config
    return config


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    from orcasaq2 import checkpoint as C
    d = str(tmp_path_factory.mktemp("exl3_ckpt"))
    q = C.write_synthetic_checkpoint(d, seed=5, dense=[DENSE], max_file_bytes=150_000, **DIMS)
    return C, d, q


def test_file_set_and_index(ckpt):
    C, d, q = ckpt
    names = sorted(os.listdir(d))
    shards = [n for n in names if n.endswith(".safetensors")]
    assert len(shards) > 1 and {"config.json", "quantization_config.json", "model.safetensors.index.json"} <= set(names)
    index = json.load(open(os.path.join(d, "model.safetensors.index.json")))
    tensors, _ = C.synthetic_tensors(seed=5, dense=[DENSE], **DIMS)
    assert set(index["weight_map"]) == set(tensors)
    assert index["metadata"]["total_size"] == sum(t.numel() * t.element_size() for t in tensors.values())
    got = dict(C.iter_checkpoint_tensors(d))
    assert set(got) == set(tensors)
    for k, t in tensors.items():                       # same seed, same bytes
        assert got[k].dtype == t.dtype and torch.equal(got[k], t), k
    assert json.load(open(os.path.join(d, "config.json")))["quantization_config"]["quant_method"] == "exl3"


def test_shapes_follow_the_packed_format(ckpt):
    C, d, q = ckpt
    st = q["tensor_storage"]
    for li in range(DIMS["layers"]):
        for suffix, ic, oc in C.layer_projections(DIMS["hidden"], DIMS["ffn"], DIMS["q_heads"], DIMS["kv_heads"], DIMS["head_dim"]):
            mod = f"model.layers.{li}.{suffix}"
            stored = st[mod]["stored_tensors"]
            if mod == DENSE:
                assert list(stored) == [mod + ".weight"] and stored[mod + ".weight"]["shape"] == [oc, ic]
                continue
            K = st[mod]["bits_per_weight"]
            assert 2 <= K <= 6
            assert stored[mod + ".trellis"] == {"shape": [ic // 16, oc // 16, 16 * K], "dtype": "int16"}
            assert stored[mod + ".suh"]["shape"] == [ic] and stored[mod + ".svh"]["shape"] == [oc]
    assert st["model.embed_tokens"]["stored_tensors"]["model.embed_tokens.qweight"]["dtype"] == "int8"
    with pytest.raises(ValueError):
        C.synthetic_tensors(**{**DIMS, "ffn": 200})


def test_manifest_drives_the_quantization_config(ckpt, cfgmod):
    C, d, _ = ckpt
    qc = cfgmod.Exl3Config.from_config(C.read_quantization_config(d))
    assert qc.get_name() == "exl3" and qc.codebook == "3inst" and qc.head_bits == 8
    assert "model.layers.0.self_attn.q_proj" in qc.quantized_prefixes
    assert "model.layers.1.mlp.down_proj" in qc.quantized_prefixes
    assert DENSE not in qc.quantized_prefixes                       # stored as a plain weight
    assert "model.embed_tokens" not in qc.quantized_prefixes        # int8 table, not a trellis
    assert cfgmod.Exl3Config.get_config_filenames() == ["quantization_config.json"]


def test_load_into_placeholders_with_stacked_renaming(ckpt, cfgmod):
    C, d, _ = ckpt
    qc = cfgmod.Exl3Config.from_config(C.read_quantization_config(d))
    H, F, QH, KVH, HD = (DIMS[k] for k in ("hidden", "ffn", "q_heads", "kv_heads", "head_dim"))
    spec = {"self_attn.qkv_proj": (H, [QH * HD, KVH * HD, KVH * HD]), "self_attn.o_proj": (QH * HD, [H]),
            "mlp.gate_up_proj": (H, [F, F]), "mlp.down_proj": (F, [H])}
    modules = {}
    for li in range(DIMS["layers"]):
        for suffix, (ic, parts) in spec.items():
            m = torch.nn.Module()
            cfgmod.Exl3LinearMethod(qc, f"model.layers.{li}.{suffix}").create_weights(m, ic, parts, ic, sum(parts), torch.half)
            modules[f"model.layers.{li}.{suffix}"] = m
    from orcasaq2.heads import Exl3EmbeddingMethod
    emb = torch.nn.Module()
    Exl3EmbeddingMethod().create_weights(emb, H, [DIMS["vocab"]], H, DIMS["vocab"], torch.half)
    modules["model.embed_tokens"] = emb
    unused = C.load_into(modules, C.iter_checkpoint_tensors(d))
    assert unused == {f"model.layers.{li}.{n}.weight" for li in range(DIMS["layers"])
                      for n in ("input_layernorm", "post_attention_layernorm")} | {"model.norm.weight"}
    tensors, _ = C.synthetic_tensors(seed=5, dense=[DENSE], **DIMS)
    qkv = modules["model.layers.0.self_attn.qkv_proj"]
    for slot, hf in enumerate(("q_proj", "k_proj", "v_proj")):      # shard ids "q","k","v" -> slots 0,1,2
        for name in ("trellis", "suh", "svh"):
            assert torch.equal(getattr(qkv, name).shards[slot], tensors[f"model.layers.0.self_attn.{hf}.{name}"])
    gu = modules["model.layers.1.mlp.gate_up_proj"]
    assert torch.equal(gu.trellis.shards[1], tensors["model.layers.1.mlp.up_proj.trellis"]) and set(gu.trellis.shards) == {0, 1}
    o1 = modules[DENSE]
    assert not o1.trellis.shards and torch.equal(o1.weight.shards[0], tensors[DENSE + ".weight"])
    assert torch.equal(emb.qweight.shards[0], tensors["model.embed_tokens.qweight"]) and 0 in emb.scales.shards
    with pytest.raises(KeyError):
        C.load_into({"model.norm": torch.nn.Module()}, [("model.norm.weight", torch.ones(4))])


def test_dense_module_gets_the_unquantized_method(ckpt, cfgmod):
    """A linear layer the manifest does not list as a trellis is routed to vLLM's dense method
    (reference: orcasaq2/config.py:141-147), a fused layer with quantised members to the EXL3 one."""
    from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
    C, d, _ = ckpt
    qc = cfgmod.Exl3Config.from_config(C.read_quantization_config(d))
    fake = LinearBase.__new__(LinearBase)              # only its type is looked at
    assert isinstance(qc.get_quant_method(fake, DENSE), UnquantizedLinearMethod)
    assert isinstance(qc.get_quant_method(fake, "model.layers.0.self_attn.qkv_proj"), cfgmod.Exl3LinearMethod)
    assert isinstance(qc.get_quant_method(fake, "model.layers.1.mlp.gate_up_proj"), cfgmod.Exl3LinearMethod)
