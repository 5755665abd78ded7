"""Synthetic EXL3 checkpoints on disk, and the name mapping a loader applies to them.

The reference is only ever exercised against a real quantised pack; there is no network here and
no such pack, so this module writes one with the same file set and tensor names from a seed:

    model-0000i-of-0000n.safetensors, model.safetensors.index.json   the tensors
    quantization_config.json   {"quant_method": "exl3", "bits", "codebook", "head_bits",
                                "tensor_storage": {module: {"stored_tensors": {name: {...}}}}}
                               (file name: orcasaq2/config.py:111-113; the manifest is what
                               Exl3Config reads to find the quantised modules, config.py:89-93)
    config.json                the architecture, with the quantization config embedded

Per linear projection `P` (names as the loader sees them before fusion, orcasaq2/config.py:183):
`P.trellis` int16 [ic/16, oc/16, 16K], `P.suh` fp16 [ic], `P.svh` fp16 [oc]; a projection left
dense carries `P.weight` [oc, ic] instead.  The embedding carries `model.embed_tokens.qweight`
int8 [V, H] and `model.embed_tokens.scales` fp16 [V] (orcasaq2/heads.py:35), norms are plain
`weight` vectors.  Values: uniform-random trellis words, +-1 sign vectors, seeded per tensor.

`load_into` walks such a checkpoint the way vLLM's model loaders do (stacked-parameter mapping
q/k/v -> qkv_proj, gate/up -> gate_up_proj, then `param.weight_loader(param, tensor, shard_id)`,
vllm/model_executor/models/qwen3_5.py:277-343), so that `create_weights` -> `_capture` ->
`process_weights_after_loading` -> `apply` run unchanged on modules built from vLLM's layer classes.
"""
from __future__ import annotations

import json
import os
from typing import Iterable, Iterator

import torch

from .ops import PACK_LAYOUT

# HF projection name -> (fused vLLM parameter name, shard id)
STACKED = {
    "q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
    "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1),
}


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def _exl3_tensors(seed: int, ic: int, oc: int, K: int) -> dict[str, torch.Tensor]:
    g = _gen(seed)
    tr = torch.randint(0, 65536, (ic // 16, oc // 16, 16 * K), generator=g, dtype=torch.int32).to(torch.int16)
    suh = (torch.randint(0, 2, (ic,), generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (oc,), generator=g) * 2 - 1).to(torch.float16)
    return {"trellis": tr, "suh": suh, "svh": svh}


def layer_projections(hidden: int, ffn: int, q_heads: int, kv_heads: int, head_dim: int):
    """(HF module suffix, ic, oc) of the seven projections of one decoder layer."""
    return [("self_attn.q_proj", hidden, q_heads * head_dim), ("self_attn.k_proj", hidden, kv_heads * head_dim),
            ("self_attn.v_proj", hidden, kv_heads * head_dim), ("self_attn.o_proj", q_heads * head_dim, hidden),
            ("mlp.gate_proj", hidden, ffn), ("mlp.up_proj", hidden, ffn), ("mlp.down_proj", ffn, hidden)]


def synthetic_tensors(*, layers: int, hidden: int, ffn: int, q_heads: int, kv_heads: int, head_dim: int,
                      vocab: int, seed: int = 0, bits: Iterable[int] = (2, 3, 4, 5, 6),
                      dense: Iterable[str] = ()) -> tuple[dict[str, torch.Tensor], dict]:
    """All tensors of a synthetic decoder plus the `tensor_storage` manifest.

    Every projection draws its bitrate from `bits` with the seed (the mixed allocation of a real
    pack); module names listed in `dense` are stored as fp16 `weight` instead of a trellis."""
    for n, v in (("hidden", hidden), ("ffn", ffn), ("q_heads*head_dim", q_heads * head_dim),
                 ("kv_heads*head_dim", kv_heads * head_dim)):
        if v % 128:
            raise ValueError(f"{n} = {v} is not a multiple of 128")
    bits = list(bits)
    dense = set(dense)
    pick = _gen(seed)
    tensors: dict[str, torch.Tensor] = {}
    storage: dict[str, dict] = {}

    def put(module: str, name: str, t: torch.Tensor):
        tensors[f"{module}.{name}"] = t
        storage.setdefault(module, {"stored_tensors": {}})["stored_tensors"][f"{module}.{name}"] = {
            "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")}

    tseed = seed * 100003 + 1
    for li in range(layers):
        for suffix, ic, oc in layer_projections(hidden, ffn, q_heads, kv_heads, head_dim):
            module = f"model.layers.{li}.{suffix}"
            K = bits[int(torch.randint(0, len(bits), (1,), generator=pick))]
            tseed += 1
            if module in dense:
                put(module, "weight", (torch.randn((oc, ic), generator=_gen(tseed)) * 0.02).to(torch.float16))
                continue
            for name, t in _exl3_tensors(tseed, ic, oc, K).items():
                put(module, name, t)
            storage[module]["bits_per_weight"] = K
        for norm in ("input_layernorm", "post_attention_layernorm"):
            tseed += 1
            put(f"model.layers.{li}.{norm}", "weight", (1.0 + 0.1 * torch.randn((hidden,), generator=_gen(tseed))).to(torch.float16))
    g = _gen(tseed + 1)
    put("model.embed_tokens", "qweight", torch.randint(-127, 128, (vocab, hidden), generator=g, dtype=torch.int32).to(torch.int8))
    put("model.embed_tokens", "scales", (torch.rand((vocab,), generator=g) * 0.02 + 1e-3).to(torch.float16))
    put("model.norm", "weight", (1.0 + 0.1 * torch.randn((hidden,), generator=g)).to(torch.float16))
    return tensors, storage


def write_synthetic_checkpoint(path: str, *, layers: int, hidden: int, ffn: int, q_heads: int, kv_heads: int,
                               head_dim: int, vocab: int, seed: int = 0, bits: Iterable[int] = (2, 3, 4, 5, 6),
                               dense: Iterable[str] = (), max_file_bytes: int = 1 << 30) -> dict:
    """Write the file set described in the module docstring into directory `path`; returns the
    quantization config that was written."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    bits = list(bits)
    tensors, storage = synthetic_tensors(layers=layers, hidden=hidden, ffn=ffn, q_heads=q_heads, kv_heads=kv_heads,
                                         head_dim=head_dim, vocab=vocab, seed=seed, bits=bits, dense=dense)
    # split into files in name order, as sharded checkpoints are
    files: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name in sorted(tensors):
        nbytes = tensors[name].numel() * tensors[name].element_size()
        if files[-1] and size + nbytes > max_file_bytes:
            files.append({})
            size = 0
        files[-1][name] = tensors[name]
        size += nbytes
    weight_map = {}
    for i, chunk in enumerate(files):
        fname = f"model-{i + 1:05d}-of-{len(files):05d}.safetensors"
        save_file({k: v.contiguous() for k, v in chunk.items()}, os.path.join(path, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in chunk})
    total = sum(t.numel() * t.element_size() for t in tensors.values())
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    kbits = [v["bits_per_weight"] for v in storage.values() if "bits_per_weight" in v]
    qcfg = {"quant_method": "exl3", "bits": round(sum(kbits) / max(1, len(kbits)), 3), "codebook": "3inst", "exl3_layout": PACK_LAYOUT,
            "head_bits": 8, "tensor_storage": storage}
    with open(os.path.join(path, "quantization_config.json"), "w") as f:
        json.dump(qcfg, f, indent=1)
    arch = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": hidden,
            "intermediate_size": ffn, "num_hidden_layers": layers, "num_attention_heads": q_heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim, "vocab_size": vocab, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": True, "torch_dtype": "float16", "rope_theta": 10000.0,
            "max_position_embeddings": 4096,
            "quantization_config": {k: v for k, v in qcfg.items() if k != "tensor_storage"}}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(arch, f, indent=1)
    return qcfg


def read_quantization_config(path: str) -> dict:
    with open(os.path.join(path, "quantization_config.json")) as f:
        return json.load(f)


def iter_checkpoint_tensors(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, CPU tensor) for every tensor of the checkpoint, file by file, like vLLM's safetensors
    weight iterator."""
    from safetensors import safe_open

    with open(os.path.join(path, "model.safetensors.index.json")) as f:
        weight_map = json.load(f)["weight_map"]
    for fname in sorted(set(weight_map.values())):
        with safe_open(os.path.join(path, fname), framework="pt", device="cpu") as sf:
            for name in sf.keys():
                yield name, sf.get_tensor(name)


def load_into(modules: dict[str, torch.nn.Module], weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
    """Deliver checkpoint tensors to `modules` (vLLM module prefix -> module) through each parameter's
    own `weight_loader`, with vLLM's stacked-parameter renaming.  Returns the tensor names that found
    no module (a loader would report them); an unknown parameter of a known module raises KeyError."""
    unused = set()
    for name, tensor in weights:
        module_name, _, pname = name.rpartition(".")
        parent, _, leaf = module_name.rpartition(".")
        shard_id = None
        if leaf in STACKED and f"{parent}.{STACKED[leaf][0]}" in modules:
            fused, shard_id = STACKED[leaf]
            module_name = f"{parent}.{fused}"
        mod = modules.get(module_name)
        if mod is None:
            unused.add(name)
            continue
        params = dict(mod.named_parameters(recurse=False))
        if pname not in params:
            raise KeyError(f"{module_name} has no parameter {pname!r} (checkpoint tensor {name})")
        p = params[pname]
        loader = getattr(p, "weight_loader", None)
        if loader is None:
            with torch.no_grad():
                p.copy_(tensor)
        elif shard_id is None:
            loader(p, tensor)
        else:
            loader(p, tensor, shard_id)
    return unused
