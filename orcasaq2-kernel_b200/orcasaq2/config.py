"""`quant_method: "exl3"` for vLLM: quantization config, shard-capturing parameter and the
linear method (reference orcasaq2/config.py:1-245, same names and call contract).

An EXL3 pack stores each projection as its own tensor set (trellis, suh, svh, optional codebook
flag tensors), with the bitrate implied by the trellis width.  The shards of a fused vLLM layer
therefore differ in shape and K, so the layer keeps a list of per-shard buffers; shapes are
known only once the loader has delivered the tensors.

Beyond the reference: tensor parallelism.  Any 128-aligned sub-block of an EXL3 matrix is itself
a valid EXL3 matrix (tiles are self-contained, the Hadamard works on independent 128-blocks, the
sign vectors are elementwise), so a rank keeps `trellis[i0/16:i1/16, o0/16:o1/16]`,
`suh[i0:i1]`, `svh[o0:o1]`.  Column-parallel layers slice the outputs of every shard,
row-parallel layers slice the inputs and leave the all-reduce to vLLM's RowParallelLinear.
"""
from typing import Any

import torch
from vllm.logger import init_logger
from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase
from vllm.model_executor.layers.quantization.base_config import (
    QuantizationConfig,
    QuantizeMethodBase,
)
from vllm.model_executor.parameter import BasevLLMParameter

from .ops import GEMM_MAX_ROWS as _GEMM_MAX_ROWS, PACK_LAYOUT, exl3_K  # noqa: F401  (registers the custom ops)

logger = init_logger(__name__)

# Fused vLLM layers and the ids their loaders use for the constituents, in concat order.
SHARD_IDS = {
    "qkv_proj": ["q", "k", "v"],
    "gate_up_proj": [0, 1],
    "in_proj_qkvz": [0, 1],
}

_FUSED_SOURCES = {
    "qkv_proj": ("q_proj", "k_proj", "v_proj"),
    "gate_up_proj": ("gate_proj", "up_proj"),
    "in_proj_qkvz": ("in_proj_qkv", "in_proj_z"),
}

_PLACEHOLDERS = ("trellis", "suh", "svh", "mcg", "mul1", "weight")


def _capture(param, loaded_weight, shard_id=None, **kw):
    """weight_loader of Exl3ShardParam: keep the tensor as delivered, keyed by slot."""
    param.shards[param.slot(shard_id)] = loaded_weight


class Exl3ShardParam(BasevLLMParameter):
    """A zero-size Parameter that collects the real per-shard tensors in `.shards`.

    vLLM wants one Parameter of known shape per weight name; EXL3 shapes are only known when
    the file is read.  The parameter carries its own `weight_loader`, so vLLM's legacy loader
    (which would assert shapes against the placeholder) is never reached (reference
    config.py:28-71)."""

    def __new__(cls, **kwargs):
        return super().__new__(cls, data=torch.empty(0))

    def __init__(self, suffix: str):
        super().__init__(data=torch.empty(0), weight_loader=_capture)
        # dict, not list: the tensor count behind a fused layer need not equal its partition
        # count (in_proj_qkvz: four partitions, two tensors)
        self.shards: dict[int, torch.Tensor] = {}
        self.suffix = suffix

    def slot(self, shard_id):
        if shard_id is None:
            return 0
        if isinstance(shard_id, int):
            return shard_id
        if isinstance(shard_id, tuple):
            return shard_id[0]
        for ids in SHARD_IDS.values():
            if shard_id in ids:
                return ids.index(shard_id)
        raise ValueError(f"unknown shard id {shard_id!r}")

    def load_column_parallel_weight(self, loaded_weight, **kw):
        _capture(self, loaded_weight, kw.get("shard_id", kw.get("loaded_shard_id")))

    load_row_parallel_weight = load_column_parallel_weight
    load_merged_column_weight = load_column_parallel_weight
    load_qkv_weight = load_column_parallel_weight


class Exl3Config(QuantizationConfig):
    """exllamav3 trellis quantization, any per-tensor bitrate (reference config.py:79-151)."""

    def __init__(self, bits: float, codebook: str, head_bits: float, full_config: dict):
        super().__init__()
        self.bits = bits
        self.codebook = codebook
        self.head_bits = head_bits
        self.full_config = full_config
        # The reference tree does not pin the packed format (bit order, order of the weights inside a
        # tile, codebook); this build fixes one and marks the packs it writes.  A pack without the
        # mark loads, but nothing guarantees that it decodes to the weights its producer meant.
        self.layout = full_config.get("exl3_layout")
        if self.layout != PACK_LAYOUT:
            logger.warning(
                "orcasaq2: quantization_config.json carries no \"exl3_layout\": \"%s\" mark (found %r). "
                "This build decodes the trellis layout it defines itself; packs written by other "
                "producers (exllamav3 included) are NOT known to be compatible and may decode to "
                "wrong weights without any error.", PACK_LAYOUT, self.layout)
        storage = full_config.get("tensor_storage") or {}
        self.quantized_prefixes = {
            prefix for prefix, entry in storage.items()
            if any(name.endswith(".trellis") for name in (entry.get("stored_tensors") or {}))
        }

    def __repr__(self):
        return (f"Exl3Config(bits={self.bits}, codebook={self.codebook!r}, "
                f"head_bits={self.head_bits}, quantized={len(self.quantized_prefixes)})")

    @classmethod
    def get_name(cls):
        return "exl3"

    @classmethod
    def get_supported_act_dtypes(cls):
        return [torch.half, torch.bfloat16]

    @classmethod
    def get_min_capability(cls):
        return 100          # the kernels are sm_100a only

    @staticmethod
    def get_config_filenames():
        return ["quantization_config.json"]

    @classmethod
    def from_config(cls, config: dict[str, Any]):
        return cls(bits=float(config.get("bits", 0.0)),
                   codebook=config.get("codebook", "mul1"),
                   head_bits=float(config.get("head_bits", 16)),
                   full_config=config)

    def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> QuantizeMethodBase | None:
        if not isinstance(layer, LinearBase):
            from vllm.model_executor.layers.vocab_parallel_embedding import (
                ParallelLMHead,
                VocabParallelEmbedding,
            )
            if isinstance(layer, ParallelLMHead):
                # an lm_head below 16 bits is an ordinary EXL3 tensor, a dense one falls back, and an int8 table
                # with per-row scales (which the reference can only serve tied to the embedding) is taken too
                from .heads import Exl3LMHeadMethod
                return Exl3LMHeadMethod(self, prefix)
            if isinstance(layer, VocabParallelEmbedding):
                from .heads import Exl3EmbeddingMethod
                return Exl3EmbeddingMethod()
            return None
        if self.quantized_prefixes:
            leaf = prefix.rsplit(".", 1)[-1]
            if not any(name in self.quantized_prefixes for name in _expand(prefix, leaf)):
                try:       # where the reference imports it from (orcasaq2/config.py:144-147)
                    from vllm.model_executor.layers.quantization.unquant import UnquantizedLinearMethod
                except ImportError:   # vLLM 0.22 keeps the class beside the linear layers
                    from vllm.model_executor.layers.linear import UnquantizedLinearMethod
                return UnquantizedLinearMethod()
        return Exl3LinearMethod(self, prefix)

    def get_scaled_act_names(self):
        return []


def _expand(prefix: str, leaf: str) -> list[str]:
    """Fused vLLM module name -> the checkpoint names of its constituents."""
    if leaf in _FUSED_SOURCES:
        stem = prefix[: len(prefix) - len(leaf)]
        return [stem + src for src in _FUSED_SOURCES[leaf]]
    return [prefix]


def slice_shard(trellis, suh, svh, i0: int, i1: int, o0: int, o1: int):
    """The EXL3 matrix restricted to input channels [i0, i1) and output channels [o0, o1);
    all four bounds must sit on 128-boundaries."""
    for v in (i0, i1, o0, o1):
        if v % 128:
            raise RuntimeError(f"EXL3 shard slice [{i0}:{i1}, {o0}:{o1}] is not 128-aligned")
    return (trellis[i0 // 16:i1 // 16, o0 // 16:o1 // 16].contiguous(),
            suh[i0:i1].contiguous(), svh[o0:o1].contiguous())


def _tp_info():
    from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size
    try:
        return get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
    except AssertionError:
        return 0, 1


class Exl3LinearMethod(LinearMethodBase):
    def __init__(self, quant_config: Exl3Config, prefix: str = ""):
        self.quant_config = quant_config
        self.prefix = prefix

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes,
                       input_size, output_size, params_dtype, **extra_weight_attrs):
        # Which form a projection takes (trellis or dense `weight`) is only known from what the
        # loader delivers: register placeholders for both and decide after loading.
        for suffix in _PLACEHOLDERS:
            layer.register_parameter(suffix, Exl3ShardParam(suffix=suffix))
        layer.exl3_out_total = sum(output_partition_sizes)
        # what this rank keeps of the full matrix (the loaders capture full tensors)
        layer.exl3_tp = dict(
            in_part=input_size_per_partition, in_full=input_size,
            out_parts=list(output_partition_sizes), out_full=output_size)

    # ---- tensor-parallel slicing -------------------------------------------------------
    def _slice_for_rank(self, layer, slot_pos, n_slots, tr, suh, svh):
        """Cut one captured shard down to this rank's part."""
        tp = getattr(layer, "exl3_tp", None)
        ic, oc = suh.numel(), svh.numel()
        if tp is None:
            return tr, suh, svh
        rank, world = _tp_info()
        i0, i1, o0, o1 = 0, ic, 0, oc
        if tp["in_part"] != tp["in_full"]:                       # row-parallel
            if ic != tp["in_full"]:
                raise RuntimeError(f"{self.prefix}: shard has {ic} inputs, layer has {tp['in_full']}")
            i0, i1 = rank * tp["in_part"], (rank + 1) * tp["in_part"]
        if sum(tp["out_parts"]) != tp["out_full"]:               # column-parallel
            parts = tp["out_parts"]
            if n_slots == len(parts):
                width = parts[slot_pos]
            elif n_slots == 1:
                width = sum(parts)
            else:
                # fewer tensors than partitions (in_proj_qkvz): split the partitions evenly
                per = len(parts) // n_slots if len(parts) % n_slots == 0 else None
                if per is None:
                    raise RuntimeError(f"{self.prefix}: cannot map {n_slots} tensors onto "
                                       f"{len(parts)} partitions")
                width = sum(parts[slot_pos * per:(slot_pos + 1) * per])
            if width > oc or oc % width:
                raise RuntimeError(f"{self.prefix}: shard of {oc} outputs cannot give {width} per rank")
            groups = oc // width                  # ranks sharing a slice when KV heads replicate
            idx = rank // max(1, world // groups) if groups < world else rank
            o0, o1 = idx * width, (idx + 1) * width
        if (i0, i1, o0, o1) == (0, ic, 0, oc):
            return tr, suh, svh
        return slice_shard(tr, suh, svh, i0, i1, o0, o1)

    def process_weights_after_loading(self, layer) -> None:
        tr, suh, svh = layer.trellis.shards, layer.suh.shards, layer.svh.shards
        mcg, mul1 = layer.mcg.shards, layer.mul1.shards
        dense = layer.weight.shards
        slots = sorted(tr) or sorted(dense)               # shard order == vLLM's concat order
        # the kernels define the default codebook at integer bitrates only; say so at load, not at the first
        # forward (which may already be inside a CUDA-graph capture)
        for i in sorted(tr):
            k_i = exl3_K(tr[i])
            if mcg.get(i) is not None or mul1.get(i) is not None or not isinstance(k_i, int) or not 1 <= k_i <= 8:
                raise RuntimeError(
                    f"{self.prefix}: shard {i} needs the "
                    f"{'mcg' if mcg.get(i) is not None else 'mul1' if mul1.get(i) is not None else 'K=' + str(k_i)} "
                    "decoder, which this build does not define (default 3INST codebook, integer K in 1..8 only)")
        known = [t.device for t in list(tr.values()) + list(dense.values()) if t.device.type == "cuda"]
        dev = known[0] if known else torch.device("cuda", torch.cuda.current_device())

        def drop_placeholders():
            for name in _PLACEHOLDERS:
                if hasattr(layer, name):
                    delattr(layer, name)

        if not tr:
            if not dense:
                raise RuntimeError(f"{self.prefix}: no trellis and no dense weight loaded")
            layer.exl3_shards = None
            w = dense[slots[0]] if len(slots) == 1 else torch.cat([dense[i] for i in slots], 0)
            w = self._slice_dense(layer, w)
            layer.exl3_dense = torch.nn.Parameter(w.contiguous().to(dev), requires_grad=False)
            drop_placeholders()
            return
        if dense:
            raise RuntimeError(f"{self.prefix}: {len(tr)} trellis and {len(dense)} dense shards; "
                               "a fused layer must be all one kind or all the other")
        layer.exl3_dense = None
        shards = []
        for pos, i in enumerate(slots):
            t_i, su_i, sv_i = self._slice_for_rank(layer, pos, len(slots), tr[i], suh[i], svh[i])
            shards.append(dict(
                trellis=t_i.contiguous().to(dev),
                suh=su_i.to(dev, torch.half).contiguous(),
                svh=sv_i.to(dev, torch.half).contiguous(),
                mcg=mcg.get(i) is not None, mul1=mul1.get(i) is not None,
                K=exl3_K(t_i), ic=su_i.numel(), oc=sv_i.numel()))
        layer.exl3_shards = shards
        if dev.type == "cuda":
            from . import _ext
            with torch.cuda.device(dev):
                _ext.ensure_gemv_workspace(dev)        # scratch exists before any capture on this stream
        got = sum(s["oc"] for s in shards)
        if got != layer.exl3_out_total:
            raise RuntimeError(f"{self.prefix}: shards give {got} outputs, layer wants "
                               f"{layer.exl3_out_total}")
        drop_placeholders()

    def _slice_dense(self, layer, w):
        tp = getattr(layer, "exl3_tp", None)
        if tp is None:
            return w
        rank, _ = _tp_info()
        if tp["in_part"] != tp["in_full"]:
            w = w[:, rank * tp["in_part"]:(rank + 1) * tp["in_part"]]
        if sum(tp["out_parts"]) != tp["out_full"] and w.shape[0] == tp["out_full"]:
            if len(tp["out_parts"]) != 1:
                raise NotImplementedError(
                    f"{self.prefix}: a dense fused layer under tensor parallelism is not supported")
            width = tp["out_parts"][0]
            w = w[rank * width:(rank + 1) * width]
        return w

    def apply(self, layer, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if layer.exl3_shards is None:
            out = torch.nn.functional.linear(x, layer.exl3_dense.to(x.dtype))
            return out + bias if bias is not None else out
        rows = x.numel() // x.shape[-1]
        xf = x.reshape(rows, x.shape[-1]).half()
        if not xf.is_contiguous():
            xf = xf.contiguous()
        sh = layer.exl3_shards
        # one opaque node for the whole layer: all shards in one launch, no concatenation
        out = torch.ops.orcasaq2.layer_gemm(
            xf, [s["trellis"] for s in sh], [s["suh"] for s in sh], [s["svh"] for s in sh],
            [s["oc"] for s in sh], [float(s["K"]) for s in sh],
            [s["mcg"] for s in sh], [s["mul1"] for s in sh]).to(x.dtype)
        out = out.reshape(*x.shape[:-1], out.shape[-1])
        return out + bias if bias is not None else out
