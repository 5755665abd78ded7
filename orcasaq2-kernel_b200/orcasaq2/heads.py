"""Embedding table and tied output head for vLLM's VocabParallelEmbedding family
(reference orcasaq2/heads.py:1-75, same class and method names).

`embed_tokens` may arrive as an int8 table with one scale per row (`qweight`, `scales`) or as a
dense `weight`.  The int8 form stays int8 in memory: the lookup gathers rows and scales only
those; the tied head streams the int8 rows through a fused kernel instead of dequantising
the whole table on every call.
"""
import torch
from vllm.model_executor.layers.quantization.base_config import QuantizeMethodBase

from . import _ext
from .config import Exl3LinearMethod, Exl3ShardParam

_SLOTS = ("qweight", "scales", "weight")


class Exl3EmbeddingMethod(QuantizeMethodBase):
    """int8 rows with a per-row scale, dequantised on the gathered rows only."""

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes,
                       input_size, output_size, params_dtype, **extra_weight_attrs):
        # either storage form may arrive; extra_weight_attrs (vLLM's vocab-sharding loader) is
        # not applied: it would assert shapes against the empty placeholders
        for name in _SLOTS:
            layer.register_parameter(name, Exl3ShardParam(suffix=name))
        layer.exl3_params_dtype = params_dtype

    def process_weights_after_loading(self, layer):
        q = layer.qweight.shards.get(0)
        s = layer.scales.shards.get(0)
        w = layer.weight.shards.get(0)
        on_gpu = [t.device for t in (q, w) if t is not None and t.device.type == "cuda"]
        dev = on_gpu[0] if on_gpu else torch.device("cuda", torch.cuda.current_device())
        for name in _SLOTS:
            if hasattr(layer, name):
                delattr(layer, name)
        lo, hi = self._vocab_range(layer, (q if q is not None else w))
        if q is None:
            if w is None:
                raise RuntimeError("embed_tokens: neither an int8 table nor a dense one loaded")
            layer.exl3_embed_q = None
            layer.exl3_embed = torch.nn.Parameter(w[lo:hi].to(dev), requires_grad=False)
            return
        if s is None:
            raise RuntimeError("embed_tokens: qweight without scales")
        layer.exl3_embed = None
        layer.exl3_embed_q = torch.nn.Parameter(q[lo:hi].contiguous().to(dev), requires_grad=False)
        layer.exl3_embed_s = torch.nn.Parameter(
            s.reshape(-1)[lo:hi].to(dev, layer.exl3_params_dtype).reshape(-1, 1).contiguous(),
            requires_grad=False)

    @staticmethod
    def _vocab_range(layer, table):
        """Rows of the table this rank keeps (vocab-parallel sharding); everything at TP 1."""
        n = 0 if table is None else table.shape[0]
        si = getattr(layer, "shard_indices", None)
        if si is None or getattr(layer, "tp_size", 1) == 1:
            return 0, n
        return min(si.org_vocab_start_index, n), min(si.org_vocab_end_index, n)

    def embedding(self, layer, input_: torch.Tensor) -> torch.Tensor:
        if layer.exl3_embed_q is None:
            return layer.exl3_embed[input_]
        return torch.ops.orcasaq2.int8_embed(layer.exl3_embed_q, layer.exl3_embed_s, input_)

    def apply(self, layer, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if layer.exl3_embed_q is None:
            out = torch.nn.functional.linear(x, layer.exl3_embed.to(x.dtype))
        else:
            rows = x.numel() // x.shape[-1]
            x2 = x.reshape(rows, x.shape[-1])
            if x2.dtype not in (torch.float16, torch.bfloat16):
                x2 = x2.to(layer.exl3_embed_s.dtype)
            out = torch.ops.orcasaq2.int8_head(layer.exl3_embed_q, layer.exl3_embed_s, x2.contiguous()).to(x.dtype)
            out = out.reshape(*x.shape[:-1], out.shape[-1])
        return out + bias if bias is not None else out


class Exl3LMHeadMethod(Exl3LinearMethod):
    """An untied output head (`ParallelLMHead`) in any of the three storage forms a pack may use for it: an EXL3
    trellis, a dense `weight`, or -- what the reference cannot load -- an int8 table with per-row scales.

    The reference hands every `ParallelLMHead` to `Exl3LinearMethod` (orcasaq2/config.py:128-132), which registers
    no `qweight` / `scales` (config.py:183), so `lm_head.qweight` has nowhere to go and an int8 head only works
    tied to the embedding (heads.py:69-75).  This method registers the int8 placeholders beside the linear ones and
    serves the int8 form with the same kernel as the tied head; the other two forms are `Exl3LinearMethod`'s."""

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes,
                       input_size, output_size, params_dtype, **extra_weight_attrs):
        super().create_weights(layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                               params_dtype, **extra_weight_attrs)
        for name in ("qweight", "scales"):
            layer.register_parameter(name, Exl3ShardParam(suffix=name))
        layer.exl3_params_dtype = params_dtype

    def process_weights_after_loading(self, layer):
        q = layer.qweight.shards.get(0)
        s = layer.scales.shards.get(0)
        for name in ("qweight", "scales"):
            if hasattr(layer, name):
                delattr(layer, name)
        layer.exl3_embed_q = None
        if q is None:
            if s is not None:
                raise RuntimeError(f"{self.prefix}: scales without qweight")
            return super().process_weights_after_loading(layer)
        if s is None:
            raise RuntimeError(f"{self.prefix}: qweight without scales")
        if layer.trellis.shards or layer.weight.shards:
            raise RuntimeError(f"{self.prefix}: an int8 table and another form of the same head were loaded")
        for name in ("trellis", "suh", "svh", "mcg", "mul1", "weight"):
            if hasattr(layer, name):
                delattr(layer, name)
        layer.exl3_shards, layer.exl3_dense = None, None
        dev = q.device if q.device.type == "cuda" else torch.device("cuda", torch.cuda.current_device())
        lo, hi = Exl3EmbeddingMethod._vocab_range(layer, q)
        layer.exl3_embed_q = torch.nn.Parameter(q[lo:hi].contiguous().to(dev), requires_grad=False)
        layer.exl3_embed_s = torch.nn.Parameter(
            s.reshape(-1)[lo:hi].to(dev, layer.exl3_params_dtype).reshape(-1, 1).contiguous(), requires_grad=False)

    def apply(self, layer, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if getattr(layer, "exl3_embed_q", None) is None:
            return super().apply(layer, x, bias)
        rows = x.numel() // x.shape[-1]
        x2 = x.reshape(rows, x.shape[-1])
        if x2.dtype not in (torch.float16, torch.bfloat16):
            x2 = x2.to(layer.exl3_embed_s.dtype)
        out = torch.ops.orcasaq2.int8_head(layer.exl3_embed_q, layer.exl3_embed_s, x2.contiguous()).to(x.dtype)
        out = out.reshape(*x.shape[:-1], out.shape[-1])
        return out + bias if bias is not None else out
