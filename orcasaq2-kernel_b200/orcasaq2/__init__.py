"""orcasaq2 on B200: the EXL3 trellis-quantized linear layer for vLLM, with its own sm_100a
kernels in place of the exllamav3 extension.

Same surface as the reference plugin's package (`register`, `reconstruct_weight`, `BLOCK`,
`_had`, `_t128`; reference orcasaq2/__init__.py:29-153), so a deployment switches by
installing this package instead.  What differs underneath:

  * every extension call lands in `orcasaq2._ext`, a ctypes binding of libexl3_b200.so
    (fused trellis-decode GEMV, Hadamard, reconstruct, int8 embedding / head kernels);
  * fused layers (qkv_proj, gate_up_proj) run all their shards in one launch and write straight
    into the concatenated output;
  * tensor parallelism is implemented (128-aligned column / row slices of each shard) where
    the reference raises.

Importing this module does not import vLLM; `register()` does.
"""
import torch

BLOCK = 128
_HAD: dict = {}


def _had(device, dtype):
    """Sylvester-ordered Hadamard matrix of size BLOCK, scaled to be orthogonal
    (reference orcasaq2/__init__.py:33-40), cached per device and dtype."""
    key = (str(device), dtype)
    m = _HAD.get(key)
    if m is None:
        idx = torch.arange(BLOCK)
        # H[a, b] = (-1)^popcount(a & b)
        bits = idx[:, None] & idx[None, :]
        pop = torch.zeros_like(bits)
        for s in range(BLOCK.bit_length() - 1):
            pop += (bits >> s) & 1
        m = (1.0 - 2.0 * (pop & 1).double()) / BLOCK ** 0.5
        m = m.to(device=device, dtype=dtype)
        _HAD[key] = m
    return m


def _t128(x):
    """Blockwise size-128 Hadamard along the last dim (reference orcasaq2/__init__.py:43-46)."""
    shape = x.shape
    blocks = x.reshape(*shape[:-1], shape[-1] // BLOCK, BLOCK)
    return (blocks @ _had(x.device, x.dtype)).reshape(shape)


def reconstruct_weight(trellis, suh, svh, mcg, mul1):
    """Deploy weight [oc, ic] in fp16:  (diag(suh) H W H diag(svh))^T, where W is the decoded
    inner weight (reference orcasaq2/__init__.py:49-61).  `mcg` / `mul1` are the checkpoint's
    flag tensors or None."""
    from . import _ext
    from .ops import exl3_K

    ic, oc = suh.numel(), svh.numel()
    inner = torch.empty((ic, oc), dtype=torch.half, device=trellis.device)
    _ext.reconstruct(inner, trellis, exl3_K(trellis), mcg is not None, mul1 is not None)
    w = inner.float()
    w = _t128(w.t()).t() * suh.float()[:, None]      # rotate and sign the input side
    w = _t128(w) * svh.float()[None, :]              # rotate and sign the output side
    return w.t().contiguous().half()


def register():
    """vLLM general-plugin entry point (`vllm.general_plugins`: orcasaq2 = orcasaq2:register).
    Idempotent.  Fails at start-up, not mid-request, when the CUDA library is missing."""
    from vllm.logger import init_logger
    from vllm.model_executor.layers.quantization import register_quantization_config

    log = init_logger("vllm.orcasaq2")
    from . import _ext
    try:
        _ext.lib()
    except Exception as e:                                   # noqa: BLE001
        raise RuntimeError(
            "orcasaq2 needs its CUDA library libexl3_b200.so and could not load it: "
            f"{type(e).__name__}: {e}") from e

    from .config import Exl3Config
    try:
        register_quantization_config("exl3")(Exl3Config)
    except (ValueError, AssertionError):
        return                                               # this process already has it
    _patch_embedding_layers(log)
    log.info("orcasaq2 (B200 kernels) armed: quant_method 'exl3' is loadable")


def _patch_embedding_layers(logger):
    """Let `embed_tokens` and `lm_head` see the EXL3 quant config.

    Model files build VocabParallelEmbedding / ParallelLMHead without passing quant_config, so
    vLLM never asks the config for a method and then looks for dense `.weight` tensors the pack
    does not have.  Both constructors are wrapped to fill an empty quant_config slot from the
    current vLLM config when that config is an Exl3Config (reference
    orcasaq2/__init__.py:97-153)."""
    import functools
    import inspect

    from vllm.model_executor.layers import vocab_parallel_embedding as vpe
    from .config import Exl3Config

    if getattr(vpe.VocabParallelEmbedding, "_orca_patched", False):
        return

    def active_config():
        try:
            from vllm.config import get_current_vllm_config
            cfg = get_current_vllm_config()
        except Exception:                                    # noqa: BLE001
            return None
        qc = getattr(cfg, "quant_config", None)
        if qc is None:
            qc = getattr(getattr(cfg, "model_config", None), "quant_config", None)
        return qc if isinstance(qc, Exl3Config) else None

    def wrap(ctor):
        signature = inspect.signature(ctor)

        @functools.wraps(ctor)
        def init(self, *args, **kwargs):
            # ParallelLMHead hands quant_config to its (also wrapped) parent positionally:
            # bind against the real signature and fill the slot only when it is empty.
            try:
                bound = signature.bind_partial(self, *args, **kwargs)
            except TypeError:
                return ctor(self, *args, **kwargs)
            if bound.arguments.get("quant_config") is None:
                qc = active_config()
                if qc is not None:
                    bound.arguments["quant_config"] = qc
                    return ctor(*bound.args, **bound.kwargs)
            return ctor(self, *args, **kwargs)
        return init

    for cls in (vpe.VocabParallelEmbedding, vpe.ParallelLMHead):
        cls.__init__ = wrap(cls.__init__)
    vpe.VocabParallelEmbedding._orca_patched = True
    logger.info("orcasaq2: embed_tokens / lm_head will receive the EXL3 quant config")
