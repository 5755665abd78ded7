"""`orcasaq2.register()` as vLLM calls it at process start (reference orcasaq2/__init__.py:64-153): the
quantization method becomes loadable, a second call changes nothing, and the wrapped constructors of
VocabParallelEmbedding / ParallelLMHead pick up the EXL3 config that model files do not pass.  Runs in
a child process because it patches vLLM classes for the life of the process.  CPU only."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent('''
    import sys, types
    sys.path.insert(0, sys.argv[1])
    import torch
    import orcasaq2
    orcasaq2.register()
    orcasaq2.register()                                   # idempotent (reference __init__.py:89-92)
    from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, get_quantization_config
    from orcasaq2.config import Exl3Config, Exl3LinearMethod
    from orcasaq2.heads import Exl3EmbeddingMethod
    assert "exl3" in QUANTIZATION_METHODS and get_quantization_config("exl3") is Exl3Config
    from vllm.model_executor.layers import vocab_parallel_embedding as vpe
    assert vpe.VocabParallelEmbedding._orca_patched
    first = vpe.VocabParallelEmbedding.__init__
    orcasaq2._patch_embedding_layers(types.SimpleNamespace(info=lambda *a, **k: None))
    assert vpe.VocabParallelEmbedding.__init__ is first   # not wrapped twice

    # one tensor-parallel rank, no engine: the group lookups the constructors make are answered here
    import vllm.model_executor.parameter as vparam
    for mod in (vpe, vparam):
        mod.get_tensor_model_parallel_rank = lambda: 0
        mod.get_tensor_model_parallel_world_size = lambda: 1
    import vllm.config as vc
    qc = Exl3Config.from_config({})
    vc.get_current_vllm_config = lambda: types.SimpleNamespace(quant_config=qc)
    emb = vpe.VocabParallelEmbedding(512, 128, params_dtype=torch.float16)          # no quant_config passed
    assert isinstance(emb.quant_method, Exl3EmbeddingMethod)
    assert {n for n, _ in emb.named_parameters()} == {"qweight", "scales", "weight"}
    head = vpe.ParallelLMHead(512, 128, params_dtype=torch.float16, prefix="lm_head")
    assert isinstance(head.quant_method, Exl3LinearMethod)
    assert {"trellis", "suh", "svh"} <= {n for n, _ in head.named_parameters()}

    # a model-level config that is not EXL3 leaves the layers as vLLM builds them
    vc.get_current_vllm_config = lambda: types.SimpleNamespace(quant_config=None, model_config=None)
    plain = vpe.VocabParallelEmbedding(512, 128, params_dtype=torch.float16)
    assert not isinstance(plain.quant_method, Exl3EmbeddingMethod) and hasattr(plain, "weight")
    print("REGISTER-OK")
''')


def test_register_and_constructor_patch():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, "-c", SCRIPT, os.path.join(ROOT, "orcasaq2-kernel_b200")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0 and "REGISTER-OK" in p.stdout, (p.stdout[-2000:], p.stderr[-4000:])


def test_package_declares_the_reference_entry_point():
    """vLLM discovers the plugin through the entry-point group the reference declares (its pyproject.toml:19-20)."""
    import tomllib
    with open(os.path.join(ROOT, "orcasaq2-kernel_b200", "pyproject.toml"), "rb") as f:
        meta = tomllib.load(f)
    assert meta["project"]["entry-points"]["vllm.general_plugins"] == {"orcasaq2": "orcasaq2:register"}
    assert "orcasaq2" in meta["tool"]["setuptools"]["packages"]
