"""A vLLM ENGINE on the synthetic EXL3 checkpoint: `LLM(model=..., quantization="exl3")` with the plugin registered
the way vLLM registers it, vLLM's own loader, scheduler, KV cache and attention backend around this library's
kernels, greedy generation from token ids.  The engine runs in a child process (its process-wide state and its share
of GPU memory go away with it); the parent compares what it returned with an oracle forward pass of the same
checkpoint (CPU oracle's trellis decode, float64 layer algebra and attention with the fp16 roundings of the real
chain): the first generated token, and the log-probabilities the engine reports for its top candidates at the first
and at the second generated position (the second one exercises decode against vLLM's own KV cache).  Both with
`enforce_eager` and in vLLM's default mode (torch.compile + CUDA graphs), in which the reference says its own
plugin must run (orcasaq2/ops.py:3-16, presets/16gb.env:21).

The reference is served exactly like this (`vllm serve` + `quant_method: "exl3"`, reference README.md, presets/*.env);
it ships no test of it."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu

DIMS = dict(layers=2, hidden=256, ffn=384, q_heads=2, kv_heads=1, head_dim=128, vocab=512)
SEED = 33
PROMPTS = [[3, 17, 200, 45, 9, 511, 77], [5, 5, 300]]
ROPE_THETA = 10000.0

_CHILD = r"""
import json, os, sys
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"            # engine core in this process: no plugin discovery needed
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
sys.path.insert(0, sys.argv[1])
import orcasaq2
from orcasaq2 import checkpoint as C
dims, seed, prompts, path = json.loads(sys.argv[2]), int(sys.argv[3]), json.loads(sys.argv[4]), sys.argv[5]
eager = sys.argv[6] == "eager"
C.write_synthetic_checkpoint(path, seed=seed, **dims)
orcasaq2.register()
from vllm import LLM, SamplingParams
extra = {} if eager else {"compilation_config": {"cudagraph_capture_sizes": [1, 2, 4]}}
llm = LLM(model=path, skip_tokenizer_init=True, quantization="exl3", dtype="float16", enforce_eager=eager,
          max_model_len=128, gpu_memory_utilization=0.08, max_num_seqs=4, enable_prefix_caching=False, **extra)
sp = SamplingParams(max_tokens=3, temperature=0.0, logprobs=5, detokenize=False)
outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp)
res = []
for o in outs:
    c = o.outputs[0]
    res.append({"prompt": list(o.prompt_token_ids), "tokens": [int(t) for t in c.token_ids],
                "logprobs": [{str(int(k)): float(v.logprob) for k, v in d.items()} for d in c.logprobs]})
print("ENGINE_RESULT " + json.dumps(res), flush=True)
"""


def _f16(a):
    return np.asarray(a, np.float64).astype(np.float32).astype(np.float16).astype(np.float64)


def _rms(h, w=None, eps=1e-6):
    y = h * (1.0 / np.sqrt((h * h).mean(-1, keepdims=True) + eps))
    return _f16(y if w is None else y * w)


def _oracle_logprobs(co, tensors, ids):
    """log-softmax of the logits at the LAST position of the token sequence `ids` (Qwen3 decoder: RMSNorm, fused
    qkv, per-head q/k RMSNorm with unit weight, rotate-half rotary, causal grouped-query attention, SiLU MLP, tied
    int8 head)."""
    d = DIMS
    hd, qh, kvh = d["head_dim"], d["q_heads"], d["kv_heads"]
    T = len(ids)
    f = lambda name: tensors[name].float().numpy().astype(np.float64)        # noqa: E731

    def lin(x, module):
        w = co.reconstruct(tensors[module + ".trellis"].numpy())
        return _f16(R.layer_np(x.astype(np.float16), w, tensors[module + ".suh"].numpy(), tensors[module + ".svh"].numpy()))

    q8, sc = tensors["model.embed_tokens.qweight"].numpy().astype(np.float64), f("model.embed_tokens.scales")
    h = _f16(q8[ids] * sc[ids][:, None])
    half = hd // 2
    inv = ROPE_THETA ** (-np.arange(half, dtype=np.float64) / half)
    ang = np.arange(T, dtype=np.float64)[:, None] * inv[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

    def rope(t):                                                             # [T, heads, hd]
        a, b = t[..., :half], t[..., half:]
        return _f16(np.concatenate([a * cos - b * sin, b * cos + a * sin], -1))

    for li in range(d["layers"]):
        pre = f"model.layers.{li}."
        x = _rms(h, f(pre + "input_layernorm.weight"))
        q = lin(x, pre + "self_attn.q_proj").reshape(T, qh, hd)
        k = lin(x, pre + "self_attn.k_proj").reshape(T, kvh, hd)
        v = lin(x, pre + "self_attn.v_proj").reshape(T, kvh, hd)
        q, k = rope(_rms(q)), rope(_rms(k))
        att = np.zeros((T, qh, hd))
        for hq in range(qh):
            hk = hq // (qh // kvh)
            s = (q[:, hq] @ k[:, hk].T) * hd ** -0.5
            s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
            p = np.exp(s - s.max(-1, keepdims=True))
            att[:, hq] = (p / p.sum(-1, keepdims=True)) @ v[:, hk]
        h = _f16(h + lin(_f16(att).reshape(T, qh * hd), pre + "self_attn.o_proj"))
        x = _rms(h, f(pre + "post_attention_layernorm.weight"))
        g, u = lin(x, pre + "mlp.gate_proj"), lin(x, pre + "mlp.up_proj")
        h = _f16(h + lin(_f16(g / (1.0 + np.exp(-g)) * u), pre + "mlp.down_proj"))
    x = _rms(h[-1:], f("model.norm.weight"))
    logits = (x @ q8.T) * sc[None, :]
    z = logits[0] - logits[0].max()
    return z - np.log(np.exp(z).sum()), logits[0]


@pytest.fixture(scope="module", params=["eager", "compiled"])
def engine_result(request, ext, tmp_path_factory):
    """`eager`: enforce_eager.  `compiled`: vLLM's default serving mode, the model's forward compiled with
    torch.compile (the plugin's kernels are opaque custom ops in it: orcasaq2::layer_gemm, ::int8_embed) and replayed
    from CUDA graphs (piecewise for prefill, full for decode)."""
    tmp = tmp_path_factory.mktemp("engine_" + request.param)
    script = tmp / "child.py"
    script.write_text(_CHILD)
    pkg = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "orcasaq2-kernel_b200")
    try:
        p = subprocess.run([sys.executable, str(script), pkg, json.dumps(DIMS), str(SEED), json.dumps(PROMPTS),
                            str(tmp / "ckpt"), request.param], capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        pytest.skip("the vLLM engine did not come up within 15 minutes on this machine")
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("ENGINE_RESULT ")]
    if not line:
        pytest.skip("the vLLM engine could not be started here: " + (p.stderr or p.stdout)[-600:])
    return json.loads(line[-1][len("ENGINE_RESULT "):])


def test_engine_generates_what_the_oracle_predicts(engine_result, coracle):
    from orcasaq2 import checkpoint as C
    tensors, _ = C.synthetic_tensors(seed=SEED, **DIMS)
    assert [r["prompt"] for r in engine_result] == PROMPTS
    for r in engine_result:
        assert len(r["tokens"]) == 3 and all(0 <= t < DIMS["vocab"] for t in r["tokens"])
        seq = list(r["prompt"])
        for step in range(2):                                       # prefill, then one decode step on the engine's own token
            ref, logits = _oracle_logprobs(coracle, tensors, seq)
            got = {int(k): v for k, v in r["logprobs"][step].items()}
            tol = 3e-2 * (logits.max() - logits.min())              # two layers of fp16 roundings against the logit spread
            if step == 0:
                assert r["tokens"][0] == int(np.argmax(ref)), (r["tokens"][0], int(np.argmax(ref)))
            assert r["tokens"][step] in got
            for tok, lp in got.items():
                assert abs(lp - ref[tok]) <= tol, (step, tok, lp, ref[tok], tol)
            # the engine's greedy choice is (within that tolerance) the oracle's best
            assert ref[r["tokens"][step]] >= ref.max() - tol
            seq.append(r["tokens"][step])
