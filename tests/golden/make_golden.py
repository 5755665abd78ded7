"""Generate tests/golden/reference_golden.npz by running the REFERENCE plugin's own Python
(imported from its checkout) on CPU.  Run once where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference forwards four calls to the exllamav3 extension, which is not part of its tree.
Those four are supplied here by the CPU oracle through a stand-in module, so the fixtures pin
everything the reference's Python does around them -- Hadamard matrix and `_t128`, the
deploy-weight algebra of `reconstruct_weight`, the order of operations and row-count dispatch of
`orcasaq2::shard_gemm`, `exl3_K`, shard-slot mapping, and the int8 embedding / head math -- but
not the trellis decode itself (no reference artefact pins that).
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import exl3_ref as R  # noqa: E402


def install_fake_extension(calls):
    co = R.COracle()

    def reconstruct(w, trellis, k, mcg, mul1):
        calls.append(("reconstruct", type(k).__name__, float(k), bool(mcg), bool(mul1)))
        w.copy_(torch.from_numpy(co.reconstruct(trellis.numpy())))

    def had_r_128(inp, out, pre, post, scale):
        calls.append(("had_r_128", pre is not None, post is not None, float(scale)))
        res = co.had_r_128(inp.numpy(), None if pre is None else pre.numpy(),
                           None if post is None else post.numpy(), scale)
        out.copy_(torch.from_numpy(res))

    def hgemm_recon(a, w, y):
        calls.append(("hgemm_recon",))
        y.copy_(torch.from_numpy(co.hgemm(a.numpy(), w.numpy())))

    def exl3_gemm(A, trellis, C, suh, A_had, svh, kernel, mcg, mul1, acc_mode):
        calls.append(("exl3_gemm", int(kernel), bool(mcg), bool(mul1), int(acc_mode)))
        w = co.reconstruct(trellis.numpy())
        y = co.layer(A.numpy(), w, suh.numpy(), svh.numpy())
        C.copy_(torch.from_numpy(y).half())

    pkg = types.ModuleType("exllamav3")
    sub = types.ModuleType("exllamav3.ext")
    ext = types.ModuleType("exllamav3.ext.exllamav3_ext")
    ext.reconstruct, ext.had_r_128, ext.hgemm_recon, ext.exl3_gemm = reconstruct, had_r_128, hgemm_recon, exl3_gemm
    pkg.ext, sub.exllamav3_ext = sub, ext
    sys.modules.update({"exllamav3": pkg, "exllamav3.ext": sub, "exllamav3.ext.exllamav3_ext": ext})


def main(ref_root):
    calls = []
    install_fake_extension(calls)
    sys.path.insert(0, ref_root)
    import orcasaq2 as ref                      # the reference package
    from orcasaq2 import ops as ref_ops
    assert os.path.abspath(ref.__file__).startswith(os.path.abspath(ref_root))
    out = {}

    # Hadamard
    h = ref._had("cpu", torch.float64)
    out["had_sign"] = np.sign(h.numpy()).astype(np.int8)
    out["had_scale"] = np.array([abs(h[0, 0].item())])
    g = torch.Generator().manual_seed(11)
    x = torch.randn((5, 384), generator=g, dtype=torch.float64)
    out["t128_in"], out["t128_out"] = x.numpy(), ref._t128(x).numpy()

    # deploy weight
    tr, suh, svh, _ = R.make_layer(21, 256, 384, 3, 1)
    suh = suh * 1.5
    out["dw_trellis"], out["dw_suh"], out["dw_svh"] = tr.numpy(), suh.numpy(), svh.numpy()
    out["dw_out"] = ref.reconstruct_weight(tr, suh, svh, None, None).numpy()

    # exl3_K
    out["k_widths"] = np.array([16, 32, 56, 64, 40, 24], np.int64)
    out["k_values"] = np.array([float(ref_ops.exl3_K(torch.empty((1, 1, int(wd))))) for wd in out["k_widths"]])
    out["k_is_int"] = np.array([isinstance(ref_ops.exl3_K(torch.empty((1, 1, int(wd)))), int) for wd in out["k_widths"]])
    out["gemm_max_rows"] = np.array([ref_ops.GEMM_MAX_ROWS])

    # shard_gemm, both branches of the row-count dispatch
    for tag, rows in (("small", 3), ("large", ref_ops.GEMM_MAX_ROWS + 1)):
        tr, suh, svh, x = R.make_layer(31 + rows, 256, 128, 4, rows)
        calls.clear()
        y = torch.ops.orcasaq2.shard_gemm(x, tr, suh, svh, 128, 4.0, False, False)
        out[f"sg_{tag}_trellis"], out[f"sg_{tag}_suh"], out[f"sg_{tag}_svh"] = tr.numpy(), suh.numpy(), svh.numpy()
        out[f"sg_{tag}_x"], out[f"sg_{tag}_y"] = x.numpy(), y.numpy()
        out[f"sg_{tag}_calls"] = np.array([repr(c) for c in calls])

    # int8 embedding / head (reference heads.py with hand-set layer attributes, CPU)
    from orcasaq2.heads import Exl3EmbeddingMethod
    from orcasaq2.patches.int8_embedding import Int8EmbeddingTable
    for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        q, s = R.make_int8_table(41, 96, 128, dt)
        layer = types.SimpleNamespace(exl3_embed_q=q, exl3_embed_s=s.reshape(-1, 1), exl3_embed=None)
        ids = torch.tensor([[0, 95, 7], [7, 33, 1]])
        m = Exl3EmbeddingMethod()
        emb = m.embedding(layer, ids)
        gx = torch.Generator().manual_seed(43)
        xin = torch.randn((4, 128), generator=gx).to(dt)
        logits = m.apply(layer, xin.float()).float()       # fp32 activations: CPU matmul in fp32
        logits_dt = m.apply(layer, xin)
        tab = Int8EmbeddingTable(q, s, dt)(ids)
        out[f"i8_{name}_q"], out[f"i8_{name}_ids"] = q.numpy(), ids.numpy()
        out[f"i8_{name}_s"] = s.view(torch.int16).numpy()
        out[f"i8_{name}_emb"] = emb.view(torch.int16).numpy()
        out[f"i8_{name}_tab"] = tab.view(torch.int16).numpy()
        out[f"i8_{name}_x"] = xin.view(torch.int16).numpy()
        out[f"i8_{name}_logits32"] = logits.numpy()
        out[f"i8_{name}_logits"] = logits_dt.view(torch.int16).numpy()

    # shard-slot mapping (needs a TP group: patch the rank lookup the parameter base class uses)
    import vllm.model_executor.parameter as vp
    vp.get_tensor_model_parallel_rank = lambda: 0
    vp.get_tensor_model_parallel_world_size = lambda: 1
    from orcasaq2.config import SHARD_IDS, Exl3ShardParam
    p = Exl3ShardParam(suffix="trellis")
    probes = [None, 0, 1, 3, (0, 1, 2), (2, 3), "q", "k", "v"]
    out["slot_probes"] = np.array([repr(s) for s in probes])
    out["slot_values"] = np.array([p.slot(s) for s in probes])
    out["shard_ids"] = np.array([repr(SHARD_IDS)])

    path = os.path.join(HERE, "reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of the reference plugin>")
    main(sys.argv[1])
