"""Per-kernel timings of libexl3_b200.so on the current GPU (CUDA events, inputs rotated past L2).

    python kernel_bench.py gemv --ic 5120 --oc 17408 --k 4 --rows 1
    python kernel_bench.py gemm_tc --ic 5120 --oc 17408 --k 3 --rows 512
    python kernel_bench.py reconstruct --ic 4096 --oc 4096 --k 4
    python kernel_bench.py int8_head --rows 1 [--vocab 151936 --hidden 5120 --bf16]
    python kernel_bench.py int8_embed --rows 4096
    python kernel_bench.py had --rows 8192 --ic 5120
    python kernel_bench.py attn --rows 32 --ctx 4096 [--qh 24 --kvh 4 --sdpa --page 16]   # decode attention, rows = batch
    python kernel_bench.py prefill        # BASELINE config 3: both shapes, M = 512 / 2048 / 8192
    python kernel_bench.py shards         # BASELINE configs 1 and 2: every shard, rows 1 / 4 / 16
    python kernel_bench.py decode_rate    # ceiling of the 3INST decode + mma.sync on this GPU, per bitrate (no HBM involved)

Each line reports the kernel's algorithmic bytes (or flops) per second.  `--iters N` launches
(default 20) after 3 warm-ups; small cases (`--iters 3`) are what the ncu recipes use.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

from orcasaq2 import _ext  # noqa: E402

DEV = None


GRAPH = False


def timeit(fn, iters, warm=3, period=1):
    """Seconds per call.  With --graph, `period` consecutive calls (one pass over the rotated
    buffers) are captured into a CUDA graph and replayed, which removes the host launch cost."""
    if GRAPH:
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            for i in range(max(warm, period)):
                fn(i)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(period):
                    fn(i)
            reps = max(2, iters // period)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / (reps * period) * 1e-3
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def shard(ic, oc, K):
    tr = torch.randint(-32768, 32768, (ic // 16, oc // 16, 16 * K), dtype=torch.int16, device=DEV)
    suh = (torch.randint(0, 2, (ic,), device=DEV) * 2 - 1).half()
    svh = (torch.randint(0, 2, (oc,), device=DEV) * 2 - 1).half()
    return dict(trellis=tr, suh=suh, svh=svh, mcg=False, mul1=False)


def sets_for(ic, spec, min_bytes=400e6, max_sets=12):
    per = sum(ic * oc * K // 8 for oc, K in spec)
    n = int(min(max_sets, max(2, min_bytes // per + 1)))
    return [[shard(ic, oc, K) for oc, K in spec] for _ in range(n)], per


def bench_gemv(ic, spec, rows, iters):
    sets, per = sets_for(ic, spec)
    x = torch.randn(rows, ic, device=DEV).half()
    y = torch.empty(rows, sum(oc for oc, _ in spec), dtype=torch.half, device=DEV)
    t = timeit(lambda i: _ext.gemv_grouped(x, sets[i % len(sets)], y), max(iters, 2 * len(sets)), period=len(sets))
    b = per + rows * ic * 2 + y.numel() * 2
    return dict(kernel="gemv", ic=ic, shards=spec, rows=rows, us=round(t * 1e6, 1), GBs=round(b / t / 1e9, 1),
                pct_of_8TBs=round(b / t / 8e12 * 100, 1), status=_ext.workspace_status(DEV))


def bench_gemm_tc(ic, oc, K, rows, iters):
    s = shard(ic, oc, K)
    x = torch.randn(rows, ic, device=DEV).to(torch.bfloat16)
    y = torch.empty(rows, oc, dtype=torch.half, device=DEV)
    t = timeit(lambda i: _ext.gemm_tc(x, s["trellis"], y, s["suh"], s["svh"]), iters)

    def dense(i):
        xf = x.half()
        xh = torch.empty_like(xf)
        _ext.had_r_128(xf, xh, s["suh"], None, 1.0)
        w = torch.empty(ic, oc, dtype=torch.half, device=DEV)
        _ext.reconstruct(w, s["trellis"], K, False, False)
        _ext.hgemm_recon(xh, w, y)
        _ext.had_r_128(y, y, None, s["svh"], 1.0)
    td = timeit(dense, iters)
    fl = 2.0 * rows * ic * oc
    return dict(kernel="gemm_tc", ic=ic, oc=oc, K=K, rows=rows, us=round(t * 1e6, 1), TFLOPS=round(fl / t / 1e12, 1),
                reconstruct_plus_library_gemm_us=round(td * 1e6, 1), reconstruct_plus_library_gemm_TFLOPS=round(fl / td / 1e12, 1),
                status=_ext.gemm_tc_status())


def bench_reconstruct(ic, oc, K, iters):
    s = shard(ic, oc, K)
    w = torch.empty(ic, oc, dtype=torch.half, device=DEV)
    t = timeit(lambda i: _ext.reconstruct(w, s["trellis"], K, False, False), iters)
    b = ic * oc * (K / 8 + 2)
    return dict(kernel="reconstruct", ic=ic, oc=oc, K=K, us=round(t * 1e6, 1), GBs=round(b / t / 1e9, 1))


def bench_int8_head(vocab, hidden, rows, bf16, iters):
    dt = torch.bfloat16 if bf16 else torch.float16
    q = torch.randint(-127, 128, (vocab, hidden), dtype=torch.int8, device=DEV)
    s = (torch.rand(vocab, device=DEV) * 0.02 + 1e-3).to(dt)
    x = torch.randn(rows, hidden, device=DEV).to(dt)
    t = timeit(lambda i: _ext.int8_head(q, s, x), iters)
    b = vocab * hidden + vocab * 2 + rows * hidden * 2 + rows * vocab * 2
    return dict(kernel="int8_head", vocab=vocab, hidden=hidden, rows=rows, dtype=str(dt), us=round(t * 1e6, 1),
                GBs=round(b / t / 1e9, 1))


def bench_int8_embed(vocab, hidden, tokens, bf16, iters):
    dt = torch.bfloat16 if bf16 else torch.float16
    q = torch.randint(-127, 128, (vocab, hidden), dtype=torch.int8, device=DEV)
    s = (torch.rand(vocab, device=DEV) * 0.02 + 1e-3).to(dt)
    ids = torch.randint(0, vocab, (tokens,), device=DEV)
    t = timeit(lambda i: _ext.int8_embed(q, s, ids), iters)
    b = tokens * (hidden + 2 + 2 * hidden)
    return dict(kernel="int8_embed", tokens=tokens, us=round(t * 1e6, 1), GBs=round(b / t / 1e9, 1))


def bench_had(rows, n, iters):
    x = torch.randn(rows, n, device=DEV).half()
    o = torch.empty_like(x)
    sv = torch.ones(n, device=DEV).half()
    t = timeit(lambda i: _ext.had_r_128(x, o, sv, None, 1.0), iters)
    return dict(kernel="had_r_128", rows=rows, n=n, us=round(t * 1e6, 1), GBs=round(rows * n * 4 / t / 1e9, 1))


def bench_attn(batch, qh, kvh, ctx, iters, sdpa, page=0, kv="fp16"):
    """Decode attention over `ctx` cached tokens; the caches are rotated so that every launch reads HBM."""
    esize = 1 if kv == "fp8" else 2
    per = 2 * batch * kvh * ctx * 256 * esize
    n = int(min(8, max(2, 400e6 // per + 1)))
    kcs = [torch.randn(batch, kvh, ctx, 256, device=DEV).half() for _ in range(n)]
    vcs = [torch.randn(batch, kvh, ctx, 256, device=DEV).half() for _ in range(n)]
    if kv == "fp8":
        kcs, vcs = [c.to(torch.float8_e4m3fn) for c in kcs], [c.to(torch.float8_e4m3fn) for c in vcs]
    q = torch.randn(batch, qh, 256, device=DEV).half()
    o = torch.empty_like(q)
    t = timeit(lambda i: _ext.decode_attn(q, kcs[i % n], vcs[i % n], ctx, out=o), max(iters, 2 * n), period=n)
    b = per + 2 * q.numel() * 2
    r = dict(kernel="decode_attn", kv=kv, batch=batch, q_heads=qh, kv_heads=kvh, ctx=ctx, us=round(t * 1e6, 1),
             GBs=round(b / t / 1e9, 1))
    if page:
        # the same tokens in page pools [pages, kv_heads, page, 256], pages in shuffled order
        npg = ctx // page
        perm = torch.randperm(batch * npg, device=DEV)
        table = torch.empty(batch * npg, dtype=torch.int32, device=DEV)
        table[perm] = torch.arange(batch * npg, dtype=torch.int32, device=DEV)     # page of (b, i) = table[b * npg + i]
        table = table.view(batch, npg)

        def pool(c):
            c8 = c.view(torch.uint8) if kv == "fp8" else c
            pg = c8.view(batch, kvh, npg, page, 256).permute(0, 2, 1, 3, 4).reshape(batch * npg, kvh, page, 256)
            out = torch.empty_like(pg)
            out[table.view(-1).long()] = pg
            return out.view(c.dtype)
        kps, vps = [pool(c) for c in kcs], [pool(c) for c in vcs]
        tp = timeit(lambda i: _ext.decode_attn_paged(q, kps[i % n], vps[i % n], table, None, npg * page, out=o),
                    max(iters, 2 * n), period=n)
        same = bool(torch.equal(_ext.decode_attn_paged(q, kps[0], vps[0], table, None, npg * page),
                                _ext.decode_attn(q, kcs[0], vcs[0], npg * page)))
        r.update(page=page, paged_us=round(tp * 1e6, 1), paged_GBs=round(b / tp / 1e9, 1), paged_equals_contiguous=same)
    if sdpa and kv == "fp16":
        import torch.nn.functional as F
        ts = timeit(lambda i: F.scaled_dot_product_attention(q.unsqueeze(2), kcs[i % n], vcs[i % n], enable_gqa=True),
                    max(iters, 2 * n), period=n)
        r.update(torch_sdpa_us=round(ts * 1e6, 1), torch_sdpa_GBs=round(b / ts / 1e9, 1))
    return r


def bench_decode_rate(iters=2000):
    """exl3_probe_decode_rate per bitrate: registers only, and through a shared-memory ring fed by bulk copies."""
    import ctypes
    L = _ext.lib()
    L.exl3_probe_decode_rate.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]
    scratch = torch.zeros((2 << 20,), dtype=torch.uint8, device=DEV)
    out = []
    for K in range(1, 9):
        row = dict(kernel="decode_rate", K=K)
        for mode, name in ((0, "registers_only_Tw_s"), (1, "smem_ring_Tw_s")):
            w = ctypes.c_double(0)
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            best = 1e9
            for rep in range(4):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                rc = L.exl3_probe_decode_rate(K, mode, iters, scratch.data_ptr(), scratch.numel(), ctypes.byref(w), st)
                b.record()
                torch.cuda.synchronize()
                assert rc == 0, rc
                if rep:
                    best = min(best, a.elapsed_time(b))
            row[name] = round(w.value / (best * 1e-3) / 1e12, 2)
            row[name.replace("Tw_s", "GBs_at_this_bitrate")] = round(w.value * K / 8 / (best * 1e-3) / 1e9, 0)
        row["status"] = int(scratch[:4].view(torch.int32).item())
        out.append(row)
    return out


def main():
    global DEV
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "gemm_tc", "reconstruct", "int8_head", "int8_embed", "had", "prefill", "shards", "attn", "decode_rate"])
    ap.add_argument("--ic", type=int, default=5120)
    ap.add_argument("--oc", type=int, default=17408)
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--qh", type=int, default=24)
    ap.add_argument("--kvh", type=int, default=4)
    ap.add_argument("--page", type=int, default=0, help="attn: also time the paged form with this page size (divides ctx)")
    ap.add_argument("--kv", choices=["fp16", "fp8"], default="fp16", help="attn: cache element type")
    ap.add_argument("--sdpa", action="store_true", help="attn: also time torch's scaled_dot_product_attention")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--graph", action="store_true", help="replay the launches from a CUDA graph")
    a = ap.parse_args()
    global GRAPH
    GRAPH = a.graph
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    DEV = torch.device("cuda", 0)
    _ext.lib()
    out = []
    if a.what == "gemv":
        out.append(bench_gemv(a.ic, [(a.oc, a.k)], a.rows, a.iters))
    elif a.what == "gemm_tc":
        out.append(bench_gemm_tc(a.ic, a.oc, a.k, a.rows, a.iters))
    elif a.what == "reconstruct":
        out.append(bench_reconstruct(a.ic, a.oc, a.k, a.iters))
    elif a.what == "int8_head":
        out.append(bench_int8_head(a.vocab, a.hidden, a.rows, a.bf16, a.iters))
    elif a.what == "int8_embed":
        out.append(bench_int8_embed(a.vocab, a.hidden, a.rows, a.bf16, a.iters))
    elif a.what == "had":
        out.append(bench_had(a.rows, a.ic, a.iters))
    elif a.what == "attn":
        out.append(bench_attn(a.rows, a.qh, a.kvh, a.ctx, a.iters, a.sdpa, a.page, a.kv))
    elif a.what == "decode_rate":
        out.extend(bench_decode_rate())
    elif a.what == "prefill":
        for ic, oc, K in ((5120, 17408, 3), (17408, 5120, 4)):
            for m in (512, 2048, 8192):
                out.append(bench_gemm_tc(ic, oc, K, m, max(3, a.iters // 4)))
    elif a.what == "shards":
        cases = [("cfg1 4096x4096", 4096, [(4096, 4)]), ("q", 5120, [(6144, 4)]), ("k", 5120, [(1024, 5)]),
                 ("v", 5120, [(1024, 6)]), ("qkv fused", 5120, [(6144, 4), (1024, 5), (1024, 6)]),
                 ("gate", 5120, [(17408, 3)]), ("gate_up fused", 5120, [(17408, 3), (17408, 3)]),
                 ("down", 17408, [(5120, 4)])]
        for rows in (1, 4, 16):
            for name, ic, spec in cases:
                r = bench_gemv(ic, spec, rows, a.iters)
                r["name"] = name
                out.append(r)
    for r in out:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
