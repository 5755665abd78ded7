"""Decode benchmark of a random-init 27B-class decoder whose every projection is an EXL3 layer
(BASELINE.json configs 4 and 5), on the kernels of this repository.

    python bench_model.py --batch 1 --ctx 4096                       # 1 GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench_model.py --batch 64 --ctx 8192                         # tensor parallel

Model: 64 layers, hidden 5120, FFN 17408, 24 query / 4 KV heads of 256, vocabulary 151936; each
projection (q, k, v, o, gate, up, down) gets a seeded bitrate from {2,..,6}; embed_tokens and the
tied lm_head are one int8 table with per-row scales.  Weights are random (no checkpoint is
involved); the KV cache is filled with random values for `ctx` tokens.  One step = one decoded
token per sequence: RMSNorm, fused qkv GEMV, rotary, attention over the cache (exl3_decode_attn; --attn sdpa for torch's), o_proj,
RMSNorm, fused gate_up GEMV, SiLU*up, down_proj, final norm, int8 head, argmax.  The whole step is
captured in a CUDA graph.  Under tensor parallelism qkv / gate_up are column-sliced, o_proj /
down_proj row-sliced with an all-reduce after each (this library's one-shot kernel over peer memory;
--allreduce nccl for the library collective), the head is vocabulary-sliced.

Prints one JSON line: tokens/s, ms per step, bytes moved per step (packed weights + KV cache) and
their share of the measured HBM bandwidth.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "orcasaq2-kernel_b200"))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402

HIDDEN, FFN, LAYERS, QH, KVH, HD, VOCAB = 5120, 17408, 64, 24, 4, 256, 151936
DIMS_27B = dict(hidden=HIDDEN, ffn=FFN, qh=QH, kvh=KVH, hd=HD, vocab=VOCAB)
TC_FROM_ROWS = 9           # batch sizes from here on take the tcgen05 path (--tc-from; measured faster from 9 rows)


def rand_shard(ic, oc, K, dev, gen):
    tr = torch.randint(-32768, 32768, (ic // 16, oc // 16, 16 * K), dtype=torch.int16, device=dev, generator=gen)
    suh = (torch.randint(0, 2, (ic,), device=dev, generator=gen) * 2 - 1).half()
    svh = (torch.randint(0, 2, (oc,), device=dev, generator=gen) * 2 - 1).half()
    return dict(trellis=tr, suh=suh, svh=svh, mcg=False, mul1=False, K=K, ic=ic, oc=oc)


class Linear:
    """One (possibly fused) EXL3 layer on this rank: list of shards + preallocated output."""

    def __init__(self, shards, rows, dev):
        from orcasaq2 import _ext
        self.ext, self.shards = _ext, shards
        col = 0
        for s in shards:
            s["out_col"] = col
            col += s["oc"]
        self.out = torch.empty((rows, col), dtype=torch.half, device=dev)
        self.rows = rows
        self.bytes = sum(s["ic"] * s["oc"] * s["K"] // 8 for s in shards)

    def __call__(self, x, in_mode=0, residual=None, out=None):
        """in_mode: 0 plain, 1 RMSNorm(x), 2 silu(x[:, :ic]) * x[:, ic:]; `residual` is added to the
        result (fused into the GEMV for <= 16 rows, into the pre- and post-pass of the tcgen05 path above)."""
        # fused layers stay on the grouped GEMV up to 16 rows (measured faster there), single shards switch earlier
        if self.rows < TC_FROM_ROWS or (len(self.shards) > 1 and self.rows <= self.ext.GEMV_MAX_ROWS):
            out = self.out if out is None else out
            self.ext.gemv_grouped(x, self.shards, out, in_mode=in_mode, residual=residual)
            return out
        # many rows: the tcgen05 path, shard by shard, each writing its column block; the norm / gated
        # activation rides in its activation pre-pass, the residual add in its post-pass
        out = self.out if out is None else out
        if self.ext.gemm_tc_grouped(x, self.shards, out, in_mode=in_mode, residual=residual):
            return out                                  # one grouped launch (up to 128 rows)
        if self.rows <= self.ext.GEMV_MAX_ROWS:
            self.ext.gemv_grouped(x, self.shards, out, in_mode=in_mode, residual=residual)
            return out
        for s in self.shards:
            c0 = s["out_col"]
            self.ext.gemm_tc(x, s["trellis"], out[:, c0:c0 + s["oc"]], s["suh"], s["svh"], in_mode=in_mode,
                             residual=None if residual is None else residual[:, c0:c0 + s["oc"]])
        return out


def rms(x, eps=1e-6):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).half()


def build(rank, world, batch, ctx, dev, layers, dims=None, kv="fp16"):
    """Random-init decoder of `layers` layers on this rank: [(qkv, o, gate_up, down, k_cache, v_cache)], the int8
    table and its scales, bytes of packed weights and of KV cache read per step, and the local head counts."""
    d = dims or DIMS_27B
    HIDDEN, FFN, QH, KVH, HD, VOCAB = d["hidden"], d["ffn"], d["qh"], d["kvh"], d["hd"], d["vocab"]
    kgen = torch.Generator().manual_seed(2026)                        # bitrates: same on every rank
    wgen = torch.Generator(device=dev).manual_seed(1234 + rank)
    qh, kvh = QH // world, max(1, KVH // world)
    model, wbytes, kvbytes = [], 0, 0
    for _ in range(layers):
        ks = torch.randint(2, 7, (7,), generator=kgen).tolist()       # q k v o gate up down
        qkv = Linear([rand_shard(HIDDEN, qh * HD, ks[0], dev, wgen), rand_shard(HIDDEN, kvh * HD, ks[1], dev, wgen),
                      rand_shard(HIDDEN, kvh * HD, ks[2], dev, wgen)], batch, dev)
        o = Linear([rand_shard(qh * HD, HIDDEN, ks[3], dev, wgen)], batch, dev)
        gu = Linear([rand_shard(HIDDEN, FFN // world, ks[4], dev, wgen), rand_shard(HIDDEN, FFN // world, ks[5], dev, wgen)], batch, dev)
        down = Linear([rand_shard(FFN // world, HIDDEN, ks[6], dev, wgen)], batch, dev)
        kc = torch.randn((batch, kvh, ctx + 1, HD), device=dev, generator=wgen).half()
        vc = torch.randn((batch, kvh, ctx + 1, HD), device=dev, generator=wgen).half()
        if kv == "fp8":                                               # e4m3 bytes, scale 1 (the engine's default)
            kc, vc = kc.to(torch.float8_e4m3fn), vc.to(torch.float8_e4m3fn)
        model.append((qkv, o, gu, down, kc, vc))
        wbytes += qkv.bytes + o.bytes + gu.bytes + down.bytes
        kvbytes += 2 * batch * kvh * ctx * HD * kc.element_size()
    vslice = VOCAB // world
    table = torch.randint(-127, 128, (vslice, HIDDEN), dtype=torch.int8, device=dev, generator=wgen)
    scales = (torch.rand((vslice,), device=dev, generator=wgen) * 0.02 + 1e-3).half()
    return model, table, scales, wbytes + vslice * HIDDEN, kvbytes, qh, kvh


def default_args(**over):
    """The command-line defaults as a namespace (for callers that run the benchmark in-process)."""
    ns = argparse.Namespace(batch=1, ctx=4096, steps=20, warmup=3, layers=LAYERS, no_graph=False, attn="own", tc_from=9,
                            allreduce="oneshot", kv="fp16")
    for k, v in over.items():
        setattr(ns, k, v)
    return ns


def make_step(model, table, scales, ids, B, ctx, qh, kvh, world, attn="own", dims=None, all_reduce=None):
    """One decode step over `model` as a closure: returns (argmax token per sequence, logits of this rank's
    vocabulary slice).  The new token's key and value go to cache position `ctx`."""
    from orcasaq2 import _ext
    HD = (dims or DIMS_27B)["hd"]
    dev = table.device
    if all_reduce is None:
        all_reduce = dist.all_reduce
    pos = torch.arange(HD // 2, device=dev).float()
    ang = ctx / (10000.0 ** (pos / (HD // 2)))
    cos, sin = torch.cos(ang).half(), torch.sin(ang).half()
    cs, sn = torch.cat([cos, cos]), torch.cat([-sin, sin])

    def rope(t):                                    # [B, heads, HD], rotate-half form in three kernels
        return torch.addcmul(t * cs, torch.roll(t, HD // 2, -1), sn)

    def step():
        h = _ext.int8_embed(table, scales, ids)                           # [B, HIDDEN] (rank-local rows)
        if world > 1:
            all_reduce(h)                                                 # vocabulary-parallel embedding
        for qkv, o, gu, down, kc, vc in model:
            y = qkv(h, in_mode=1)
            if attn == "sdpa":
                qk = rope(y[:, :(qh + kvh) * HD].reshape(B, qh + kvh, HD))    # query and key heads in one pass
                q, k = qk[:, :qh], qk[:, qh:]
                v = y[:, (qh + kvh) * HD:].reshape(B, kvh, HD)
                kc[:, :, ctx] = k
                vc[:, :, ctx] = v
                att = F.scaled_dot_product_attention(q.unsqueeze(2), kc, vc, enable_gqa=True)   # [B, qh, 1, HD]
            else:
                _ext.rope_append(y, cos, sin, kc, vc, ctx, qh)            # rotary + cache append, one launch
                q = torch.as_strided(y, (B, qh, HD), (y.stride(0), HD, 1))
                att = _ext.decode_attn(q, kc, vc, ctx + 1)                # [B, qh, HD], split-KV kernel of this library
            if world > 1:
                a = o(att.reshape(B, qh * HD))
                all_reduce(a)
                h = h + a
            else:
                h = o(att.reshape(B, qh * HD), residual=h)           # residual add in the epilogue
            g = gu(h, in_mode=1)
            if world > 1:
                d = down(g, in_mode=2)
                all_reduce(d)
                h = h + d
            else:
                h = down(g, in_mode=2, residual=h)
        logits = _ext.int8_head(table, scales, rms(h))                    # vocabulary slice of this rank
        return logits.argmax(-1), logits

    return step


def run(args):
    """Build the decoder on this rank, time `args.steps` decode steps, and return the result line as a dict on
    rank 0 (None elsewhere).  Joins the process group that is there, or creates one when launched multi-rank
    without one."""
    global TC_FROM_ROWS
    TC_FROM_ROWS = max(9, min(17, args.tc_from))
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    from orcasaq2 import _ext
    _ext.lib()
    B, ctx = args.batch, args.ctx
    kv = getattr(args, "kv", "fp16")
    if kv == "fp8" and args.attn != "own":
        raise SystemExit("--kv fp8 needs this library's attention kernel (--attn own)")
    model, table, scales, wbytes, kvbytes, qh, kvh = build(rank, world, B, ctx, dev, args.layers, kv=kv)
    ids = torch.randint(0, table.shape[0], (B,), device=dev)
    ar = None
    if world > 1 and getattr(args, "allreduce", "oneshot") == "oneshot":
        from orcasaq2 import comm
        ar = comm.OneShotAllReduce(max_values=max(64, B) * HIDDEN, device=dev)
    step = make_step(model, table, scales, ids, B, ctx, qh, kvh, world, args.attn,
                     all_reduce=None if ar is None else ar.all_reduce)

    for _ in range(max(2, args.warmup)):
        step()
    torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            step()                                   # warm the side stream's workspace before capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
    run_once = graph.replay if graph is not None else step
    for _ in range(3):
        run_once()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_once()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank != 0:
        return None
    peak = 6549.8
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:                                                 # noqa: BLE001
        pass
    per_gpu = (wbytes + kvbytes) / (ms * 1e-3) / 1e9
    return {
        "metric": "27B EXL3 decode tokens/s", "value": round(B / (ms * 1e-3), 2), "unit": "tok/s",
        "ms_per_step": round(ms, 4), "n_gpus": world, "batch": B, "ctx": ctx, "layers": args.layers,
        "cuda_graph": graph is not None, "status_word": _ext.workspace_status(dev) | (ar.status() if ar is not None else 0),
        "allreduce": "one-shot kernel over peer memory" if ar is not None else ("nccl" if world > 1 else None),
        "per_gpu_bytes_per_step": {"packed_weights": wbytes, "kv_cache": kvbytes},
        "per_gpu_hbm_gbs": round(per_gpu, 1), "frac_of_measured_hbm": round(per_gpu / peak, 4),
        "kv_cache_dtype": kv, "data": "synthetic (random-init weights, random KV cache)", "attention": "exl3_decode_attn" if args.attn == "own" else "torch SDPA (library)",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=LAYERS, help="fewer layers for a quick functional run")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--attn", choices=["own", "sdpa"], default="own",
                    help="decode attention: this library's kernel, or torch's scaled_dot_product_attention")
    ap.add_argument("--kv", choices=["fp16", "fp8"], default="fp16", help="KV cache: fp16, or e4m3 with scale 1")
    ap.add_argument("--tc-from", type=int, default=9, help="smallest batch that takes the tcgen05 path (9..17)")
    ap.add_argument("--allreduce", default="oneshot", choices=["oneshot", "nccl"],
                    help="tensor parallel: this library's one-shot all-reduce over peer memory, or the NCCL collective")
    args = ap.parse_args()
    line = run(args)
    if line is not None:
        print(json.dumps(line), flush=True)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # leave without tearing down NCCL under a live captured graph (that teardown can block)
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
