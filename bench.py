"""Benchmark of the EXL3 fused decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows R] [--impl reference]

Workload (`config.workload`): the mixed-bitwidth decode shards of one 27B-class decoder layer --
qkv_proj (q 5120->6144 @4 bpw, k 5120->1024 @5, v 5120->1024 @6; one grouped launch),
gate_up_proj (2 x 5120->17408 @3; one grouped launch), down_proj (17408->5120 @4) -- at batch
`--rows` (default 1), fp16 activations ~N(0,1), uniform-random trellis words, +-1 sign vectors.
One step = one pass over the three fused layers: six kernel launches (an activation pre-pass and the
GEMV per layer).  Three independent weight sets (3 x 134 MB) are rotated so no step finds its trellis
in the 126 MB L2.

metric  = algorithmic bytes (trellis + activations in + out) moved per second, whole job.
value   = inputs resident in HBM: ONE CUDA graph of exactly `--steps` steps, replayed >= 100 times and
          for >= 250 ms, every replay timed with CUDA events (max over ranks); the median replay is
          reported, its spread is in `timing`.  `by_rows` repeats this at 1 / 4 / 16 rows.
e2e     = same metric through the plugin's custom op with HOST activations, every step: pinned host activations
          -> device, three `orcasaq2::layer_gemm` calls, every result -> pinned host; replayed from a CUDA
          graph (the plugin's serving mode) in which the copies of later inputs and earlier results run on
          side branches beside the layers.  The eager time (per layer: copy in, op, copy out, one stream) is
          reported beside it.
N > 1   = the same layer under tensor parallelism (column-parallel qkv / gate_up, row-parallel
          down_proj followed by this library's one-shot all-reduce over peer memory; `--allreduce nccl`
          uses the library collective instead), strong scaling: the job's total bytes are fixed.
          The line then also carries `decoder_27b_tp`: the 27B decoder of bench_model.py at batch 64 with
          an 8192-token cache on the same ranks (BASELINE config 5).
prefill       = (N = 1) BASELINE config 3 on the same GPU: TFLOPS of the tcgen05 decode-GEMM and of the reference's
                many-row route at M = 512 / 2048 / 8192, both shapes.
roofline      = the dominant kernel (gate_up grouped GEMV) alone, graph-replayed; `roofline_by_k` (N = 1):
                one 5120->17408 shard at 2..6 bits per weight, 1 and 16 rows.

decoder_27b = (N = 1 only, after the timed region, `--no-decoder` skips it) tokens/s of the random-init 27B
          decoder of bench_model.py at batch 1 and 32 with a 4096-token cache (batch 32 also with an fp8 cache), each run in a child
          process; the second half of the headline metric, reported beside the GEMV figure and
          not part of `value`, `e2e` or `ms_per_step`; with the same decoder's token rate on the host
          cores extrapolated from per-layer CPU timings.

`--impl reference` times the CPU restatement of the reference path (PyTorch on the host cores:
decode -> Hadamard -> matmul) over the same whole step.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "orcasaq2-kernel_b200"))

# (name, ic, [(oc, K), ...]) -- one grouped launch each
LAYERS = [
    ("qkv_proj", 5120, [(6144, 4), (1024, 5), (1024, 6)]),
    ("gate_up_proj", 5120, [(17408, 3), (17408, 3)]),
    ("down_proj", 17408, [(5120, 4)]),
]
N_SETS = 3
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(ic, spec, rows):
    """trellis + activations in + activations out (sign vectors, <0.1 %, left out)."""
    return sum(ic * oc * K // 8 for oc, K in spec) + rows * ic * 2 + rows * sum(oc for oc, _ in spec) * 2


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:                                    # noqa: BLE001
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:                                    # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------ GPU arm
def make_shard(torch, ic, oc, K, seed, device):
    g = torch.Generator(device="cpu").manual_seed(seed)
    tr = torch.randint(0, 65536, (ic // 16, oc // 16, 16 * K), generator=g, dtype=torch.int32).to(torch.int16)
    suh = (torch.randint(0, 2, (ic,), generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (oc,), generator=g) * 2 - 1).to(torch.float16)
    return dict(trellis=tr.to(device), suh=suh.to(device), svh=svh.to(device), mcg=False, mul1=False,
                K=K, ic=ic, oc=oc)


def tp_slice(name, ic, spec, rank, world):
    """This rank's part of a layer: column-parallel slices every shard's outputs, row-parallel
    (down_proj) slices the inputs.  Replicated KV heads: a shard narrower than 128*world keeps
    128-wide groups and ranks share them."""
    if world == 1:
        return ic, spec, (0, ic), [(0, oc) for oc, _ in spec]
    if name == "down_proj":
        part = ic // world
        return part, spec, (rank * part, (rank + 1) * part), [(0, oc) for oc, _ in spec]
    out, rng = [], []
    for oc, K in spec:
        width = max(128, oc // world)
        groups = oc // width
        idx = rank // max(1, world // groups) if groups < world else rank
        out.append((width, K))
        rng.append((idx * width, (idx + 1) * width))
    return ic, out, (0, ic), rng


def build_sets(torch, device, rank, world):
    """N_SETS independent weight sets of this rank's slices (seeded; the full tensors are never
    materialised for world > 1: a slice of random words is random words)."""
    sets = []
    for s in range(N_SETS):
        layers = []
        for li, (name, ic, spec) in enumerate(LAYERS):
            ic_r, spec_r, _, _ = tp_slice(name, ic, spec, rank, world)
            shards = [make_shard(torch, ic_r, oc, K, 1000 * 2 + 100 * s + 10 * li + i + 7919 * rank, device)
                      for i, (oc, K) in enumerate(spec_r)]
            col = 0
            for sh in shards:
                sh["out_col"] = col
                col += sh["oc"]
            layers.append((name, ic_r, shards, col))
        sets.append(layers)
    return sets


def _leave(world):
    """End a multi-rank run without tearing NCCL down under a live captured graph (that teardown can
    block): agree that everyone is done, flush, and exit the process."""
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def _graph_of(torch, body, steps, warm):
    """Capture `steps` calls of body(i) into one CUDA graph on a side stream (after `warm` eager calls on that
    stream, so every scratch buffer exists before capture)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(warm):
            body(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(steps):
                body(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return graph


def time_replays(torch, dist, graph, world, dev, min_region_ms, min_replays, max_replays=5000):
    """Replay `graph` often enough that the timed region lasts at least `min_region_ms`, with a CUDA event
    between replays; every replay's time is the max over ranks.  Returns per-replay milliseconds (sorted) and
    the length of the whole region."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    est = torch.tensor([a.elapsed_time(b) / 5.0], device=dev)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MAX)          # every rank must issue the same number of replays
    n = int(min(max_replays, max(min_replays, min_region_ms / max(float(est.item()), 1e-4) + 1)))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
    barrier()
    evs[0].record()
    for i in range(n):
        graph.replay()
        evs[i + 1].record()
    barrier()
    t = torch.tensor([evs[i].elapsed_time(evs[i + 1]) for i in range(n)], device=dev)
    region = torch.tensor([evs[0].elapsed_time(evs[n])], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(region, op=dist.ReduceOp.MAX)
    return sorted(t.tolist()), float(region.item())


def _spread(ts, per):
    """median / min / p10 / p90 / max of per-replay times, divided by `per` (steps or launches per replay)."""
    n = len(ts)
    q = lambda f: ts[min(n - 1, int(f * n))] / per               # noqa: E731
    return {"median": round(ts[n // 2] / per, 6), "min": round(ts[0] / per, 6), "p10": round(q(0.10), 6),
            "p90": round(q(0.90), 6), "max": round(ts[-1] / per, 6), "replays": n}


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from orcasaq2 import _ext
    from orcasaq2 import ops  # noqa: F401  (registers orcasaq2::layer_gemm)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _ext.lib()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rows, K_steps = args.rows, max(1, args.steps)
    warm = max(3, args.warmup)
    sets = build_sets(torch, dev, rank, world)
    # row-parallel partial sums: this library's one-shot all-reduce over peer memory (--allreduce nccl: the library collective)
    ar = None
    if world > 1 and args.allreduce == "oneshot":
        from orcasaq2 import comm
        ar = comm.OneShotAllReduce(max_values=64 * 5120, device=dev)

    def all_reduce(t):
        if ar is not None:
            ar.all_reduce(t)
        else:
            dist.all_reduce(t)

    def make_io(r):
        xs_ = {ic: torch.randn((r, ic), generator=torch.Generator().manual_seed(5)).half().to(dev)
               for ic in {l[1] for l in sets[0]}}
        ys_ = [[torch.empty((r, tot), dtype=torch.half, device=dev) for (_, _, _, tot) in layers] for layers in sets]
        return xs_, ys_

    def stepper(xs_, ys_, only=None):
        def step(i):
            layers, out = sets[i % N_SETS], ys_[i % N_SETS]
            for li, ((name, ic_r, shards, _), y) in enumerate(zip(layers, out)):
                if only is not None and li != only:
                    continue
                _ext.gemv_grouped(xs_[ic_r], shards, y)
                if world > 1 and name == "down_proj":
                    all_reduce(y)                           # row-parallel partial sums
        return step

    def bytes_per_step(r):
        return sum(algorithmic_bytes(ic, spec, r) for _, ic, spec in LAYERS)

    # ---- the timed region: ONE CUDA graph holding exactly `--steps` steps (weight sets rotated, so no step
    # finds its trellis in L2), replayed at least 100 times and for at least 250 ms; every replay is timed by
    # itself with CUDA events and the median replay is the figure reported.  Launches and, for N > 1, the NCCL
    # all-reduces are issued by the GPU front end, so the host's launch cost is not what gets measured.
    xs, ys = make_io(rows)
    step = stepper(xs, ys)
    for i in range(warm):
        step(i)
    torch.cuda.synchronize()
    if ar is not None and ar.status():
        raise SystemExit("bench.py: the one-shot all-reduce timed out waiting for a peer during warm-up")
    sampler = ClockSampler(local)
    if args.no_graph:
        graph = None
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K_steps):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        tm = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ts, region_ms = [float(tm.item())], float(tm.item())
    else:
        graph = _graph_of(torch, step, K_steps, N_SETS)
        sampler.start()
        ts, region_ms = time_replays(torch, dist, graph, world, dev, 250.0 if not args.skip_extras else 0.0,
                                     100 if not args.skip_extras else 1)
    if region_ms < 400 and graph is not None and not args.skip_extras:
        # keep the GPU under the same load long enough for the 100 ms clock sampler to see it
        for _ in range(int((400 - region_ms) / max(ts[len(ts) // 2], 1e-3)) + 1):
            graph.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    spread = _spread(ts, K_steps)
    ms_step = spread["median"]
    full_bytes = bytes_per_step(rows)
    value = full_bytes / (ms_step * 1e-3) / 1e9
    launches_per_layer = 2                            # the activation pre-pass and the GEMV

    if args.skip_extras:
        if rank == 0:
            print(json.dumps({"metric": "EXL3 fused decode GEMV throughput (trellis + activation bytes)",
                              "value": round(value, 1), "unit": "GB/s", "ms_per_step": round(ms_step, 5),
                              "steps": K_steps, "config": {"workload": ",".join(l[0] for l in LAYERS), "rows": rows},
                              "note": "profiling run: extras skipped"}), flush=True)
        _leave(world)
        return

    # ---- the other batch sizes BASELINE config 2 names, same method, shorter regions
    by_rows = {str(rows): {"value": round(value, 1), "ms_per_step": round(ms_step, 5)}}
    if not args.no_graph:
        for r in (1, 4, 16):
            if r == rows:
                continue
            xr, yr = make_io(r)
            g = _graph_of(torch, stepper(xr, yr), K_steps, N_SETS)
            tr_, _ = time_replays(torch, dist, g, world, dev, 60.0, 30)
            m = tr_[len(tr_) // 2] / K_steps
            by_rows[str(r)] = {"value": round(bytes_per_step(r) / (m * 1e-3) / 1e9, 1), "ms_per_step": round(m, 5)}
            del g, xr, yr

    # ---- end to end: host activations in, host outputs back, through the plugin's custom op
    hx = {ic: x.cpu().pin_memory() for ic, x in xs.items()}
    hy = [torch.empty((rows, tot), dtype=torch.half).pin_memory() for (_, _, _, tot) in sets[0]]
    lay_args = [[([s["trellis"] for s in sh], [s["suh"] for s in sh], [s["svh"] for s in sh],
                  [s["oc"] for s in sh], [float(s["K"]) for s in sh], [False] * len(sh), [False] * len(sh))
                 for (_, _, sh, _) in layers] for layers in sets]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def e2e_step(i):
        layers = sets[i % N_SETS]
        for li, (name, ic_r, _, _) in enumerate(layers):
            xd = hx[ic_r].to(dev, non_blocking=True)
            y = torch.ops.orcasaq2.layer_gemm(xd, *lay_args[i % N_SETS][li])
            if world > 1 and name == "down_proj":
                all_reduce(y)
            hy[li].copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    n_e2e = max(K_steps, 200)
    for i in range(3):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    barrier()
    e2e_eager_s = (time.perf_counter() - t0) / n_e2e
    e2e_s, e2e_mode = e2e_eager_s, "eager: per layer H2D copy, plugin op, D2H copy; one sync per step"
    if not args.no_graph:
        # The serving mode of the plugin (the op is built to replay inside CUDA graphs): per weight set
        # one graph of [pinned host x -> device, the three plugin ops, outputs -> pinned host]; a step
        # rewrites the host activations, replays the graph and waits for the outputs.
        # Inside the graph the copies run on two side branches: the input of a later layer arrives while the earlier
        # layers compute, and a layer's result leaves for the host while the next layer computes.  Only the first
        # input copy and the last result copy are exposed.  Every layer still gets its activations from pinned host
        # memory and every result is read back, every step.
        ics = sorted(xs)
        hxs = {ic: hx[ic] for ic in ics}                      # pinned host activations, one per distinct input
        dxv = {ic: torch.empty_like(xs[ic]) for ic in ics}
        hys = [torch.empty((rows, tot), dtype=torch.half).pin_memory() for (_, _, _, tot) in sets[0]]
        cin, cout = torch.cuda.Stream(), torch.cuda.Stream()

        def e2e_body(si):
            main = torch.cuda.current_stream()
            first_ic = sets[si][0][1]
            dxv[first_ic].copy_(hxs[first_ic], non_blocking=True)
            cin.wait_stream(main)
            with torch.cuda.stream(cin):
                for ic in ics:
                    if ic != first_ic:
                        dxv[ic].copy_(hxs[ic], non_blocking=True)
            arrived = {first_ic}
            for li, (name, ic_r, _, tot) in enumerate(sets[si]):
                if ic_r not in arrived:
                    main.wait_stream(cin)
                    arrived.update(ics)
                y = torch.ops.orcasaq2.layer_gemm(dxv[ic_r], *lay_args[si][li])
                if world > 1 and name == "down_proj":
                    all_reduce(y)
                cout.wait_stream(main)
                with torch.cuda.stream(cout):
                    hys[li].copy_(y, non_blocking=True)
                    y.record_stream(cout)
            main.wait_stream(cin)
            main.wait_stream(cout)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        e2e_graphs = []
        with torch.cuda.stream(side):
            for si in range(N_SETS):
                e2e_body(si)
            torch.cuda.synchronize()
            for si in range(N_SETS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    e2e_body(si)
                e2e_graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

        def e2e_graph_step(i):
            for ic in ics:
                hxs[ic][0, 0] = 0.001 * (i % 7)     # the host inputs are live, not baked into the graph
            e2e_graphs[i % N_SETS].replay()
            torch.cuda.synchronize()

        for i in range(3):
            e2e_graph_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            e2e_graph_step(i)
        barrier()
        e2e_s = (time.perf_counter() - t0) / n_e2e
        e2e_mode = ("CUDA-graph replay per step of [pinned host activations -> device, three orcasaq2::layer_gemm ops, "
                    "every result -> pinned host]; the copies of later inputs and earlier results run on side branches "
                    "of the graph beside the layers; host inputs rewritten before and one sync after every replay; "
                    f"{n_e2e} steps timed on the host clock")
        e2e_graph_bytes = (sum(h.numel() * 2 for h in hxs.values()), sum(h.numel() * 2 for h in hys))
    if world > 1:
        t = torch.tensor([e2e_s, e2e_eager_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, e2e_eager_s = float(t[0].item()), float(t[1].item())
    h2d = sum(rows * ic_r * 2 for (_, ic_r, _, _) in sets[0])
    d2h = sum(rows * tot * 2 for (_, _, _, tot) in sets[0])
    if not args.no_graph:
        h2d, d2h = e2e_graph_bytes                 # what the graph mode copies: distinct inputs once, all results

    # ---- roofline of the dominant kernel (the gate_up grouped GEMV), alone: a graph of N_SETS launches over
    # the rotated weight sets (3 x 67 MB > L2), replayed; duration per launch from CUDA events around each replay
    gi = max(range(len(sets[0])), key=lambda j: sum(s_["ic"] * s_["oc"] * s_["K"] for s_ in sets[0][j][2]))
    name, ic_r, _, _ = sets[0][gi]
    spec_r = [(s["oc"], s["K"]) for s in sets[0][gi][2]]
    kb = algorithmic_bytes(ic_r, spec_r, rows)
    xg, yg = make_io(rows)

    def one_layer(i):
        _ext.gemv_grouped(xg[ic_r], sets[i % N_SETS][gi][2], yg[i % N_SETS][gi])

    peak, kind = measured_peaks()
    if args.no_graph:
        avg_ms = ms_step
    else:
        g = _graph_of(torch, one_layer, 2 * N_SETS, N_SETS)
        tl, _ = time_replays(torch, dist, g, 1, dev, 40.0, 50)          # this rank's own kernel, no collective inside
        avg_ms = tl[len(tl) // 2] / (2 * N_SETS)
    achieved = kb / (avg_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": f"gemv_kernel ({name}, {len(spec_r)} shard(s), one launch)",
            "achieved": round(achieved, 1), "peak": peak, "peak_kind": f"of {kind}", "unit": "GB/s",
            "frac": round(achieved / peak, 4), "frac_of_8000_nominal": round(achieved / 8000.0, 4),
            "algorithmic_bytes_per_launch": kb, "avg_launch_us": round(avg_ms * 1e3, 2),
            "timing": "median graph replay of 6 launches over 3 rotated weight sets, CUDA events on the replay stream",
            "traffic": NCU_TRAFFIC_BYTES.get((rows, world))}
    by_k = roofline_by_k(torch, dist, _ext, dev, peak) if world == 1 and rank == 0 and not args.no_graph else None
    prefill = prefill_block(torch, _ext, dev) if world == 1 and rank == 0 and not args.no_graph else None
    cpu = cpu_baseline(rows) if world == 1 and rank == 0 else None
    ar_block = None
    if world > 1 and not args.no_graph:
        # the exchange by itself: [rows, 5120] fp16, 20 calls per graph replay, this library's kernel and NCCL's
        ar_block = {"values": rows * 5120, "unit": "us per call", "used_in_step": args.allreduce}
        t_ar = torch.randn((rows, 5120), device=dev).half()
        for nm, fn in (("oneshot", (lambda: ar.all_reduce(t_ar)) if ar is not None else None), ("nccl", lambda: dist.all_reduce(t_ar))):
            if fn is None:
                continue
            g = _graph_of(torch, lambda i: fn(), 20, 3)
            tl, _ = time_replays(torch, dist, g, world, dev, 20.0, 20)
            ar_block[nm] = round(tl[len(tl) // 2] / 20 * 1e3, 2)
            del g
        if ar is not None:
            ar_block["status_word"] = ar.status()
    used_graph = graph is not None
    tp_model = None
    if world > 1 and not args.no_decoder:
        # BASELINE config 5 on the same ranks and kernels: the 27B decoder under tensor parallelism
        del sets, xs, ys, xg, yg, lay_args, graph
        torch.cuda.empty_cache()
        import bench_model
        try:
            tp_model = bench_model.run(bench_model.default_args(batch=64, ctx=8192, steps=10, warmup=2, allreduce=args.allreduce))
        except Exception as e:                                          # noqa: BLE001
            tp_model = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        torch.cuda.empty_cache()
        try:                                                            # the same with an e4m3 KV cache (scale 1)
            tp8 = bench_model.run(bench_model.default_args(batch=64, ctx=8192, steps=10, warmup=2, allreduce=args.allreduce,
                                                           kv="fp8"))
        except Exception as e:                                          # noqa: BLE001
            tp8 = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        if tp_model is not None and tp8 is not None:
            tp_model["fp8_kv"] = {k: tp8[k] for k in ("value", "ms_per_step", "per_gpu_hbm_gbs", "status_word", "unavailable")
                                  if k in tp8}
    if rank != 0:
        _leave(world)
        return
    line = {
        "metric": "EXL3 fused decode GEMV throughput (trellis + activation bytes)", "value": round(value, 1),
        "unit": "GB/s", "n_gpus": world, "steps": K_steps, "warmup": warm,
        "ms_per_step": round(ms_step, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"mixed-bitwidth decode shards of one layer (qkv 4/5/6 bpw, gate_up 3 bpw, "
                               f"down 4 bpw), rows={rows}", "rows": rows,
                   "bytes_per_step": full_bytes, "l2": "inputs larger than L2: 3 weight sets of 134 MB rotated",
                   "parallelism": f"tp{world}" if world > 1 else "single GPU",
                   "pct_of_8TBs_nominal": round(value / 8000.0 * 100, 2)},
        "timing": {"method": f"one CUDA graph of {K_steps} steps replayed {spread['replays']} times, each replay timed "
                             "with CUDA events (max over ranks); value = median replay",
                   "timed_region_ms": round(region_ms, 2), "ms_per_step": spread},
        "by_rows": by_rows,
        "e2e": {"value": round(full_bytes / e2e_s / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3, 5), "mode": e2e_mode,
                "eager_ms_per_step": round(e2e_eager_s * 1e3, 5)},
        # kernels of this library per step: per fused layer the activation pre-pass and the GEMV, plus the all-reduce at N > 1
        "gpu_launches": K_steps * spread["replays"] * (len(LAYERS) * launches_per_layer + (1 if ar is not None else 0)),
        "cuda_graph": used_graph,
        "clocks": clocks, "roofline": roof,
    }
    if isinstance(clocks, dict) and clocks.get("sm_mhz"):
        # clock-normalised step time (us x GHz = thousands of SM cycles per step): comparable between runs whose
        # sampled clocks differ
        line["timing"]["kcycles_per_step"] = round(ms_step * 1e3 * float(clocks["sm_mhz"]) / 1e3, 1)
    if by_k is not None:
        line["roofline_by_k"] = by_k
    if prefill is not None:
        line["prefill"] = prefill
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if world == 1 and not args.no_decoder:
        line["decoder_27b"] = decoder_tok_s()
        if cpu is not None and "decoder_27b_tok_s" in cpu:
            line["decoder_27b"]["cpu_tok_s_bs1"] = cpu["decoder_27b_tok_s"]
            b1 = line["decoder_27b"].get("bs1", {}).get("value")
            if b1 and cpu["decoder_27b_tok_s"]:
                line["decoder_27b"]["gpu_over_cpu_bs1"] = round(b1 / cpu["decoder_27b_tok_s"], 1)
    if ar_block is not None:
        line["allreduce"] = ar_block
    if tp_model is not None:
        line["decoder_27b_tp"] = tp_model
    print(json.dumps(line), flush=True)
    _leave(world)


def _takes_pair_kernel(rows, ic, oc):
    """The library's own choice between its two many-row kernels (exl3_gemm_tc.cu, use_dense), restated for the label."""
    if (oc // 128) % 2:
        return False
    return rows >= 1024 or (oc >= 2048 and (rows >= 640 or (rows >= 384 and ic >= 2 * oc)))


def prefill_block(torch, _ext, dev):
    """BASELINE config 3: M tokens x (5120 -> 17408 at 3 bpw, 17408 -> 5120 at 4 bpw), bf16 activations: TFLOPS of the
    library's tcgen05 path (exl3_gemm_tc: in-kernel decode up to 1023 rows; from 1024 rows the weight is rebuilt once
    and a dense GEMM runs on CTA pairs) and of the reference's own route for many rows with a library GEMM (rotate,
    rebuild the weight, torch.matmul, rotate back: orcasaq2/ops.py:50-59), CUDA events over 8 calls after 2 warm-ups."""
    peaks = {"burst": 1679.6, "sustained": 1385.7}
    try:
        mp = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peaks = {"burst": float(mp["bf16_tflops"]), "sustained": float(mp["bf16_tflops_sustained"])}
    except Exception:                                        # noqa: BLE001
        pass
    out = {"unit": "TFLOP/s", "flops": "2*M*ic*oc (decode and Hadamard not counted)", "peak_bf16_tflops": peaks, "cases": []}

    def timed(fn, n=8):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n * 1e-3

    for ic, oc, K in ((5120, 17408, 3), (17408, 5120, 4)):
        sh = make_shard(torch, ic, oc, K, 7000 + K, dev)
        for m in (512, 2048, 8192):
            x = torch.randn((m, ic), generator=torch.Generator().manual_seed(m)).to(torch.bfloat16).to(dev)
            y = torch.empty((m, oc), dtype=torch.half, device=dev)
            t_tc = timed(lambda: _ext.gemm_tc(x, sh["trellis"], y, sh["suh"], sh["svh"]))

            def route():
                xf = x.half()
                xh = torch.empty_like(xf)
                _ext.had_r_128(xf, xh, sh["suh"], None, 1.0)
                w = torch.empty((ic, oc), dtype=torch.half, device=dev)
                _ext.reconstruct(w, sh["trellis"], K, False, False)
                _ext.hgemm_recon(xh, w, y)
                _ext.had_r_128(y, y, None, sh["svh"], 1.0)
            t_rt = timed(route)
            fl = 2.0 * m * ic * oc
            out["cases"].append({"shape": f"{ic}->{oc} @{K}bpw", "M": m,
                                 "tcgen05_tflops": round(fl / t_tc / 1e12, 1),
                                 "tcgen05_frac_of_burst_peak": round(fl / t_tc / 1e12 / peaks["burst"], 3),
                                 "rotate_reconstruct_library_gemm_tflops": round(fl / t_rt / 1e12, 1),
                                 "plugin_dispatch": "tcgen05: decode once + dense GEMM on CTA pairs" if _takes_pair_kernel(m, ic, oc)
                                 else "tcgen05: in-kernel decode"})
            del x, y
        del sh
        torch.cuda.empty_cache()
    out["status_word"] = _ext.gemm_tc_status()
    return out


# Decode + mma.sync rate of the 3INST codebook with no memory access at all (registers only, every SM busy),
# in 10^12 weights per second on B200 at 1.9 GHz, per bitrate: the ceiling of any kernel that decodes this
# codebook with integer instructions and consumes the codewords with mma.sync (profiles/decode_rate_b200.md).
DECODE_CEILING_TWS = {2: 6.14, 3: 5.51, 4: 5.91, 5: 5.39, 6: 5.36}


def roofline_by_k(torch, dist, _ext, dev, peak):
    """One 5120 -> 17408 shard at 2..6 bits per weight, 1 and 16 rows: achieved bytes/s against the HBM peak and
    weights/s against the decode ceiling of that bitrate."""
    out = {"shape": "5120->17408, one shard", "unit": "GB/s", "peak": peak, "decode_ceiling_tw_s": DECODE_CEILING_TWS,
           "note": "frac = achieved / HBM peak; of_ceiling = weights per second / register-only decode+mma rate"}
    ic, oc = 5120, 17408
    for K in (2, 3, 4, 5, 6):
        per = ic * oc * K // 8
        n = int(max(3, 400e6 // per + 1))
        shards = [[make_shard(torch, ic, oc, K, 9000 + 10 * K + i, dev)] for i in range(n)]
        for r in (1, 16):
            x = torch.randn((r, ic), generator=torch.Generator().manual_seed(6)).half().to(dev)
            y = torch.empty((r, oc), dtype=torch.half, device=dev)
            g = _graph_of(torch, lambda i: _ext.gemv_grouped(x, shards[i % n], y), n, min(n, 3))
            ts, _ = time_replays(torch, dist, g, 1, dev, 30.0, 20)
            sec = ts[len(ts) // 2] / n * 1e-3
            b = algorithmic_bytes(ic, [(oc, K)], r)
            out[f"k{K}_rows{r}"] = {"achieved": round(b / sec / 1e9, 1), "frac": round(b / sec / 1e9 / peak, 4),
                                    "us": round(sec * 1e6, 2), "tw_s": round(ic * oc / sec / 1e12, 3),
                                    "of_ceiling": round(ic * oc / sec / 1e12 / DECODE_CEILING_TWS[K], 3)}
            del g
        del shards
        torch.cuda.empty_cache()
    return out


def decoder_tok_s():
    """The second half of the headline metric, after the timed region and outside every figure above: the
    random-init 27B decoder of bench_model.py at batch 1 and 32 (4096-token cache; batch 32 also with an e4m3
    cache), each in a process of its own.  Any failure or a run over its time limit is reported in place of the number; it never
    fails the benchmark."""
    import subprocess
    out = {"unit": "tok/s", "ctx": 4096, "source": "bench_model.py (CUDA-graph replay, 64 layers)"}
    script = os.path.join(ROOT, "bench_model.py")
    for batch, kv in ((1, "fp16"), (32, "fp16"), (32, "fp8")):
        key = f"bs{batch}" + ("" if kv == "fp16" else "_fp8_kv")
        try:
            p = subprocess.run([sys.executable, script, "--batch", str(batch), "--ctx", "4096", "--steps", "10", "--kv", kv],
                               capture_output=True, text=True, timeout=180)
            last = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
            if p.returncode != 0 or not last:
                out[key] = {"unavailable": f"exit code {p.returncode}"}
                continue
            r = json.loads(last[-1])
            out[key] = {"value": r["value"], "ms_per_step": r["ms_per_step"], "status_word": r.get("status_word")}
        except Exception as e:                                          # noqa: BLE001
            out[key] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return out


# per-launch DRAM traffic of the gate_up kernel from ncu (dram__bytes_read.sum + write), keyed by
# (rows, world); filled from the captures summarised under profiles/
NCU_TRAFFIC_BYTES = {(1, 1): 67_866_112, (16, 1): 68_354_816}     # profiles/gemv_kernel_gate_up_rows1.md: DRAM bytes read + written of one launch


# ------------------------------------------------------------------------------------ CPU arms
def _cpu_inputs(R, rows):
    """Seeded inputs of one whole step on the host: every shard of every fused layer of LAYERS."""
    out = []
    for li, (_, ic, spec) in enumerate(LAYERS):
        for i, (oc, K) in enumerate(spec):
            tr, suh, svh, x = R.make_layer(4242 + 10 * li + i, ic, oc, K, rows)
            out.append((x, tr, suh, svh))
    return out


def _cpu_step_once(torch, R, inputs, threads):
    """One pass of the reference's CPU PyTorch path (decode -> Hadamard -> matmul -> Hadamard) over all six shards
    of the workload; seconds."""
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    for x, tr, suh, svh in inputs:
        y = R.torch_layer(x, tr, suh, svh)
    dt = time.perf_counter() - t0
    assert torch.isfinite(y.float()).all()
    return dt


def cpu_baseline(rows):
    """The oracle's PyTorch-CPU path on the host cores over the whole workload step, as the same metric
    (algorithmic bytes per second), on a bounded number of passes; plus the C/OpenMP oracle on the same step and
    the 27B decoder's CPU token rate extrapolated from per-layer timings."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import exl3_ref as R
    threads = os.cpu_count() or 1
    inputs = _cpu_inputs(R, rows)
    full_bytes = sum(algorithmic_bytes(ic, spec, rows) for _, ic, spec in LAYERS)
    _cpu_step_once(torch, R, inputs, threads)
    n, total = 0, 0.0
    while total < 10.0 and n < 6:
        total += _cpu_step_once(torch, R, inputs, threads)
        n += 1
    sec = total / n
    out = {"value": round(full_bytes / sec / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
           "sample": f"the whole step (all six shards, {full_bytes} bytes), rows={rows}, {n} passes of {sec:.2f} s "
                     f"(PyTorch-CPU restatement of the reference path, torch.set_num_threads({threads}))"}
    try:                                                    # second CPU number: the C/OpenMP oracle, same step
        co = R.COracle()
        t0 = time.perf_counter()
        for x, tr, suh, svh in inputs:
            co.layer(x.numpy(), co.reconstruct(tr.numpy()), suh.numpy(), svh.numpy())
        out["c_openmp_value"] = round(full_bytes / (time.perf_counter() - t0) / 1e9, 4)
    except Exception as e:                                  # noqa: BLE001
        out["c_openmp_value"] = None
        out["c_openmp_error"] = str(e)[:80]
    try:
        # 27B decoder at batch 1 on the same cores: a layer is the step above plus o_proj (6144 -> 5120); the head is
        # the reference's dequantise-then-linear on one eighth of the vocabulary, times eight; attention left out
        # (it would only lower the figure)
        tr, suh, svh, x = R.make_layer(4300, 6144, 5120, 4, 1)
        torch.set_num_threads(threads)
        t0 = time.perf_counter()
        R.torch_layer(x, tr, suh, svh)
        o_sec = time.perf_counter() - t0
        q, sc = R.make_int8_table(4301, 151936 // 8, 5120)
        xh = torch.randn((1, 5120), generator=torch.Generator().manual_seed(7)).half()
        t0 = time.perf_counter()
        R.int8_head_torch(q, sc, xh)
        head_sec = 8 * (time.perf_counter() - t0)
        tok = 1.0 / (64 * (sec + o_sec) + head_sec)
        out["decoder_27b_tok_s"] = round(tok, 5)
        out["decoder_27b_note"] = (f"extrapolated: 64 x ({sec:.2f} s step + {o_sec:.2f} s o_proj) + {head_sec:.2f} s head "
                                   f"per token on {threads} cores, attention not counted")
    except Exception as e:                                  # noqa: BLE001
        out["decoder_27b_error"] = str(e)[:80]
    return out


def run_reference(args):
    """The reference's CPU implementation of the path (its PyTorch restatement: the trellis kernels themselves live
    in a wheel that is not part of the reference tree), host cores only.  Same metric and config as the GPU arm;
    a step is one pass over all six shards of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import exl3_ref as R
    threads = os.cpu_count() or 1
    rows = args.rows
    inputs = _cpu_inputs(R, rows)
    warm = max(1, min(args.warmup, 5))
    first = [_cpu_step_once(torch, R, inputs, threads) for _ in range(warm)]
    # the whole run must end within a few minutes whatever --steps is
    steps = max(1, min(args.steps, int(240.0 / max(first[-1], 1e-3))))
    t = [_cpu_step_once(torch, R, inputs, threads) for _ in range(steps)]
    sec = sum(t) / len(t)
    full_bytes = sum(algorithmic_bytes(i, spec, rows) for _, i, spec in LAYERS)
    v = round(full_bytes / sec / 1e9, 4)
    sample = f"the whole step: all six shards ({full_bytes} bytes), rows={rows}, {steps} steps after {warm} warm-up"
    print(json.dumps({
        "impl": "reference", "metric": "EXL3 fused decode GEMV throughput (trellis + activation bytes)",
        "value": v, "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps,
        "warmup": warm, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"mixed-bitwidth decode shards of one layer (qkv 4/5/6 bpw, gate_up 3 bpw, "
                               f"down 4 bpw), rows={rows}", "rows": rows, "bytes_per_step": full_bytes,
                   "parallelism": "host cores"},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=1, choices=range(1, 17))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=[l[0] for l in LAYERS],
                    help="run just this fused layer each step (small case for profiling)")
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--allreduce", default="oneshot", choices=["oneshot", "nccl"],
                    help="N > 1: how the row-parallel partial sums are added (this library's one-shot kernel over peer "
                         "memory, or the NCCL collective)")
    ap.add_argument("--no-decoder", action="store_true",
                    help="skip the 27B decoder runs reported beside the GEMV figure (N = 1 only)")
    ap.add_argument("--skip-extras", action="store_true",
                    help="skip the end-to-end, roofline and CPU-baseline legs (profiling runs)")
    args = ap.parse_args()
    if args.only:
        LAYERS[:] = [l for l in LAYERS if l[0] == args.only]
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
