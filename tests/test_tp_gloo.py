"""Tensor-parallel data path on CPU ranks (gloo, world size 2): every rank cuts its slice with the
plugin's own slicing code, runs the oracle layer on it, and the collectives vLLM would issue
(concatenation of column-parallel outputs, all-reduce of row-parallel partial sums) reproduce the
unsharded layer.  Also the failure path: a rank that never joins makes the others time out on the
host, not hang."""
import os
import sys
import types

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    for p in (os.path.join(ROOT, "orcasaq2-kernel_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import exl3_ref as R
    import vllm.model_executor.parameter as vp
    vp.get_tensor_model_parallel_rank = lambda: rank
    vp.get_tensor_model_parallel_world_size = lambda: world
    from orcasaq2 import config as cfg
    cfg._tp_info = lambda: (rank, world)
    co = R.COracle()
    m = cfg.Exl3LinearMethod(cfg.Exl3Config.from_config({}), "l.x")
    ic, rows = 256, 3
    x = torch.randn((rows, ic), generator=torch.Generator().manual_seed(1)).half()
    # column-parallel fused layer (two shards, different bitrates)
    spec = [(256, 3), (512, 5)]
    full = [R.make_layer(10 + i, ic, oc, K, 1)[:3] for i, (oc, K) in enumerate(spec)]
    layer = types.SimpleNamespace(exl3_tp=dict(in_part=ic, in_full=ic, out_parts=[oc // world for oc, _ in spec],
                                               out_full=sum(oc for oc, _ in spec)))
    outs = []
    for pos, (t, a, b) in enumerate(full):
        ts, as_, bs = m._slice_for_rank(layer, pos, len(full), t, a, b)
        outs.append(torch.from_numpy(co.layer(x.numpy(), co.reconstruct(ts.numpy()), as_.numpy(), bs.numpy())))
    mine = torch.cat(outs, 1)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    # row-parallel layer: partial sums, all-reduce
    t, a, b = R.make_layer(20, ic * world, 128, 4, 1)[:3]
    x2 = torch.randn((rows, ic * world), generator=torch.Generator().manual_seed(2)).half()
    layer2 = types.SimpleNamespace(exl3_tp=dict(in_part=ic, in_full=ic * world, out_parts=[128], out_full=128))
    ts, as_, bs = m._slice_for_rank(layer2, 0, 1, t, a, b)
    part = torch.from_numpy(co.layer(np.ascontiguousarray(x2.numpy()[:, rank * ic:(rank + 1) * ic]),
                                     co.reconstruct(ts.numpy()), as_.numpy(), bs.numpy()))
    dist.all_reduce(part)
    if rank == 0:
        ref_cols = [co.layer(x.numpy(), co.reconstruct(tt.numpy()), aa.numpy(), bb.numpy()) for tt, aa, bb in full]
        # rank r holds columns [r*w, (r+1)*w) of every shard: reassemble shard by shard
        got = []
        for pos, (oc, _) in enumerate(spec):
            w = oc // world
            off = sum(o // world for o, _ in spec[:pos])
            got.append(np.concatenate([g.numpy()[:, off:off + w] for g in gathered], 1))
        ok_col = all(np.allclose(g, r, atol=1e-3) for g, r in zip(got, ref_cols))
        ref_row = co.layer(x2.numpy(), co.reconstruct(t.numpy()), a.numpy(), b.numpy())
        q.put((ok_col, bool(np.allclose(part.numpy(), ref_row, atol=1e-3))))
    dist.destroy_process_group()


def test_two_rank_column_and_row_parallel():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok_col, ok_row = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok_col and ok_row


def _lonely(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        q.put("joined")
    except Exception as e:                                   # noqa: BLE001
        q.put("timeout:" + type(e).__name__)


def test_missing_rank_is_a_host_side_timeout():
    """Failure detection without touching a GPU: rank 1 never starts; rank 0 gets an exception
    from the rendezvous within its short timeout instead of waiting forever."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely, args=(0, 2, 29950 + os.getpid() % 40, q))
    p.start()
    msg = q.get(timeout=120)
    p.join(timeout=30)
    assert msg.startswith("timeout:")


def _oneshot_worker(rank, world, port, q):
    """The exchange of the one-shot all-reduce, played with gloo: every rank publishes its partial (all_gather
    stands in for the peers' mapped buffers), then adds ALL partials itself in rank order in fp32."""
    sys.path.insert(0, os.path.join(ROOT, "orcasaq2-kernel_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from orcasaq2 import comm
    ok = True
    for it, n in enumerate([5120, 64 * 5120, 8]):
        part = (torch.randn((n,), generator=torch.Generator().manual_seed(7 * it + rank)) * 80).half()
        slots = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(slots, part)
        mine = comm.allreduce_reference(slots)
        # every rank ends with bitwise the same tensor ...
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        ok = ok and all(torch.equal(e, mine) for e in everyone)
        # ... which is the library all-reduce's sum up to one fp16 rounding of a differently ordered sum
        lib = part.clone().float()
        dist.all_reduce(lib)
        ok = ok and bool(((mine.float() - lib).abs() <= lib.abs() * 2 ** -10 + 1e-3).all())
    if rank == 0:
        q.put(ok)
    dist.destroy_process_group()


def test_one_shot_all_reduce_algebra_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + os.getpid() % 200
    procs = [ctx.Process(target=_oneshot_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok
