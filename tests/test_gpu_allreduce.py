"""The one-shot all-reduce kernel (exl3_allreduce_oneshot) through the C ABI.

On ONE GPU the ranks of a two-rank exchange are played one after the other on two communication buffers of the
same device -- never two kernels that wait for each other at the same time.  "Rank 1" goes first with a small
poll limit: it publishes its partial, signals, finds no signal from rank 0, gives up, sets its status word and
returns (this is the bounded wait running out, on a flag nothing sets).  Rank 0 then finds rank 1's signal and
completes; rank 1, called again, completes too.  With two or more GPUs the same exchange also runs for real in
child processes (NCCL only carries the handles and the comparison).
"""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib(ext):
    from orcasaq2 import comm
    return comm._bind(ext.lib())


def _alloc(L, nbytes):
    p, h = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    assert L.exl3_comm_alloc(nbytes, ctypes.byref(p), h) == 0
    return p.value


def _status(L, buf):
    w = ctypes.c_uint(0)
    assert L.exl3_comm_status(buf, ctypes.byref(w)) == 0
    return w.value


def _call(L, ptrs, rank, world, nbytes, t, out, limit):
    return L.exl3_allreduce_oneshot(ptrs, rank, world, nbytes, t.data_ptr(), out.data_ptr(), t.numel(), limit,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("n", [5120, 64 * 5120, 8, 4096 + 8])
def test_two_ranks_played_in_turn_and_a_wait_that_runs_out(ext, n):
    from orcasaq2 import comm
    L = _lib(ext)
    nbytes = L.exl3_allreduce_buffer_bytes(64 * 5120)
    bufs = [_alloc(L, nbytes), _alloc(L, nbytes)]
    ptrs = (ctypes.c_void_p * 8)(*bufs)
    g = torch.Generator().manual_seed(n)
    p = [torch.randn((n,), generator=g).half().cuda() for _ in range(2)]
    want = comm.allreduce_reference(p)
    try:
        out1 = torch.full((n,), 7.0, dtype=torch.half, device="cuda")
        assert _call(L, ptrs, 1, 2, nbytes, p[1], out1, 2000) == 0      # nobody has signalled: gives up after 2000 polls
        torch.cuda.synchronize()
        assert _status(L, bufs[1]) != 0 and _status(L, bufs[0]) == 0      # ... and says so; the context is still usable
        assert torch.all(out1 == 7.0)                                     # nothing was written
        out0 = torch.empty_like(out1)
        assert _call(L, ptrs, 0, 2, nbytes, p[0], out0, 1 << 20) == 0    # rank 1's signal and data are there
        assert _call(L, ptrs, 1, 2, nbytes, p[1], out1, 1 << 20) == 0    # and now rank 0's are too
        torch.cuda.synchronize()
        assert torch.equal(out0, want) and torch.equal(out1, want)        # bitwise the same on both ranks
        assert _status(L, bufs[0]) == 0
        # a second generation (the other data slot), in place
        q = [(t.float() * 0.5 - 1.0).half() for t in p]
        want2 = comm.allreduce_reference(q)
        a, b = q[0].clone(), q[1].clone()
        assert _call(L, ptrs, 1, 2, nbytes, b, b, 2000) == 0              # runs out again: b keeps the partial
        torch.cuda.synchronize()
        assert torch.equal(b, q[1])
        assert _call(L, ptrs, 0, 2, nbytes, a, a, 1 << 20) == 0
        assert _call(L, ptrs, 1, 2, nbytes, b, b, 1 << 20) == 0
        torch.cuda.synchronize()
        assert torch.equal(a, want2) and torch.equal(b, want2)
    finally:
        torch.cuda.synchronize()
        for b_ in bufs:
            L.exl3_comm_free(b_)


def test_single_rank_and_argument_checks(ext):
    L = _lib(ext)
    nbytes = L.exl3_allreduce_buffer_bytes(8192)
    buf = _alloc(L, nbytes)
    ptrs = (ctypes.c_void_p * 8)(buf)
    t = torch.randn(8192).half().cuda()
    try:
        out = torch.empty_like(t)
        assert _call(L, ptrs, 0, 1, nbytes, t, out, 0) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, t)
        assert _call(L, ptrs, 0, 1, nbytes, t[:12], out[:12], 0) == -1          # not a multiple of 8
        assert _call(L, ptrs, 1, 1, nbytes, t, out, 0) == -1                      # rank outside the group
        assert _call(L, ptrs, 0, 9, nbytes, t, out, 0) == -1                      # more ranks than the kernel serves
        big = torch.zeros(16384, dtype=torch.half, device="cuda")
        assert _call(L, ptrs, 0, 1, nbytes, big, big, 0) == -5                    # more values than the buffer holds
        assert _call(L, ptrs, 0, 1, nbytes, t[4:4 + 8184], out[:8184], 0) == -2   # misaligned input
        assert L.exl3_allreduce_oneshot(None, 0, 1, nbytes, t.data_ptr(), out.data_ptr(), 8192, 0, None) == -6
    finally:
        torch.cuda.synchronize()
        L.exl3_comm_free(buf)


@pytest.mark.parametrize("world", [3, 4, 8])
@pytest.mark.parametrize("n", [5120, 48 * 5120])
def test_more_ranks_played_in_turn(ext, world, n):
    """The same on one GPU with 3, 4 and 8 ranks (both forms of the exchange): ranks world-1 .. 1 go first and give
    up (each has published its partial and signalled everybody), rank 0 then finds everything and completes, and
    the others complete when called again.  Every rank must produce the same bytes."""
    from orcasaq2 import comm
    L = _lib(ext)
    nbytes = L.exl3_allreduce_buffer_bytes(64 * 5120)
    bufs = [_alloc(L, nbytes) for _ in range(world)]
    ptrs = (ctypes.c_void_p * 8)(*bufs)
    g = torch.Generator().manual_seed(n + world)
    p = [torch.randn((n,), generator=g).half().cuda() for _ in range(world)]
    want = comm.allreduce_reference(p)
    outs = [torch.full((n,), 7.0, dtype=torch.half, device="cuda") for _ in range(world)]
    try:
        for gen in range(3):                                              # three generations: both slots and a reuse
            for r in range(world - 1, 0, -1):
                assert _call(L, ptrs, r, world, nbytes, p[r], outs[r], 500) == 0
            torch.cuda.synchronize()
            assert all(torch.all(o == 7.0) for o in outs[1:])             # nobody could finish yet
            assert all(_status(L, b) != 0 for b in bufs[1:]) and _status(L, bufs[0]) == 0
            for r in range(world):
                assert _call(L, ptrs, r, world, nbytes, p[r], outs[r], 1 << 20) == 0
            torch.cuda.synchronize()
            for o in outs:
                assert torch.equal(o, want)
            p = [(t.float() * 0.75 + 0.125 * (gen + 1)).half() for t in p]
            want = comm.allreduce_reference(p)
            for o in outs:
                o.fill_(7.0)
    finally:
        torch.cuda.synchronize()
        for b_ in bufs:
            L.exl3_comm_free(b_)


_CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from orcasaq2 import comm
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
ar = comm.OneShotAllReduce(max_values=64 * 5120)
ok = True
for it, n in enumerate([5120, 64 * 5120, 5120, 8, 32 * 5120, 5120]):
    p = torch.randn((n,), generator=torch.Generator().manual_seed(100 * it + rank)).half().cuda()
    parts = [torch.empty_like(p) for _ in range(world)]
    dist.all_gather(parts, p)
    want = comm.allreduce_reference(parts)
    got = ar.all_reduce(p.clone())
    torch.cuda.synchronize()
    ok = ok and torch.equal(got, want)
# replayed from a CUDA graph: generations and slots advance on the device
x = torch.randn((5120,), generator=torch.Generator().manual_seed(rank)).half().cuda()
y = torch.empty_like(x)
s = torch.cuda.Stream()
s.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(s):
    ar.all_reduce(x, y); torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        ar.all_reduce(x, y)
torch.cuda.current_stream().wait_stream(s)
parts = [torch.empty_like(x) for _ in range(world)]
dist.all_gather(parts, x)
want = comm.allreduce_reference(parts)
for _ in range(7):
    y.zero_(); g.replay(); torch.cuda.synchronize()
    ok = ok and torch.equal(y, want)
ok = ok and ar.status() == 0
t = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(t, op=dist.ReduceOp.MIN)
torch.cuda.synchronize(); dist.barrier()
if rank == 0:
    print("ALLREDUCE_OK" if int(t.item()) == 1 else "ALLREDUCE_MISMATCH", flush=True)
sys.stdout.flush()
os._exit(0)
"""


@pytest.mark.parametrize("world", [2, 4, 8])
def test_real_exchange_between_processes(ext, world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    pkg = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "orcasaq2-kernel_b200")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), str(script), pkg],
                       capture_output=True, text=True, timeout=300, env=env)
    assert "ALLREDUCE_OK" in p.stdout, (p.stdout[-2000:], p.stderr[-3000:])
