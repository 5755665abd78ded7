"""One-shot all-reduce over peer memory for the partial outputs of row-parallel EXL3 layers.

The reference plugin refuses tensor parallelism outright (orcasaq2/config.py:173-177); with it enabled, every
row-parallel projection (o_proj, down_proj) ends in an all-reduce of a [rows, hidden] fp16 tensor
(vllm/model_executor/layers/linear.py:1556-1559) -- 10 KB to 640 KB at decode batch sizes, 128 of them per
token on a 64-layer model.  That is latency, not bandwidth, so instead of a library collective this module
drives `exl3_allreduce_oneshot`: one kernel launch in which every rank publishes its partial in a buffer its
peers have mapped, signals them, waits (with a bound) for their signals and adds all partials in rank order with
plain peer loads.  All ranks obtain bitwise the same sum.

Set-up exchanges CUDA IPC handles through the process group (any backend); the kernels use plain loads and
stores on peer memory only.  There is no fallback: if the buffers cannot be mapped, construction raises.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _ext

MAX_RANKS = 8


def allreduce_reference(partials):
    """What every rank must end up with: the partials added in fp32 in rank order, rounded to fp16 once."""
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:
        acc = acc + p.float()
    return acc.half()


def _bind(L):
    vp, ci, sz, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_longlong
    if getattr(L, "_exl3_comm_bound", False):
        return L
    L.exl3_allreduce_buffer_bytes.restype = sz
    L.exl3_allreduce_buffer_bytes.argtypes = [sz]
    L.exl3_allreduce_oneshot.restype = ci
    L.exl3_allreduce_oneshot.argtypes = [ctypes.POINTER(vp), ci, ci, sz, vp, vp, ll, ci, vp]
    L.exl3_comm_alloc.restype = ci
    L.exl3_comm_alloc.argtypes = [sz, ctypes.POINTER(vp), ctypes.c_char_p]
    L.exl3_comm_open.restype = ci
    L.exl3_comm_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    for name in ("exl3_comm_close", "exl3_comm_free"):
        getattr(L, name).restype = ci
        getattr(L, name).argtypes = [vp]
    L.exl3_comm_status.restype = ci
    L.exl3_comm_status.argtypes = [vp, ctypes.POINTER(ctypes.c_uint)]
    L._exl3_comm_bound = True
    return L


class OneShotAllReduce:
    """All-reduce of fp16 tensors of up to `max_values` elements among the ranks of `group` (one GPU each, one node).

    `all_reduce(t)` sums `t` in place on the current stream; it can be captured in a CUDA graph (the buffer slot
    and the generation are chosen on the device).  Every rank must make the same calls in the same order."""

    def __init__(self, group=None, max_values: int = 64 * 5120, device=None, spin_limit: int = 0):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if not 1 <= self.world <= MAX_RANKS:
            raise RuntimeError(f"one-shot all-reduce serves 1..{MAX_RANKS} ranks, got {self.world}")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.spin_limit = int(spin_limit)
        self.L = _bind(_ext.lib())
        self.max_values = int(max_values)
        self.nbytes = int(self.L.exl3_allreduce_buffer_bytes(self.max_values))
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _ext._check(self.L.exl3_comm_alloc(self.nbytes, ctypes.byref(own), handle), "exl3_comm_alloc")
            self.own = own.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.opened = []
            ptrs = (ctypes.c_void_p * MAX_RANKS)()
            for r in range(self.world):
                if r == self.rank:
                    ptrs[r] = self.own
                    continue
                p = ctypes.c_void_p()
                _ext._check(self.L.exl3_comm_open(handles[r], ctypes.byref(p)), f"exl3_comm_open(rank {r})")
                self.opened.append(p.value)
                ptrs[r] = p.value
            self.ptrs = ptrs
        dist.barrier(group=group)              # every buffer is zeroed and mapped before anyone's first signal

    def all_reduce(self, t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        out = t if out is None else out
        for x, name in ((t, "input"), (out, "output")):
            if x.device != self.device or x.dtype != torch.float16 or not x.is_contiguous():
                raise RuntimeError(f"one-shot all-reduce: {name} must be a contiguous fp16 tensor on {self.device}")
        n = t.numel()
        if n % 8 or n > self.max_values or out.numel() != n:
            raise RuntimeError(f"one-shot all-reduce: {n} values (need a multiple of 8, at most {self.max_values})")
        _ext._check(self.L.exl3_allreduce_oneshot(self.ptrs, self.rank, self.world, self.nbytes, t.data_ptr(),
                                                  out.data_ptr(), n, self.spin_limit, _ext._stream(t)),
                    "exl3_allreduce_oneshot")
        return out

    def status(self) -> int:
        """Sticky status word of this rank's buffer: non-zero after a bounded wait ran out (waits for the device)."""
        w = ctypes.c_uint(0)
        with torch.cuda.device(self.device):
            _ext._check(self.L.exl3_comm_status(self.own, ctypes.byref(w)), "exl3_comm_status")
        return int(w.value)

    def close(self):
        """Unmap the peers' buffers and free the own one; collective (no rank may still be inside a call)."""
        if getattr(self, "own", None) is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self.opened:
                self.L.exl3_comm_close(p)
            dist.barrier(group=self.group)
            self.L.exl3_comm_free(self.own)
        self.own, self.opened = None, []
