"""CPU oracle for the EXL3 linear-layer path (numpy / PyTorch-CPU form).  TEST INFRASTRUCTURE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
module; the shipped package never does, and it fails loudly without its CUDA library.

PARITY UNPINNED for the trellis decode: the reference forwards the decode to the
exllamav3 v1.5.1 extension (docker/Dockerfile:20,31-38), which is not part of the reference
tree, and the tree holds no test or golden vector for it.  The decode here restates the
published QTIP "3INST" codebook (arXiv 2406.11235) on this repository's packing
conventions (the same ones `exl3_oracle.c` states in its header).  Everything the reference
tree does pin is followed and is checked against fixtures generated from the reference's own
Python (tests/golden/make_golden.py):

  pipeline order            orcasaq2/ops.py:44-60
  Hadamard `_had`, `_t128`  orcasaq2/__init__.py:33-46
  deploy weight             orcasaq2/__init__.py:49-61
  exl3_K                    orcasaq2/ops.py:28-34
  int8 embedding / head     orcasaq2/heads.py:61-75, orcasaq2/patches/int8_embedding.py:40-43

Two forms live here: `*_np` functions (numpy, integer-exact, the readable statement of the
format) and `torch_*` functions (vectorised PyTorch on CPU: "the reference's CPU PyTorch
path" that the benchmark times).  `COracle` loads the C/OpenMP restatement for large shapes.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

BLOCK = 128
MUL, ADD, MASK, XOR = 89226354, 64248484, 0x8FFF8FFF, 0x3B603B60

_HERE = os.path.dirname(os.path.abspath(__file__))


# ----------------------------------------------------------------------------- format
def tile_perm():
    """(rows[256], cols[256]): position of sequence index t inside its 16x16 tile."""
    t = np.arange(256)
    c, i = t >> 5, t & 31
    p, q = c >> 2, c & 3
    r = 8 * ((i >> 2) & 1) + 4 * ((i >> 1) & 1) + q
    col = 4 * (i >> 3) + 2 * (i & 1) + p
    return r.astype(np.int64), col.astype(np.int64)


def decode_state_np(state):
    """uint16 states -> fp16 weights (3INST): one 32-bit multiply-add, one mask-xor, one
    fp16 add of the two halves."""
    s = np.asarray(state).astype(np.uint64) & 0xFFFF
    z = (s * MUL + ADD) & 0xFFFFFFFF
    z = (z & MASK) ^ XOR
    lo = (z & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    hi = (z >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    return (lo + hi).astype(np.float16)       # exact fp32 sum, one RN-even rounding


def tile_states_np(trellis_u16, K):
    """[..., 16K] uint16 -> [..., 256] states (sequence order)."""
    u = np.asarray(trellis_u16).astype(np.uint32)
    nwords = 16 * K
    assert u.shape[-1] == nwords
    n = np.arange(256) * K
    q, o = n >> 4, (n & 15).astype(np.uint32)
    v = u[..., q] | (u[..., (q + 1) % nwords] << 16)
    return ((v >> o) & 0xFFFF).astype(np.uint16)


def exl3_K(trellis):
    """orcasaq2/ops.py:28-34."""
    k = trellis.shape[-1] / 16
    return int(k) if float(k).is_integer() else k


def reconstruct_np(trellis_i16):
    """trellis [ic/16, oc/16, 16K] (int16 bit patterns) -> inner weight [ic, oc] fp16."""
    tr = np.asarray(trellis_i16).view(np.uint16)
    ti, tj, nw = tr.shape
    K = nw // 16
    assert nw == 16 * K
    vals = decode_state_np(tile_states_np(tr, K))            # [ti, tj, 256]
    r, c = tile_perm()
    w = np.empty((ti, tj, 16, 16), np.float16)
    w[:, :, r, c] = vals
    return w.transpose(0, 2, 1, 3).reshape(ti * 16, tj * 16)


# ----------------------------------------------------------------------------- Hadamard
def had128_matrix(dtype=np.float64):
    h = np.array([[1.0]])
    while h.shape[0] < BLOCK:
        h = np.block([[h, h], [h, -h]])
    return (h / np.sqrt(BLOCK)).astype(dtype)


def t128_np(x):
    """Blockwise 128-Hadamard along the last dim (orcasaq2/__init__.py:43-46), float64."""
    x = np.asarray(x, np.float64)
    s = x.shape
    return (x.reshape(*s[:-1], s[-1] // BLOCK, BLOCK) @ had128_matrix()).reshape(s)


def had_r_128_np(x_f16, pre=None, post=None, scale=1.0):
    v = np.asarray(x_f16, np.float16).astype(np.float64)
    if pre is not None:
        v = v * np.asarray(pre, np.float16).astype(np.float64)
    v = t128_np(v)
    if post is not None:
        v = v * np.asarray(post, np.float16).astype(np.float64)
    return (v * scale).astype(np.float32).astype(np.float16)


def layer_np(x_f16, w_f16, suh, svh):
    """y = (((x*suh) H) W) H * svh in float64 from fp16 inputs (no intermediate rounding)."""
    x = np.asarray(x_f16).astype(np.float64) * np.asarray(suh).astype(np.float64)
    y = t128_np(x) @ np.asarray(w_f16).astype(np.float64)
    return t128_np(y) * np.asarray(svh).astype(np.float64)


def deploy_weight_np(w_f16, suh, svh):
    """[oc, ic] deploy weight, the algebra of orcasaq2/__init__.py:58-61 in float64."""
    w = np.asarray(w_f16).astype(np.float64)
    w = t128_np(w.T).T * np.asarray(suh).astype(np.float64)[:, None]
    w = t128_np(w) * np.asarray(svh).astype(np.float64)[None, :]
    return w.T


# ----------------------------------------------------------------------------- int8 paths
def int8_embed_torch(q, s, ids):
    """orcasaq2/heads.py:61-67: gather, cast, scale on the gathered rows."""
    rows = q[ids].to(s.dtype)
    return rows * s.reshape(-1, 1)[ids]


def int8_head_torch(q, s, x):
    """orcasaq2/heads.py:69-75: dequantise the table to x.dtype, then a linear."""
    w = q.to(x.dtype) * s.reshape(-1, 1).to(x.dtype)
    return torch.nn.functional.linear(x.float(), w.to(x.dtype).float())


# ----------------------------------------------------------------------------- torch CPU path
_TORCH_HAD = {}


def _torch_had(dtype):
    if dtype not in _TORCH_HAD:
        _TORCH_HAD[dtype] = torch.from_numpy(had128_matrix()).to(dtype)
    return _TORCH_HAD[dtype]


def torch_t128(x):
    s = x.shape
    return (x.reshape(*s[:-1], s[-1] // BLOCK, BLOCK) @ _torch_had(x.dtype)).reshape(s)


def torch_reconstruct(trellis_i16):
    """Vectorised PyTorch-CPU decode: trellis int16 [ti, tj, 16K] -> [ic, oc] fp16."""
    ti, tj, nw = trellis_i16.shape
    K = nw // 16
    u = trellis_i16.to(torch.int64) & 0xFFFF
    n = torch.arange(256) * K
    q, o = n >> 4, n & 15
    v = u[..., q] | (u[..., (q + 1) % nw] << 16)
    st = (v >> o) & 0xFFFF
    z = (st * MUL + ADD) & 0xFFFFFFFF
    z = (z & MASK) ^ XOR
    lo = (z & 0xFFFF).to(torch.int32).to(torch.int16).view(torch.float16)
    hi = (z >> 16).to(torch.int32).to(torch.int16).view(torch.float16)
    vals = (lo.float() + hi.float()).half()
    r, c = tile_perm()
    w = torch.empty((ti, tj, 16, 16), dtype=torch.float16)
    w[:, :, torch.from_numpy(r), torch.from_numpy(c)] = vals
    return w.permute(0, 2, 1, 3).reshape(ti * 16, tj * 16).contiguous()


def torch_layer(x, trellis_i16, suh, svh):
    """The reference pipeline on CPU: decode -> Hadamard(x*suh) -> matmul -> Hadamard * svh
    (orcasaq2/ops.py:53-59 with each extension call replaced by its CPU restatement).
    fp16 inputs, fp32 arithmetic, fp16 result."""
    w = torch_reconstruct(trellis_i16).float()
    xh = torch_t128(x.float() * suh.float())
    y = xh @ w
    return (torch_t128(y) * svh.float()).half()


# ----------------------------------------------------------------------------- C oracle
class COracle:
    """ctypes view of libexl3_oracle.so (built from exl3_oracle.c by oracle/Makefile)."""

    def __init__(self, build=True):
        so = os.path.join(_HERE, "libexl3_oracle.so")
        if not os.path.exists(so) and build:
            subprocess.check_call(["make", "-C", _HERE, "-s"])
        self.lib = ctypes.CDLL(so)
        self.lib.exl3_oracle_decode_state.restype = ctypes.c_uint16
        self.lib.exl3_oracle_decode_state.argtypes = [ctypes.c_uint32]

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    def decode_state(self, s):
        return np.array([self.lib.exl3_oracle_decode_state(int(s))], np.uint16).view(np.float16)[0]

    def tile_states(self, tile_u16, K):
        tile = np.ascontiguousarray(tile_u16, np.uint16)
        out = np.empty(256, np.uint16)
        self.lib.exl3_oracle_tile_states(self._p(tile), ctypes.c_int(K), self._p(out))
        return out

    def tile_perm(self):
        r, c = np.empty(256, np.int32), np.empty(256, np.int32)
        self.lib.exl3_oracle_tile_perm(self._p(r), self._p(c))
        return r, c

    def reconstruct(self, trellis_i16):
        tr = np.ascontiguousarray(np.asarray(trellis_i16)).view(np.uint16)
        ti, tj, nw = tr.shape
        w = np.empty((ti * 16, tj * 16), np.uint16)
        rc = self.lib.exl3_oracle_reconstruct(self._p(tr), ti * 16, tj * 16, nw // 16, self._p(w))
        if rc:
            raise RuntimeError(f"exl3_oracle_reconstruct: {rc}")
        return w.view(np.float16)

    def had_r_128(self, x_f16, pre=None, post=None, scale=1.0):
        x = np.ascontiguousarray(x_f16, np.float16)
        rows, n = x.reshape(-1, x.shape[-1]).shape
        out = np.empty_like(x)
        pre = None if pre is None else np.ascontiguousarray(pre, np.float16)
        post = None if post is None else np.ascontiguousarray(post, np.float16)
        rc = self.lib.exl3_oracle_had_r_128(
            self._p(x), self._p(out), None if pre is None else self._p(pre),
            None if post is None else self._p(post), ctypes.c_float(scale), rows, n)
        if rc:
            raise RuntimeError(f"exl3_oracle_had_r_128: {rc}")
        return out

    def layer(self, x_f16, w_f16, suh, svh):
        x = np.ascontiguousarray(x_f16, np.float16)
        w = np.ascontiguousarray(w_f16, np.float16)
        suh = np.ascontiguousarray(suh, np.float16)
        svh = np.ascontiguousarray(svh, np.float16)
        rows, ic = x.shape
        oc = w.shape[1]
        y = np.empty((rows, oc), np.float32)
        rc = self.lib.exl3_oracle_layer(self._p(x), rows, self._p(w), ic, oc, self._p(suh),
                                        self._p(svh), self._p(y))
        if rc:
            raise RuntimeError(f"exl3_oracle_layer: {rc}")
        return y

    def hgemm(self, a_f16, w_f16):
        a = np.ascontiguousarray(a_f16, np.float16)
        w = np.ascontiguousarray(w_f16, np.float16)
        y = np.empty((a.shape[0], w.shape[1]), np.float16)
        rc = self.lib.exl3_oracle_hgemm(self._p(a), self._p(w), self._p(y), a.shape[0],
                                        a.shape[1], w.shape[1])
        if rc:
            raise RuntimeError(f"exl3_oracle_hgemm: {rc}")
        return y

    def int8_embed(self, q, s_bits, ids, is_bf16):
        q = np.ascontiguousarray(q, np.int8)
        s = np.ascontiguousarray(s_bits, np.uint16).reshape(-1)
        ids = np.ascontiguousarray(ids, np.int64).reshape(-1)
        out = np.empty((ids.size, q.shape[1]), np.uint16)
        rc = self.lib.exl3_oracle_int8_embed(self._p(q), self._p(s), self._p(ids), ids.size,
                                             q.shape[0], q.shape[1], int(is_bf16), self._p(out))
        if rc:
            raise RuntimeError(f"exl3_oracle_int8_embed: {rc}")
        return out

    def int8_head(self, q, s_bits, x_bits, is_bf16):
        q = np.ascontiguousarray(q, np.int8)
        s = np.ascontiguousarray(s_bits, np.uint16).reshape(-1)
        x = np.ascontiguousarray(x_bits, np.uint16)
        out = np.empty((x.shape[0], q.shape[0]), np.float32)
        rc = self.lib.exl3_oracle_int8_head(self._p(q), self._p(s), self._p(x), x.shape[0],
                                            q.shape[0], q.shape[1], int(is_bf16), self._p(out))
        if rc:
            raise RuntimeError(f"exl3_oracle_int8_head: {rc}")
        return out


# ----------------------------------------------------------------------------- synthetic inputs
def make_layer(seed, ic, oc, K, rows, act_dtype=torch.float16):
    """Seeded synthetic EXL3 layer: uniform-random uint16 trellis words, +-1 sign vectors,
    N(0,1) activations."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    tr = torch.randint(0, 65536, (ic // 16, oc // 16, 16 * K), generator=g, dtype=torch.int32)
    tr = tr.to(torch.int16)        # keeps the low 16 bits: uint16 bit patterns in int16
    suh = (torch.randint(0, 2, (ic,), generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (oc,), generator=g) * 2 - 1).to(torch.float16)
    x = torch.randn((rows, ic), generator=g).to(act_dtype)
    return tr, suh, svh, x


def make_int8_table(seed, vocab, hidden, dtype=torch.float16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randint(-127, 128, (vocab, hidden), generator=g, dtype=torch.int32).to(torch.int8)
    s = (torch.rand((vocab,), generator=g) * 0.02 + 1e-3).to(dtype)
    return q, s
