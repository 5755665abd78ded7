"""The C-ABI library loads and exports every function declared in include/exl3_b200.h; argument
checks that run before any CUDA call are exercised here without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "exl3_b200.h")
LIB = os.path.join(ROOT, "orcasaq2-kernel_b200", "orcasaq2", "libexl3_b200.so")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        import __graft_entry__
        __graft_entry__.build()
    return ctypes.CDLL(LIB)


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(exl3_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert {"exl3_reconstruct", "exl3_had_r_128", "exl3_gemv_grouped", "exl3_gemv",
            "exl3_int8_embed", "exl3_int8_head", "exl3_strerror"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n


def test_version_and_strerror(lib):
    lib.exl3_strerror.restype = ctypes.c_char_p
    assert lib.exl3_abi_version() >= 1
    for code in range(0, -7, -1):
        assert lib.exl3_strerror(code)
    assert b"unknown" in lib.exl3_strerror(-99)


def test_argument_checks_without_gpu(lib):
    vp = ctypes.c_void_p
    lib.exl3_reconstruct.argtypes = [vp, vp] + [ctypes.c_int] * 5 + [vp]
    assert lib.exl3_reconstruct(None, None, 128, 128, 8, 0, 0, None) == -6          # NULL
    fake = vp(4096)     # never dereferenced: these calls fail validation first
    assert lib.exl3_reconstruct(fake, fake, 100, 128, 8, 0, 0, None) == -1           # shape
    assert lib.exl3_reconstruct(fake, fake, 128, 128, 7, 0, 0, None) == -3           # K = 3.5
    assert lib.exl3_reconstruct(fake, fake, 128, 128, 8, 1, 0, None) == -3           # mcg
    assert lib.exl3_reconstruct(vp(4100), fake, 128, 128, 8, 0, 0, None) == -2       # alignment
    lib.exl3_had_r_128.argtypes = [vp, vp, vp, vp, ctypes.c_float, ctypes.c_int, ctypes.c_int, vp]
    assert lib.exl3_had_r_128(fake, fake, None, None, 1.0, 1, 100, None) == -1
    assert lib.exl3_had_r_128(fake, fake, None, None, 1.0, 0, 128, None) == 0         # empty input


def test_gemv_plan_and_workspace(lib):
    class Shard(ctypes.Structure):
        _fields_ = [("trellis", ctypes.c_void_p), ("suh", ctypes.c_void_p), ("svh", ctypes.c_void_p),
                    ("oc", ctypes.c_int), ("k2", ctypes.c_int), ("mcg", ctypes.c_int),
                    ("mul1", ctypes.c_int), ("out_col", ctypes.c_int)]
    lib.exl3_gemv_workspace_bytes.restype = ctypes.c_size_t
    lib.exl3_gemv_workspace_bytes.argtypes = [ctypes.POINTER(Shard), ctypes.c_int, ctypes.c_int, ctypes.c_int]
    vp = ctypes.c_void_p
    lib.exl3_gemv_grouped.argtypes = [ctypes.POINTER(Shard), ctypes.c_int, vp, vp, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, vp, ctypes.c_size_t, vp]
    arr = (Shard * 3)(Shard(4096, 4096, 4096, 6144, 8, 0, 0, 0), Shard(4096, 4096, 4096, 1024, 10, 0, 0, 6144),
                      Shard(4096, 4096, 4096, 1024, 12, 0, 0, 7168))
    need = lib.exl3_gemv_workspace_bytes(arr, 3, 16, 5120)
    assert 256 < need < 64 << 20 and need % 4 == 0
    assert lib.exl3_gemv_workspace_bytes(arr, 3, 17, 5120) == 0      # too many rows
    assert lib.exl3_gemv_workspace_bytes(arr, 3, 1, 5000) == 0       # ic not a multiple of 128
    fake = vp(4096)
    assert lib.exl3_gemv_grouped(arr, 3, fake, fake, 1, 5120, 8192, None, 0, None) == -5    # no workspace
    assert lib.exl3_gemv_grouped(arr, 3, fake, fake, 1, 5120, 4096, fake, 1 << 30, None) == -1  # ldy too small
    arr[1].mul1 = 1
    assert lib.exl3_gemv_grouped(arr, 3, fake, fake, 1, 5120, 8192, fake, 1 << 30, None) == -3


def test_decode_attn_argument_checks(lib):
    vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.exl3_decode_attn_workspace_bytes.restype = ctypes.c_size_t
    lib.exl3_decode_attn_workspace_bytes.argtypes = [ci] * 4
    lib.exl3_decode_attn.argtypes = [vp] * 5 + [ctypes.c_size_t] + [ci] * 5 + [ll] * 4 + [ctypes.c_float, vp]
    assert lib.exl3_decode_attn_workspace_bytes(1, 24, 4, 4096) > 0           # one sequence is split
    assert lib.exl3_decode_attn_workspace_bytes(512, 24, 4, 4096) == 0        # enough sequences: no split
    assert lib.exl3_decode_attn_workspace_bytes(1, 24, 5, 4096) == 0          # heads do not divide
    fake = vp(4096)
    args = lambda **kw: [kw.get("q", fake), fake, fake, fake, None, 0, kw.get("B", 512), kw.get("qh", 24),
                         kw.get("kvh", 4), kw.get("hd", 256), kw.get("L", 64), 24 * 256, 24 * 256,
                         4 * 64 * 256, kw.get("hs", 64 * 256), 0.0625, None]
    assert lib.exl3_decode_attn(*args(q=None)) == -6
    assert lib.exl3_decode_attn(*args(hd=128)) == -3
    assert lib.exl3_decode_attn(*args(qh=40)) == -3                           # ten query heads per KV head
    assert lib.exl3_decode_attn(*args(qh=25)) == -1
    assert lib.exl3_decode_attn(*args(L=0)) == -1
    assert lib.exl3_decode_attn(*args(hs=63 * 256)) == -1                     # head stride shorter than seq_len rows
    assert lib.exl3_decode_attn(*args(B=1, L=4096, hs=4096 * 256)) == -5                     # split, but no workspace


def test_decode_attn_fp8_argument_checks(lib):
    vp, ci, ll, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.exl3_decode_attn_fp8_workspace_bytes.restype = ctypes.c_size_t
    lib.exl3_decode_attn_fp8_workspace_bytes.argtypes = [ci] * 4
    lib.exl3_decode_attn_fp8.argtypes = [vp] * 5 + [ctypes.c_size_t] + [ci] * 5 + [ll] * 4 + [cf, cf, cf, vp]
    lib.exl3_rope_append_fp8.argtypes = [vp, ci, vp, vp, ci, vp, vp] + [ci] * 5 + [ll, ll, cf, cf, vp]
    assert lib.exl3_decode_attn_fp8_workspace_bytes(1, 24, 4, 4096) > lib.exl3_decode_attn_workspace_bytes(1, 24, 4, 4096)
    fake = vp(4096)
    args = lambda **kw: [kw.get("q", fake), fake, fake, fake, None, 0, 512, 24, 4, kw.get("hd", 256), 64, 24 * 256,
                         24 * 256, 4 * 64 * 256, kw.get("hs", 64 * 256), 0.0625, kw.get("ks", 1.0), kw.get("vs", 1.0), None]
    assert lib.exl3_decode_attn_fp8(*args(q=None)) == -6
    assert lib.exl3_decode_attn_fp8(*args(hd=128)) == -3
    assert lib.exl3_decode_attn_fp8(*args(hs=64 * 256 + 8)) == -1             # byte strides must be multiples of 16
    assert lib.exl3_decode_attn_fp8(*args(ks=0.0)) == -1
    assert lib.exl3_decode_attn_fp8(*args(vs=-1.0)) == -1
    assert lib.exl3_rope_append_fp8(fake, 32 * 256, fake, fake, 0, fake, fake, 1, 24, 4, 256, 3, 4 * 64 * 256, 64 * 256,
                                    0.0, 1.0, None) == -1
    assert lib.exl3_rope_append_fp8(fake, 32 * 256, fake, None, 0, fake, fake, 1, 24, 4, 256, 3, 4 * 64 * 256, 64 * 256,
                                    1.0, 1.0, None) == -6


def test_decode_attn_paged_argument_checks(lib):
    vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.exl3_decode_attn_paged.argtypes = [vp] * 7 + [ctypes.c_size_t] + [ci] * 7 + [ll] * 5 + [ctypes.c_float, vp]
    fake = vp(4096)

    def call(**kw):
        return lib.exl3_decode_attn_paged(kw.get("q", fake), fake, fake, kw.get("bt", fake), None, fake, None, 0,
                                          512, kw.get("qh", 24), 4, kw.get("hd", 256), kw.get("L", 64),
                                          kw.get("page", 32), kw.get("bts", 2), 24 * 256, 24 * 256, 4 * 32 * 256,
                                          32 * 256, kw.get("ts", 256), 0.0625, None)
    assert call(bt=None) == -6
    assert call(hd=64) == -3
    assert call(qh=36) == -3
    assert call(page=24) == -1                 # not a multiple of 16
    assert call(L=65) == -1                    # three pages needed, the table holds two per sequence
    assert call(ts=100) == -1
