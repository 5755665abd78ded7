"""Stand-in for `exllamav3.ext.exllamav3_ext`: the same positional entry points the plugin
calls (orcasaq2/ops.py:47-59 and orcasaq2/__init__.py:57 of the reference), bound with ctypes
to this package's sm_100a library `libexl3_b200.so` (C ABI in include/exl3_b200.h).

There is no CPU path and no fallback: a missing library or a non-CUDA tensor raises.
PyTorch is used only for device memory and the current stream.
"""
from __future__ import annotations

import ctypes
import os
import threading
import warnings

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libexl3_b200.so")
_lib = None
_lock = threading.Lock()

MAX_SHARDS = 8
GEMV_MAX_ROWS = 16


class Exl3Shard(ctypes.Structure):
    _fields_ = [("trellis", ctypes.c_void_p), ("suh", ctypes.c_void_p), ("svh", ctypes.c_void_p),
                ("oc", ctypes.c_int), ("k_times_2", ctypes.c_int), ("mcg", ctypes.c_int),
                ("mul1", ctypes.c_int), ("out_col", ctypes.c_int)]


class Exl3GemvFusion(ctypes.Structure):
    _fields_ = [("in_mode", ctypes.c_int), ("norm_weight", ctypes.c_void_p), ("eps", ctypes.c_float),
                ("ldx", ctypes.c_int), ("residual", ctypes.c_void_p), ("ld_residual", ctypes.c_int)]


IN_PLAIN, IN_RMSNORM, IN_SILU_MUL = 0, 1, 2


def library_path() -> str:
    return _LIB_PATH


def lib():
    """Load the CUDA library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(_LIB_PATH):
                    raise RuntimeError(
                        f"{_LIB_PATH} is missing: build it with `python build.py` in "
                        f"{os.path.dirname(_HERE)} (needs nvcc, sm_100a). There is no CPU fallback.")
                L = ctypes.CDLL(_LIB_PATH)
                vp, ci, cf, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
                L.exl3_abi_version.restype = ci
                L.exl3_strerror.restype = ctypes.c_char_p
                L.exl3_strerror.argtypes = [ci]
                L.exl3_reconstruct.argtypes = [vp, vp, ci, ci, ci, ci, ci, vp]
                L.exl3_had_r_128.argtypes = [vp, vp, vp, vp, cf, ci, ci, vp]
                L.exl3_gemv_workspace_bytes.restype = sz
                L.exl3_gemv_workspace_bytes.argtypes = [ctypes.POINTER(Exl3Shard), ci, ci, ci]
                L.exl3_gemv_grouped.argtypes = [ctypes.POINTER(Exl3Shard), ci, vp, vp, ci, ci, ci, vp, sz, vp]
                L.exl3_gemv.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp, sz, vp]
                L.exl3_gemv_grouped_ex.argtypes = [ctypes.POINTER(Exl3Shard), ci, vp, vp, ci, ci, ci, vp, sz,
                                                   ctypes.POINTER(Exl3GemvFusion), vp]
                L.exl3_gemv_grouped_ex.restype = ci
                ll = ctypes.c_longlong
                L.exl3_int8_embed.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp]
                L.exl3_int8_head.argtypes = [vp, vp, vp, vp, ci, ci, ci, ll, ci, vp]
                L.exl3_gemm_tc.argtypes = [vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ci, ci, vp]
                L.exl3_gemm_tc_scratch_bytes.restype = sz
                L.exl3_gemm_tc_scratch_bytes.argtypes = [ci, ci, ci]
                L.exl3_gemm_tc.restype = ci
                L.exl3_gemm_tc_ex.argtypes = [vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ci, ci, ci,
                                              ctypes.POINTER(Exl3GemvFusion), vp]
                L.exl3_gemm_tc_ex.restype = ci
                L.exl3_gemm_tc_grouped_scratch_bytes.restype = sz
                L.exl3_gemm_tc_grouped_scratch_bytes.argtypes = [ctypes.POINTER(Exl3Shard), ci, ci, ci]
                L.exl3_gemm_tc_grouped.argtypes = [ctypes.POINTER(Exl3Shard), ci, vp, vp, ci, ci, ci, vp, sz, ci,
                                                   ctypes.POINTER(Exl3GemvFusion), vp]
                L.exl3_gemm_tc_grouped.restype = ci
                L.exl3_gemm_tc_status.restype = ctypes.c_uint
                L.exl3_gemv_static_capacity.restype = sz
                L.exl3_gemv_grouped_static.argtypes = [ctypes.POINTER(Exl3Shard), ci, vp, vp, ci, ci, ci, vp]
                L.exl3_gemv_grouped_static.restype = ci
                L.exl3_gemv_static_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
                L.exl3_gemv_static_status.restype = ci
                L.exl3_decode_attn_workspace_bytes.restype = sz
                L.exl3_decode_attn_workspace_bytes.argtypes = [ci, ci, ci, ci]
                L.exl3_decode_attn.argtypes = [vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ll, ll, ll, ll, cf, vp]
                L.exl3_decode_attn.restype = ci
                L.exl3_decode_attn_paged.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ci, ci,
                                                     ll, ll, ll, ll, ll, cf, vp]
                L.exl3_decode_attn_paged.restype = ci
                L.exl3_rope_append.argtypes = [vp, ci, vp, vp, ci, vp, vp, ci, ci, ci, ci, ci, ll, ll, vp]
                L.exl3_rope_append.restype = ci
                L.exl3_decode_attn_fp8_workspace_bytes.restype = sz
                L.exl3_decode_attn_fp8_workspace_bytes.argtypes = [ci, ci, ci, ci]
                L.exl3_decode_attn_fp8.argtypes = [vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ll, ll, ll, ll, cf, cf, cf, vp]
                L.exl3_decode_attn_fp8.restype = ci
                L.exl3_decode_attn_paged_fp8.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ci, ci,
                                                         ll, ll, ll, ll, ll, cf, cf, cf, vp]
                L.exl3_decode_attn_paged_fp8.restype = ci
                L.exl3_rope_append_fp8.argtypes = [vp, ci, vp, vp, ci, vp, vp, ci, ci, ci, ci, ci, ll, ll, cf, cf, vp]
                L.exl3_rope_append_fp8.restype = ci
                for name in ("exl3_reconstruct", "exl3_had_r_128", "exl3_gemv_grouped", "exl3_gemv",
                             "exl3_int8_embed", "exl3_int8_head"):
                    getattr(L, name).restype = ci
                _lib = L
    return _lib


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what}: {lib().exl3_strerror(rc).decode()} ({rc})")


def _cuda(t: torch.Tensor, name: str, dtype=None):
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise RuntimeError(f"{name} must be a CUDA tensor (this build has no CPU path)")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise RuntimeError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    return t


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _k2(k) -> int:
    k2 = float(k) * 2.0
    if not k2.is_integer():
        raise RuntimeError(f"unsupported bitrate K={k}")
    return int(k2)


def _trellis_dims(trellis: torch.Tensor):
    if trellis.dim() != 3 or trellis.dtype not in (torch.int16, torch.uint16):
        raise RuntimeError("trellis must be a 3-D int16 tensor [ic/16, oc/16, 16*K]")
    return trellis.shape[0] * 16, trellis.shape[1] * 16, trellis.shape[2] / 16


# --------------------------------------------------------------------------- workspaces
# Scratch for the fused GEMV: rotated activations, partial sums of shared output blocks, arrival
# tickets, a status word.  One buffer per (device, stream), zero-filled when allocated; the kernels
# leave the tickets at zero.  The default size covers every launch of the 27B-class shapes at up to
# 16 rows, so the buffer made by `ensure_gemv_workspace` (called when a layer's weights are loaded)
# is the one every later launch uses and nothing is allocated under CUDA-graph capture.  A launch
# that does need more gets a new, larger buffer; the old one is kept alive, because graphs captured
# earlier still write to it.
GEMV_WORKSPACE_BYTES = 16 << 20
_workspaces: dict = {}
_retired: list = []


def gemv_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            # it still works (the buffer then lives in the graph's memory pool and its zero-fill is
            # replayed with the graph), but it ties the scratch to that graph: say so once
            warnings.warn(
                "orcasaq2: the fused GEMV is allocating its scratch buffer inside a CUDA-graph capture; "
                "call orcasaq2._ext.ensure_gemv_workspace(device) on the capturing stream before the "
                "capture (any warm-up call on that stream does it too)", RuntimeWarning, stacklevel=3)
        if ws is not None:
            _retired.append(ws)
        ws = torch.zeros(max(nbytes, GEMV_WORKSPACE_BYTES), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def ensure_gemv_workspace(device: torch.device, nbytes: int = 0) -> None:
    """Allocate (and zero) the GEMV scratch of the current stream of `device` now, outside of any
    capture, so that the first launch on that stream allocates nothing."""
    gemv_workspace(torch.device(device), nbytes)


def workspace_status(device: torch.device) -> int:
    """OR of the sticky device-side status words of this device's workspaces (0 = healthy)."""
    st = 0
    for (idx, _), ws in _workspaces.items():
        if idx == device.index:
            st |= int(ws[:4].view(torch.int32).item())
    return st


def gemv_static_status(device: torch.device) -> int:
    """Sticky status word of the built-in scratch that gemv_grouped_static uses on `device`."""
    word = ctypes.c_uint(0)
    with torch.cuda.device(device):
        _check(lib().exl3_gemv_static_status(ctypes.byref(word)), "exl3_gemv_static_status")
    return int(word.value)


# --------------------------------------------------------------------------- entry points
def reconstruct(w: torch.Tensor, trellis: torch.Tensor, k, mcg: bool, mul1: bool) -> None:
    """w[ic, oc] (fp16, out) <- decoded trellis.  ext.reconstruct, ops.py:56 of the reference."""
    _cuda(w, "w", torch.float16)
    _cuda(trellis, "trellis")
    ic, oc, kk = _trellis_dims(trellis)
    if float(k) != kk:
        raise RuntimeError("packed dimension 2 is incorrect size")
    if tuple(w.shape) != (ic, oc):
        raise RuntimeError(f"w has shape {tuple(w.shape)}, trellis implies {(ic, oc)}")
    _check(lib().exl3_reconstruct(w.data_ptr(), trellis.data_ptr(), ic, oc, _k2(k), int(bool(mcg)),
                                  int(bool(mul1)), _stream(w)), "exl3_reconstruct")


def had_r_128(inp: torch.Tensor, out: torch.Tensor, pre_scale, post_scale, scale: float) -> None:
    """out <- H128(inp * pre) * post * scale along the last dim.  ext.had_r_128, ops.py:54,59."""
    _cuda(inp, "in", torch.float16)
    _cuda(out, "out", torch.float16)
    if inp.shape != out.shape:
        raise RuntimeError("had_r_128: in and out differ in shape")
    n = inp.shape[-1]
    rows = inp.numel() // n if n else 0
    for nm, v in (("pre_scale", pre_scale), ("post_scale", post_scale)):
        if v is not None:
            _cuda(v, nm, torch.float16)
            if v.numel() != n:
                raise RuntimeError(f"{nm} has {v.numel()} elements, expected {n}")
    _check(lib().exl3_had_r_128(inp.data_ptr(), out.data_ptr(),
                                None if pre_scale is None else pre_scale.data_ptr(),
                                None if post_scale is None else post_scale.data_ptr(),
                                float(scale), rows, n, _stream(inp)), "exl3_had_r_128")


def gemv_grouped(x: torch.Tensor, shards, y: torch.Tensor, in_mode: int = IN_PLAIN, norm_weight=None,
                 eps: float = 1e-6, residual=None) -> None:
    """y[:, cols of shard s] <- H(H(f(x)*suh_s) W_s) * svh_s (+ residual) for every shard, one launch.
    `shards` is a sequence of dicts with trellis, suh, svh, mcg, mul1 and (optionally) out_col;
    columns default to the running sum of the shard widths.  f is the identity, an RMSNorm
    (in_mode=IN_RMSNORM, optional norm_weight) or silu(x[:, :ic]) * x[:, ic:] (IN_SILU_MUL, x has
    2*ic columns); `residual` ([rows, y.shape[1]] fp16, may be y itself) is added in the epilogue."""
    _cuda(x, "x", torch.float16)
    _cuda(y, "y", torch.float16)
    rows = x.shape[0]
    ic = x.shape[1] // 2 if in_mode == IN_SILU_MUL else x.shape[1]
    arr = _shard_array(x, shards, ic)
    L = lib()
    need = L.exl3_gemv_workspace_bytes(arr, len(shards), rows, ic)
    ws = gemv_workspace(x.device, need) if need else None
    fus = None
    if in_mode != IN_PLAIN or residual is not None:
        if norm_weight is not None:
            _cuda(norm_weight, "norm_weight", torch.float16)
        if residual is not None:
            _cuda(residual, "residual", torch.float16)
            if residual.shape != y.shape:
                raise RuntimeError("residual must have the shape of y")
        fus = Exl3GemvFusion(in_mode, None if norm_weight is None else norm_weight.data_ptr(), float(eps), x.stride(0),
                             None if residual is None else residual.data_ptr(),
                             0 if residual is None else residual.stride(0))
    _check(L.exl3_gemv_grouped_ex(arr, len(shards), x.data_ptr(), y.data_ptr(), rows, ic, y.stride(0),
                                  None if ws is None else ws.data_ptr(), 0 if ws is None else ws.numel(),
                                  None if fus is None else ctypes.byref(fus), _stream(x)), "exl3_gemv_grouped")


def _shard_array(x: torch.Tensor, shards, ic=None):
    ic = x.shape[1] if ic is None else ic
    arr = (Exl3Shard * len(shards))()
    col = 0
    for i, s in enumerate(shards):
        tr = _cuda(s["trellis"], "trellis")
        tic, toc, kk = _trellis_dims(tr)
        if tic != ic:
            raise RuntimeError(f"shard {i}: trellis has {tic} input channels, x has {ic}")
        _cuda(s["suh"], "suh", torch.float16)
        _cuda(s["svh"], "svh", torch.float16)
        oc_col = s.get("out_col", col)
        arr[i] = Exl3Shard(tr.data_ptr(), s["suh"].data_ptr(), s["svh"].data_ptr(), toc, _k2(kk),
                           int(bool(s.get("mcg"))), int(bool(s.get("mul1"))), oc_col)
        col = oc_col + toc
    return arr


def gemv_grouped_static(x: torch.Tensor, shards, y: torch.Tensor) -> None:
    """gemv_grouped on the library's built-in scratch: for callers that may not allocate device
    memory where the layer runs.  No workspace tensor is created here or in the library; a launch
    that needs more scratch than the built-in array holds raises.  Calls on one device share that
    array, so they must not overlap on the GPU."""
    _cuda(x, "x", torch.float16)
    _cuda(y, "y", torch.float16)
    arr = _shard_array(x, shards)
    with torch.cuda.device(x.device):                 # the library uses the current device's scratch
        _check_static(x, shards, y, arr)


def _check_static(x, shards, y, arr):
    _check(lib().exl3_gemv_grouped_static(arr, len(shards), x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1],
                                          y.stride(0), _stream(x)), "exl3_gemv_grouped_static")


def exl3_gemm(A, trellis, C, suh, A_had, svh, kernel: int, mcg: bool, mul1: bool, acc_mode: int) -> None:
    """C[rows, oc] <- H(H(A*suh) W) * svh, fused.  ext.exl3_gemm, ops.py:47-49 of the reference.
    A_had is the reference's scratch operand; this implementation keeps the rotated
    activations on chip and leaves it untouched.  kernel: -1 = automatic."""
    if acc_mode != 0:
        raise RuntimeError("exl3_gemm: only acc_mode 0 is implemented")
    rows = A.shape[0]
    if rows <= GEMV_MAX_ROWS:
        gemv_grouped(A, [dict(trellis=trellis, suh=suh, svh=svh, mcg=mcg, mul1=mul1)], C)
        return
    # more rows than one decode pass holds: walk the batch in passes of 16 rows
    for r0 in range(0, rows, GEMV_MAX_ROWS):
        r1 = min(rows, r0 + GEMV_MAX_ROWS)
        gemv_grouped(A[r0:r1], [dict(trellis=trellis, suh=suh, svh=svh, mcg=mcg, mul1=mul1)], C[r0:r1])


def hgemm_recon(a: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[rows, oc] <- a[rows, ic] @ w[ic, oc], fp16.  ext.hgemm_recon, ops.py:57: a plain
    dense GEMM, which the reference leaves to cuBLAS; so does this (torch.matmul)."""
    _cuda(a, "a", torch.float16)
    _cuda(w, "w", torch.float16)
    _cuda(y, "y", torch.float16)
    torch.matmul(a, w, out=y)


_DT = (torch.float16, torch.bfloat16)
HEAD_MAX_ROWS = 64          # rows per pass over the table (EXL3_INT8_HEAD_MAX_ROWS)


def int8_embed(qweight: torch.Tensor, scales: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Gather int8 rows and scale them: [*ids.shape, hidden] in scales.dtype."""
    _cuda(qweight, "qweight", torch.int8)
    _cuda(scales, "scales", _DT)
    if not isinstance(ids, torch.Tensor) or ids.device.type != "cuda":
        raise RuntimeError("ids must be a CUDA tensor")
    if ids.dtype not in (torch.int64, torch.int32):
        raise RuntimeError(f"ids has dtype {ids.dtype}, expected int64 or int32")
    vocab, hidden = qweight.shape
    if scales.numel() != vocab:
        raise RuntimeError("scales must hold one value per table row")
    flat = ids.reshape(-1).contiguous()
    out = torch.empty((flat.numel(), hidden), dtype=scales.dtype, device=qweight.device)
    if flat.numel() == 0:
        return out.reshape(*ids.shape, hidden)
    _check(lib().exl3_int8_embed(qweight.data_ptr(), scales.data_ptr(), flat.data_ptr(), out.data_ptr(),
                                 flat.numel(), vocab, hidden, int(scales.dtype == torch.bfloat16),
                                 int(flat.dtype == torch.int32), None, _stream(qweight)),
           "exl3_int8_embed")
    return out.reshape(*ids.shape, hidden)


def int8_head(qweight: torch.Tensor, scales: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """logits [rows, vocab] in x.dtype = x @ (q * s)^T without dequantising the table."""
    _cuda(qweight, "qweight", torch.int8)
    _cuda(x, "x", _DT)
    _cuda(scales, "scales", _DT)
    if scales.dtype != x.dtype:
        scales = scales.to(x.dtype)
    vocab, hidden = qweight.shape
    rows = x.shape[0]
    if x.shape[1] != hidden or scales.numel() != vocab:
        raise RuntimeError("int8_head: shapes of x, qweight and scales do not agree")
    out = torch.empty((rows, vocab), dtype=x.dtype, device=x.device)
    L = lib()
    # one pass over the table serves up to 64 rows (16 when the hidden size is not a multiple of 256)
    per_pass = HEAD_MAX_ROWS if hidden % 256 == 0 else 16
    for r0 in range(0, rows, per_pass):
        r1 = min(rows, r0 + per_pass)
        _check(L.exl3_int8_head(qweight.data_ptr(), scales.data_ptr(), x[r0:r1].data_ptr(),
                                out[r0:r1].data_ptr(), r1 - r0, vocab, hidden, vocab,
                                int(x.dtype == torch.bfloat16), _stream(x)), "exl3_int8_head")
    return out


def _rows_view(t: torch.Tensor, name: str, dtype):
    """A CUDA matrix whose rows are contiguous (it may be a column block of a wider one)."""
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise RuntimeError(f"{name} must be a CUDA tensor (this build has no CPU path)")
    if t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise RuntimeError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise RuntimeError(f"{name} must be a matrix with contiguous rows")
    return t


def gemm_tc(x: torch.Tensor, trellis: torch.Tensor, y: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor,
            mcg: bool = False, mul1: bool = False, in_mode: int = IN_PLAIN, norm_weight=None, eps: float = 1e-6,
            residual=None) -> None:
    """y[rows, oc] <- H(H(f(x)*suh) W) * svh (+ residual) for many rows: in-kernel trellis decode feeding
    tcgen05.mma (operand in tensor memory up to 128 rows, in shared memory above).  x fp16 or bf16, y
    fp16; y may be a column block of a wider matrix.  in_mode / norm_weight / eps / residual as in
    gemv_grouped (f = identity, RMSNorm, or silu(x[:, :ic]) * x[:, ic:])."""
    _rows_view(x, "x", _DT)
    _rows_view(y, "y", torch.float16)
    _cuda(trellis, "trellis")
    _cuda(suh, "suh", torch.float16)
    _cuda(svh, "svh", torch.float16)
    ic, oc, kk = _trellis_dims(trellis)
    rows = x.shape[0]
    need = 2 * ic if in_mode == IN_SILU_MUL else ic
    if x.shape[1] != need or tuple(y.shape) != (rows, oc) or suh.numel() != ic or svh.numel() != oc:
        raise RuntimeError("gemm_tc: shapes of x, y, suh, svh do not match the trellis")
    L = lib()
    nbytes = L.exl3_gemm_tc_scratch_bytes(rows, ic, oc)
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x.device)     # freed on exit, like the reference's xh / w
    fused = in_mode != IN_PLAIN or residual is not None or not y.is_contiguous() or not x.is_contiguous()
    if not fused:
        _check(L.exl3_gemm_tc(x.data_ptr(), trellis.data_ptr(), y.data_ptr(), suh.data_ptr(), svh.data_ptr(),
                                  scratch.data_ptr(), nbytes, rows, ic, oc, _k2(kk), int(bool(mcg)), int(bool(mul1)),
                                  int(x.dtype == torch.bfloat16), _stream(x)), "exl3_gemm_tc")
        return
    if norm_weight is not None:
        _cuda(norm_weight, "norm_weight", torch.float16)
    if residual is not None:
        _rows_view(residual, "residual", torch.float16)
        if residual.shape != y.shape:
            raise RuntimeError("residual must have the shape of y")
    fus = Exl3GemvFusion(in_mode, None if norm_weight is None else norm_weight.data_ptr(), float(eps), x.stride(0),
                         None if residual is None else residual.data_ptr(),
                         0 if residual is None else residual.stride(0))
    rc = L.exl3_gemm_tc_ex(x.data_ptr(), trellis.data_ptr(), y.data_ptr(), suh.data_ptr(), svh.data_ptr(),
                           scratch.data_ptr(), nbytes, rows, ic, oc, _k2(kk), int(bool(mcg)), int(bool(mul1)),
                           int(x.dtype == torch.bfloat16), y.stride(0), ctypes.byref(fus), _stream(x))
    if rc == -3 and not (bool(mcg) or bool(mul1)) and (residual is not None or not y.is_contiguous()):
        # an unsplit many-row shape: the kernel rotates y in place, so the pitch and the residual are applied here
        tmp = torch.empty((rows, oc), dtype=torch.float16, device=x.device)
        fus2 = Exl3GemvFusion(in_mode, fus.norm_weight, float(eps), x.stride(0), None, 0)
        _check(L.exl3_gemm_tc_ex(x.data_ptr(), trellis.data_ptr(), tmp.data_ptr(), suh.data_ptr(), svh.data_ptr(),
                                 scratch.data_ptr(), nbytes, rows, ic, oc, _k2(kk), 0, 0,
                                 int(x.dtype == torch.bfloat16), oc, ctypes.byref(fus2), _stream(x)), "exl3_gemm_tc_ex")
        if residual is not None:
            torch.add(tmp, residual, out=y)
        else:
            y.copy_(tmp)
        return
    _check(rc, "exl3_gemm_tc_ex")


def gemm_tc_grouped(x: torch.Tensor, shards, y: torch.Tensor, in_mode: int = IN_PLAIN, norm_weight=None,
                    eps: float = 1e-6, residual=None) -> bool:
    """All shards of a fused layer at 17..128 rows in three launches (the grouped form of gemm_tc): shard s
    writes y[:, out_col_s : out_col_s + oc_s].  Returns False, having done nothing, when the shapes are
    outside what the grouped kernel takes (more than 128 rows, an unsupported codebook);
    the caller then goes shard by shard."""
    _rows_view(x, "x", _DT)
    _rows_view(y, "y", torch.float16)
    rows = x.shape[0]
    ic = x.shape[1] // 2 if in_mode == IN_SILU_MUL else x.shape[1]
    arr = _shard_array(x, shards, ic)
    L = lib()
    nbytes = L.exl3_gemm_tc_grouped_scratch_bytes(arr, len(shards), rows, ic)
    if nbytes == 0:
        return False
    if y.shape[0] != rows:
        raise RuntimeError("gemm_tc_grouped: y has a different number of rows than x")
    if norm_weight is not None:
        _cuda(norm_weight, "norm_weight", torch.float16)
    if residual is not None:
        _rows_view(residual, "residual", torch.float16)
        if residual.shape != y.shape:
            raise RuntimeError("residual must have the shape of y")
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=x.device)
    fus = Exl3GemvFusion(in_mode, None if norm_weight is None else norm_weight.data_ptr(), float(eps), x.stride(0),
                         None if residual is None else residual.data_ptr(),
                         0 if residual is None else residual.stride(0))
    _check(L.exl3_gemm_tc_grouped(arr, len(shards), x.data_ptr(), y.data_ptr(), rows, ic, y.stride(0),
                                  scratch.data_ptr(), nbytes, int(x.dtype == torch.bfloat16), ctypes.byref(fus),
                                  _stream(x)), "exl3_gemm_tc_grouped")
    return True


def gemm_tc_status() -> int:
    return int(lib().exl3_gemm_tc_status())


# --------------------------------------------------------------------------- decode attention
FP8 = torch.float8_e4m3fn


def _kv_dtype(q, k, v, names):
    """fp16 query; caches both fp16 or both e4m3.  Returns True for an fp8 cache."""
    for t, name in zip((q, k, v), names):
        if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
            raise RuntimeError(f"{name} must be a CUDA tensor (this build has no CPU path)")
    if q.dtype != torch.float16 or k.dtype != v.dtype or k.dtype not in (torch.float16, FP8):
        raise RuntimeError(f"{names[0]} must be fp16, {names[1]} / {names[2]} both fp16 or both float8_e4m3fn")
    return k.dtype == FP8


def decode_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_len: int,
                scale: float | None = None, out: torch.Tensor | None = None, k_scale: float = 1.0,
                v_scale: float = 1.0) -> torch.Tensor:
    """softmax(q K^T * scale) V for one query token per sequence.

    q [B, q_heads, 256] fp16 (last two dimensions contiguous); k_cache, v_cache [B, kv_heads, capacity, 256]
    fp16, or float8_e4m3fn holding value / k_scale and value / v_scale, with contiguous rows, of which tokens
    0 .. seq_len-1 are read; query head h uses KV head h // (q_heads // kv_heads).  Returns [B, q_heads, 256] fp16."""
    fp8 = _kv_dtype(q, k_cache, v_cache, ("q", "k_cache", "v_cache"))
    if q.dim() != 3 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape or v_cache.stride() != k_cache.stride():
        raise RuntimeError("decode_attn: q must be [B, heads, 256], the caches [B, kv_heads, capacity, 256] with equal strides")
    B, qh, hd = q.shape
    kvh, cap = k_cache.shape[1], k_cache.shape[2]
    if k_cache.shape[0] != B or k_cache.shape[3] != hd or q.stride(2) != 1 or q.stride(1) != hd \
            or k_cache.stride(3) != 1 or k_cache.stride(2) != hd or not 0 < seq_len <= cap:
        raise RuntimeError("decode_attn: inconsistent shapes or strides")
    if out is None:
        out = torch.empty((B, qh, hd), dtype=torch.float16, device=q.device)
    elif out.shape != (B, qh, hd) or out.dtype != torch.float16 or out.stride(2) != 1 or out.stride(1) != hd:
        raise RuntimeError("decode_attn: out must be [B, heads, 256] fp16 with contiguous heads")
    L = lib()
    need = (L.exl3_decode_attn_fp8_workspace_bytes if fp8 else L.exl3_decode_attn_workspace_bytes)(B, qh, kvh, seq_len)
    ws = torch.empty((need,), dtype=torch.uint8, device=q.device) if need else None
    args = (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
            ws.data_ptr() if ws is not None else None, need, B, qh, kvh, hd, int(seq_len),
            q.stride(0), out.stride(0), k_cache.stride(0), k_cache.stride(1),
            float(hd ** -0.5 if scale is None else scale))
    if fp8:
        _check(L.exl3_decode_attn_fp8(*args, float(k_scale), float(v_scale), _stream(q)), "exl3_decode_attn_fp8")
    else:
        _check(L.exl3_decode_attn(*args, _stream(q)), "exl3_decode_attn")
    return out


def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, k_cache: torch.Tensor,
                v_cache: torch.Tensor, pos: int, q_heads: int, k_scale: float = 1.0, v_scale: float = 1.0) -> None:
    """Rotate the query and key heads of qkv [B, (q_heads + 2 kv_heads) * 256] in place (rotate-half form) and
    write the rotated keys and the values to k_cache / v_cache [B, kv_heads, capacity, 256] at token `pos`.
    cos, sin: [128] fp16 (one position for all sequences) or [B, 128].  float8_e4m3fn caches receive
    value / k_scale and value / v_scale."""
    for t, name in ((qkv, "qkv"), (cos, "cos"), (sin, "sin")):
        if not isinstance(t, torch.Tensor) or t.device.type != "cuda" or t.dtype != torch.float16:
            raise RuntimeError(f"{name} must be a CUDA fp16 tensor (this build has no CPU path)")
    fp8 = _kv_dtype(qkv, k_cache, v_cache, ("qkv", "k_cache", "v_cache"))
    if qkv.dim() != 2 or qkv.stride(1) != 1 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape \
            or v_cache.stride() != k_cache.stride() or k_cache.stride(3) != 1 or k_cache.stride(2) != k_cache.shape[3]:
        raise RuntimeError("rope_append: qkv must be [B, n] with contiguous rows, the caches [B, kv_heads, capacity, 256]")
    B, kvh, cap, hd = k_cache.shape
    if qkv.shape[0] != B or qkv.shape[1] < (q_heads + 2 * kvh) * hd or not 0 <= pos < cap:
        raise RuntimeError("rope_append: inconsistent shapes")
    if cos.shape != sin.shape or cos.shape[-1] != hd // 2 or not cos.is_contiguous() or not sin.is_contiguous() \
            or (cos.dim() == 2 and cos.shape[0] != B) or cos.dim() > 2:
        raise RuntimeError("rope_append: cos / sin must be [128] or [B, 128], contiguous")
    args = (qkv.data_ptr(), qkv.stride(0), cos.data_ptr(), sin.data_ptr(), hd // 2 if cos.dim() == 2 else 0,
            k_cache.data_ptr(), v_cache.data_ptr(), B, q_heads, kvh, hd, int(pos), k_cache.stride(0), k_cache.stride(1))
    if fp8:
        _check(lib().exl3_rope_append_fp8(*args, float(k_scale), float(v_scale), _stream(qkv)), "exl3_rope_append_fp8")
    else:
        _check(lib().exl3_rope_append(*args, _stream(qkv)), "exl3_rope_append")


def decode_attn_paged(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                      seq_lens: torch.Tensor | None, max_seq_len: int, layout: str = "HND",
                      scale: float | None = None, out: torch.Tensor | None = None, k_scale: float = 1.0,
                      v_scale: float = 1.0) -> torch.Tensor:
    """decode_attn over a paged cache.  k_pages / v_pages: [pages, kv_heads, page_size, 256] (layout "HND") or
    [pages, page_size, kv_heads, 256] ("NHD"), fp16 or float8_e4m3fn (value / scale), rows contiguous; block_table
    int32 [B, >= ceil(max_seq_len / page_size)]; seq_lens int32 [B] or None (every sequence has max_seq_len tokens)."""
    fp8 = _kv_dtype(q, k_pages, v_pages, ("q", "k_pages", "v_pages"))
    if layout not in ("HND", "NHD") or k_pages.dim() != 4 or v_pages.shape != k_pages.shape \
            or v_pages.stride() != k_pages.stride() or k_pages.stride(3) != 1:
        raise RuntimeError("decode_attn_paged: page pools must be 4-D with equal shapes and strides, layout HND or NHD")
    hdim, tdim = (1, 2) if layout == "HND" else (2, 1)
    kvh, page_size, hd = k_pages.shape[hdim], k_pages.shape[tdim], k_pages.shape[3]
    B, qh = q.shape[0], q.shape[1]
    if q.dim() != 3 or q.shape[2] != hd or q.stride(2) != 1 or q.stride(1) != hd:
        raise RuntimeError("decode_attn_paged: q must be [B, heads, 256] with contiguous heads")
    if block_table.device != q.device or block_table.dtype != torch.int32 or block_table.dim() != 2 \
            or block_table.shape[0] != B or block_table.stride(1) != 1:
        raise RuntimeError("decode_attn_paged: block_table must be a CUDA int32 [B, n] tensor")
    if seq_lens is not None and (seq_lens.device != q.device or seq_lens.dtype != torch.int32
                                 or seq_lens.shape != (B,) or not seq_lens.is_contiguous()):
        raise RuntimeError("decode_attn_paged: seq_lens must be a CUDA int32 [B] tensor")
    if out is None:
        out = torch.empty((B, qh, hd), dtype=torch.float16, device=q.device)
    elif out.shape != (B, qh, hd) or out.dtype != torch.float16 or out.stride(2) != 1 or out.stride(1) != hd:
        raise RuntimeError("decode_attn_paged: out must be [B, heads, 256] fp16 with contiguous heads")
    L = lib()
    need = (L.exl3_decode_attn_fp8_workspace_bytes if fp8 else L.exl3_decode_attn_workspace_bytes)(
        B, qh, kvh, int(max_seq_len))
    ws = torch.empty((need,), dtype=torch.uint8, device=q.device) if need else None
    args = (q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
            None if seq_lens is None else seq_lens.data_ptr(), out.data_ptr(),
            ws.data_ptr() if ws is not None else None, need, B, qh, kvh, hd,
            int(max_seq_len), page_size, block_table.stride(0) if B > 1 else block_table.shape[1],
            q.stride(0), out.stride(0), k_pages.stride(0), k_pages.stride(hdim),
            k_pages.stride(tdim), float(hd ** -0.5 if scale is None else scale))
    if fp8:
        _check(L.exl3_decode_attn_paged_fp8(*args, float(k_scale), float(v_scale), _stream(q)),
               "exl3_decode_attn_paged_fp8")
    else:
        _check(L.exl3_decode_attn_paged(*args, _stream(q)), "exl3_decode_attn_paged")
    return out
