"""The EXL3 shard GEMM as PyTorch custom ops, so the layer stays one opaque node under
torch.compile and replays inside CUDA graphs (reference orcasaq2/ops.py:1-66).

`orcasaq2::shard_gemm` keeps the reference schema.  `orcasaq2::layer_gemm` is the grouped form
used by `Exl3LinearMethod.apply`: every shard of a fused layer in one launch, written straight
into the concatenated output.

Row-count dispatch (reference ops.py:25,46).  Up to 16 rows: the fused decode GEMV (HBM-bound
streaming of the packed trellis; a single shard moves to the tensor-memory kernel below from 9 rows).  From 17 rows: `exl3_gemm_tc`.  For few hundred rows that is
one pass over the packed weights with no dense copy in memory -- up to 128 rows the decoded weights go from registers into tensor memory and are the A
operand of tcgen05.mma; above that they are staged as swizzled shared-memory tiles.  From 1024 rows (from 384 .. 640 rows for wide layers, where it measured faster) the library decodes once (the reference's own idea
for many rows, ops.py:50-59: rotate, rebuild the weight into scratch, dense GEMM, rotate back) and runs its own dense tcgen05 GEMM on CTA pairs, whose
epilogue rotates and scales the output rows in registers (no separate pass).  The reference's route with a library GEMM (`_dense_path`) remains for shapes the pair kernel
does not take (an odd number of 128-channel output blocks) and behind ORCA_EXL3_TC_MAX_ROWS.  GEMM_MAX_ROWS keeps the
reference's name and default; it is the bound up to which the packed trellis is read directly
when the tcgen05 path is switched off (ORCA_EXL3_TC=0).
"""
import os
from typing import List

import torch
from torch import Tensor

from . import _ext

# Name of the packed layout this build reads and writes (bit order, order of the weights inside a tile,
# "3INST" codebook); synthetic checkpoints carry it in quantization_config.json as "exl3_layout".
PACK_LAYOUT = "orcasaq2-b200-3inst-v1"

GEMM_MAX_ROWS = int(os.environ.get("ORCA_EXL3_GEMM_MAX_ROWS", "144"))
USE_TC = os.environ.get("ORCA_EXL3_TC", "1") != "0"
TC_MAX_ROWS = int(os.environ.get("ORCA_EXL3_TC_MAX_ROWS", str(1 << 30)))
TC_PAIR_MIN_ROWS = 1024          # from here exl3_gemm_tc wants an even number of 128-channel output blocks


def _tc_takes(rows: int, oc: int) -> bool:
    """Whether exl3_gemm_tc is the route for this many rows of a shard with `oc` outputs."""
    return USE_TC and rows <= TC_MAX_ROWS and (rows < TC_PAIR_MIN_ROWS or (oc // 128) % 2 == 0)
# 9..16 rows, measured on B200 (us per call, GEMV against the tensor-memory kernel): a single shard with many
# input channels is faster on the tensor-memory kernel (17408 -> 5120 at 4 bpw: 40.5 / 45.0 against 40.3 / 40.6 at
# 9 / 16 rows), a fused layer on the grouped GEMV (2 x 5120 -> 17408 at 3 bpw: 64.8 / 67.7 against 74.3 / 74.7;
# qkv: 27.1 / 30.6 against 29.4 / 29.3).  So single shards switch at 9 rows, fused layers at 17.
TC_MIN_ROWS_SINGLE = int(os.environ.get("ORCA_EXL3_TC_MIN_ROWS", "9"))
TC_MIN_ROWS_GROUPED = int(os.environ.get("ORCA_EXL3_TC_MIN_ROWS_GROUPED", "17"))


def exl3_K(trellis: Tensor):
    """Bits per weight from the packed width: last dim / 16.  The half rates (1.5/2.5/3.5) are
    kept as floats -- a 3.5-bit tile packs 56 words, and flooring would silently give 3
    (reference ops.py:28-34)."""
    k = trellis.shape[-1] / 16
    return int(k) if float(k).is_integer() else k


def _narrow_k(k: float):
    return int(k) if float(k).is_integer() else k


def _dense_path(x: Tensor, trellis: Tensor, suh: Tensor, svh: Tensor, k, mcg: bool, mul1: bool,
                y: Tensor) -> None:
    """rows > GEMM_MAX_ROWS: rotate, rebuild the weight into scratch, dense GEMM, rotate back."""
    xh = torch.empty_like(x)
    _ext.had_r_128(x, xh, suh, None, 1.0)
    w = torch.empty((x.shape[1], y.shape[1]), dtype=torch.half, device=x.device)
    _ext.reconstruct(w, trellis, k, mcg, mul1)
    _ext.hgemm_recon(xh, w, y)
    del w, xh                        # scratch only: keeping it would undo the compression
    _ext.had_r_128(y, y, None, svh, 1.0)


@torch.library.custom_op("orcasaq2::shard_gemm", mutates_args=())
def shard_gemm(x: Tensor, trellis: Tensor, suh: Tensor, svh: Tensor,
               oc: int, k: float, mcg: bool, mul1: bool) -> Tensor:
    k = _narrow_k(k)
    rows = x.shape[0]
    y = torch.empty((rows, oc), dtype=torch.half, device=x.device)
    if rows == 0:
        return y
    small_tc = USE_TC and TC_MIN_ROWS_SINGLE <= rows <= _ext.GEMV_MAX_ROWS
    if (rows <= _ext.GEMV_MAX_ROWS and not small_tc) or (not USE_TC and rows <= GEMM_MAX_ROWS):
        _ext.exl3_gemm(x, trellis, y, suh, x, svh, -1, mcg, mul1, 0)
    elif _tc_takes(rows, oc):
        _ext.gemm_tc(x, trellis, y, suh, svh, mcg, mul1)
    else:
        _dense_path(x, trellis, suh, svh, k, mcg, mul1, y)
    return y


@shard_gemm.register_fake
def _shard_gemm_fake(x: Tensor, trellis: Tensor, suh: Tensor, svh: Tensor,
                     oc: int, k: float, mcg: bool, mul1: bool) -> Tensor:
    return x.new_empty((x.shape[0], oc), dtype=torch.half)


@torch.library.custom_op("orcasaq2::layer_gemm", mutates_args=())
def layer_gemm(x: Tensor, trellis: List[Tensor], suh: List[Tensor], svh: List[Tensor],
               ocs: List[int], ks: List[float], mcg: List[bool], mul1: List[bool]) -> Tensor:
    """All shards of one layer: returns [rows, sum(ocs)] fp16, shard outputs side by side."""
    rows = x.shape[0]
    total = sum(ocs)
    y = torch.empty((rows, total), dtype=torch.half, device=x.device)
    if rows == 0:
        return y
    n = len(trellis)
    shards = [dict(trellis=trellis[i], suh=suh[i], svh=svh[i], mcg=mcg[i], mul1=mul1[i]) for i in range(n)]
    # from the row count measured above: one grouped launch of the tensor-memory kernel where its shapes apply; it
    # declines other shapes without doing anything
    tc_from = TC_MIN_ROWS_SINGLE if n == 1 else TC_MIN_ROWS_GROUPED
    if (USE_TC and tc_from <= rows <= TC_MAX_ROWS and n <= _ext.MAX_SHARDS
            and _ext.gemm_tc_grouped(x, shards, y)):
        pass
    elif rows > _ext.GEMV_MAX_ROWS and all(_tc_takes(rows, oc) for oc in ocs):
        col = 0
        for i in range(n):
            # every shard writes its own column block of y (no torch.cat, reference config.py:242)
            _ext.gemm_tc(x, trellis[i], y[:, col:col + ocs[i]], suh[i], svh[i], mcg[i], mul1[i])
            col += ocs[i]
    elif rows <= GEMM_MAX_ROWS:
        for g0 in range(0, n, _ext.MAX_SHARDS):
            grp = shards[g0:g0 + _ext.MAX_SHARDS]
            col0 = sum(ocs[:g0])
            c = col0
            for s, oc in zip(grp, ocs[g0:g0 + _ext.MAX_SHARDS]):
                s["out_col"] = c
                c += oc
            for r0 in range(0, rows, _ext.GEMV_MAX_ROWS):
                r1 = min(rows, r0 + _ext.GEMV_MAX_ROWS)
                _ext.gemv_grouped(x[r0:r1], grp, y[r0:r1])
    else:
        col = 0
        for i in range(n):
            yi = torch.empty((rows, ocs[i]), dtype=torch.half, device=x.device)
            _dense_path(x, trellis[i], suh[i], svh[i], _narrow_k(ks[i]), mcg[i], mul1[i], yi)
            y[:, col:col + ocs[i]] = yi
            col += ocs[i]
    return y


@layer_gemm.register_fake
def _layer_gemm_fake(x: Tensor, trellis: List[Tensor], suh: List[Tensor], svh: List[Tensor],
                     ocs: List[int], ks: List[float], mcg: List[bool], mul1: List[bool]) -> Tensor:
    return x.new_empty((x.shape[0], sum(ocs)), dtype=torch.half)


# The int8 embedding gather and the int8 head as opaque ops, for the same reason as shard_gemm (reference ops.py:3-16):
# the kernels are reached through ctypes, which Dynamo cannot trace, and the embedding sits INSIDE the model's
# compiled forward (vllm/model_executor/layers/vocab_parallel_embedding.py:484).  The reference's own gather is plain
# torch indexing (heads.py:61-67) and needs no op.
@torch.library.custom_op("orcasaq2::int8_embed", mutates_args=())
def int8_embed(qweight: Tensor, scales: Tensor, ids: Tensor) -> Tensor:
    return _ext.int8_embed(qweight, scales, ids)


@int8_embed.register_fake
def _int8_embed_fake(qweight: Tensor, scales: Tensor, ids: Tensor) -> Tensor:
    return scales.new_empty((*ids.shape, qweight.shape[1]))


@torch.library.custom_op("orcasaq2::int8_head", mutates_args=())
def int8_head(qweight: Tensor, scales: Tensor, x: Tensor) -> Tensor:
    return _ext.int8_head(qweight, scales, x)


@int8_head.register_fake
def _int8_head_fake(qweight: Tensor, scales: Tensor, x: Tensor) -> Tensor:
    return x.new_empty((x.shape[0], qweight.shape[0]))
