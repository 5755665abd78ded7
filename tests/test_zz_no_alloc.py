"""The allocation-free GEMV entry point (built-in scratch) against the regular one.

Some hosts cannot allocate device memory at the point where a layer runs -- the serving process
gave all free memory to its cache pool, or its hot path bans allocator calls.  For them the
library offers exl3_gemv_grouped_static, which keeps the kernel's scratch in a fixed array of its
own.  This test calls it through the C ABI, twice in a row, and requires the same bytes as the
regular entry point; it also checks that an over-sized request is refused and that the call does
not grow the CUDA memory in use.  Kept in its own file so that it is collected after every other
test."""
import ctypes

import pytest
import torch

import exl3_ref as R

pytestmark = pytest.mark.gpu


def _layer(seed, ic, spec, rows):
    shards = []
    for i, (oc, K) in enumerate(spec):
        tr, suh, svh, _ = R.make_layer(seed + i, ic, oc, K, 1)
        shards.append(dict(trellis=tr.cuda(), suh=suh.cuda(), svh=svh.cuda(), mcg=False, mul1=False))
    x = torch.randn((rows, ic), generator=torch.Generator().manual_seed(seed)).half().cuda()
    return shards, x, sum(oc for oc, _ in spec)


@pytest.mark.parametrize("ic,spec,rows", [
    (1024, [(768, 4), (256, 5), (256, 6)], 1),        # fused, mixed bitrate, split over the inputs
    (5120, [(1024, 3)], 4),
    (2048, [(256, 2), (128, 6)], 9),
])
def test_static_scratch_matches_regular_entry_point(ext, ic, spec, rows):
    shards, x, total = _layer(900 + ic + rows, ic, spec, rows)
    want = torch.empty((rows, total), dtype=torch.half, device="cuda")
    ext.gemv_grouped(x, shards, want)
    torch.cuda.synchronize()
    for attempt in range(2):                                  # two calls in a row share the array
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        ext.gemv_grouped_static(x, shards, got)
        assert torch.cuda.memory_allocated() == before        # nothing was allocated for it
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {attempt}"
    # a different input right after, same array
    x2 = (x.float() * 0.5 + 1.0).half()
    ext.gemv_grouped(x2, shards, want)
    got = torch.empty_like(want)
    ext.gemv_grouped_static(x2, shards, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # a first call made on a stream of its own works the same way (nothing is queued at set-up)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got2 = torch.empty_like(want)
        ext.gemv_grouped_static(x2, shards, got2)
    side.synchronize()
    assert torch.equal(got2, want)
    # no bounded wait inside those launches ran out: the built-in array's sticky status word is clear
    assert ext.gemv_static_status(x.device) == 0


def test_static_scratch_rejects_oversized_request(ext):
    cap = ext.lib().exl3_gemv_static_capacity()
    assert 1 << 20 <= cap <= 16 << 20
    shards, x, total = _layer(77, 17408, [(128, 4)] * 8, 16)  # eight shards' rotated activations: more than it holds
    arr = ext._shard_array(x, shards)
    need = ext.lib().exl3_gemv_workspace_bytes(arr, 8, 16, 17408)
    assert need > cap
    y = torch.zeros((16, total), dtype=torch.half, device="cuda")
    with pytest.raises(RuntimeError, match="workspace"):
        ext.gemv_grouped_static(x, shards, y)
    torch.cuda.synchronize()
    assert torch.count_nonzero(y) == 0                        # nothing was launched
    ext.gemv_grouped(x, shards, y)                            # the regular entry point still serves it
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()
