"""GPU: the allocation-free GEMV entry point against the regular one.

Some hosts cannot let a library call cudaMalloc while they run (all device memory is
already owned by their own allocator, or allocation after start-up is forbidden).
mi_gemv_q4_q8_noalloc serves them with scratch that is part of the library image.
This file checks, through the C ABI, that it returns what mi_gemv_q4_q8 returns, on two
calls in a row (the scratch is shared and keeps the previous call's contents, so the
second call is the one that shows whether it is cleared properly), and that a request
beyond the fixed capacity is refused with a clear error.

The file name sorts last on purpose: if it fails, a run that stops at the first failure
has already run every other test.  It passes alone in a fresh process as well.
"""
import numpy as np
import pytest

import oracle_util as ou

pytestmark = pytest.mark.gpu


def _case(ctx, rows, cols, count, seed):
    import torch
    rng = np.random.default_rng(seed)
    raw = np.concatenate([ou.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)) for _ in range(count)])
    x = rng.standard_normal(cols).astype(np.float32)
    w = ctx.upload_q4_0(raw, rows, cols, count)
    xq = torch.empty(cols, dtype=torch.int8, device="cuda")
    xd = torch.empty(cols // 32, dtype=torch.float16, device="cuda")
    ctx.quant_q8(torch.from_numpy(x).cuda(), xq, xd)
    bias = torch.from_numpy(rng.standard_normal(rows).astype(np.float32)).cuda()
    return w, xq, xd, bias


@pytest.mark.parametrize("rows,cols,count", [(256, 1536, 1), (1536, 8960, 1), (200, 3584, 3), (8960, 1536, 1)])
def test_noalloc_entry_point_matches_regular_entry_point_twice(ctx, rows, cols, count):
    import torch
    w, xq, xd, bias = _case(ctx, rows, cols, count, seed=rows + cols)
    ref = torch.zeros((count, rows), dtype=torch.float32, device="cuda")
    ctx.gemv_q4_q8(w, xq, xd, ref, bias=bias)
    ctx.sync()
    want = ref.cpu().numpy()
    for call in range(2):                                   # second call: scratch holds the first call's leftovers
        y = torch.full((count, rows), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        ctx.gemv_q4_q8_noalloc(w, xq, xd, y, bias=bias)
        ctx.sync()
        # what the entry point exists for: the device's free memory is the same after the call (these shapes are K-split,
        # the regular entry point grows a scratch buffer for them)
        assert torch.cuda.mem_get_info()[0] == free_before, f"call {call} changed the free device memory"
        got = y.cpu().numpy()
        # the tolerance of the GEMV parity tests (1e-3 of the output scale); both paths sum in
        # double and round once, so in practice the bits are equal
        assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max(), f"call {call}"
        assert np.array_equal(got, want), f"call {call}"


def test_noalloc_entry_point_refuses_what_does_not_fit(ctx, pkg):
    import torch
    # a stack with more than 2048 row groups that the kernel still K-splits (fewer groups than twice the
    # warps of the grid): it needs more arrival counters than the built-in scratch has
    limit = ctx.sm_count * 8 * 2
    if limit <= 2100:
        pytest.skip("this GPU does not K-split a stack of more than 2048 row groups")
    rows, cols = 32 * 23, 512
    count = (min(limit - 1, 2300) // 23)
    assert 2048 < count * 23 < limit
    raw = np.zeros(count * rows * (cols // 32) * 18, dtype=np.uint8)
    w = ctx.upload_q4_0(raw, rows, cols, count)
    xq = torch.zeros(cols, dtype=torch.int8, device="cuda")
    xd = torch.zeros(cols // 32, dtype=torch.float16, device="cuda")
    y = torch.zeros((count, rows), dtype=torch.float32, device="cuda")
    with pytest.raises(pkg.MinferError) as e:
        ctx.gemv_q4_q8_noalloc(w, xq, xd, y)
    assert e.value.status == 8 and "built-in scratch" in str(e.value)
    ctx.sync()
    # the other limit: few enough row groups for the counters, but groups x K-splits x 32 partial sums beyond 65536
    groups = 1100
    ks = min(-(-(2 * ctx.sm_count * 8) // groups), 2)        # the kernel's split for this stack, capped by its two tiles per row group
    if ks > 1 and groups * ks * 32 > 65536:
        rows2 = 32 * groups
        raw2 = np.zeros(rows2 * (cols // 32) * 18, dtype=np.uint8)
        w2 = ctx.upload_q4_0(raw2, rows2, cols, 1)
        y2 = torch.zeros((1, rows2), dtype=torch.float32, device="cuda")
        with pytest.raises(pkg.MinferError) as e2:
            ctx.gemv_q4_q8_noalloc(w2, xq, xd, y2)
        assert e2.value.status == 8 and "partial sums" in str(e2.value)
        ctx.sync()
