"""GPU parity of the multi-token q4_0 x q8_0 GEMM (tcgen05 int8 MMA) through the C ABI.

Bars: every token's row of Y equals, bit for bit, what the GEMV entry point returns for
that token alone - for every M (the reference checks the same property with a logit hash
over step sizes, src/mega.cu:1198-1204) - and is within 1e-3 relative of the CPU oracle.
"""
import numpy as np
import pytest

import oracle_util as ou

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def _setup(ctx, rows, cols, M, seed):
    import torch
    rng = np.random.default_rng(seed)
    raw = ou.quantize_q4_0((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    X = rng.standard_normal((M, cols)).astype(np.float32)
    X[0, :32] = 0.0
    w = ctx.upload_q4_0(raw, rows, cols)
    xq = torch.empty((M, cols), dtype=torch.int8, device="cuda")
    xd = torch.empty((M, cols // 32), dtype=torch.float16, device="cuda")
    ctx.quant_q8(torch.from_numpy(X).cuda(), xq, xd, n=cols, M=M)
    return raw, X, w, xq, xd


@pytest.mark.parametrize("rows,cols", [(128, 256), (1536, 1536), (256, 1536), (1536, 8960), (200, 896), (8960, 1536), (96, 64)])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_gemm_rows_equal_gemv_bit_for_bit_and_match_oracle(ctx, rows, cols, M):
    import torch
    raw, X, w, xq, xd = _setup(ctx, rows, cols, M, seed=rows + cols + M)
    bias = torch.from_numpy(np.random.default_rng(2).standard_normal(rows).astype(np.float32)).cuda()
    Y = torch.full((M, rows), float("nan"), dtype=torch.float32, device="cuda")
    ctx.gemm_q4_q8(w, xq, xd, M, Y, bias=bias)
    ctx.sync()
    Yh = Y.cpu().numpy()
    for m in range(M):
        y1 = torch.zeros(rows, dtype=torch.float32, device="cuda")
        ctx.gemv_q4_q8(w, xq[m], xd[m], y1, bias=bias)
        ctx.sync()
        assert np.array_equal(Yh[m], y1.cpu().numpy()), f"token {m} of {M}"
    eq, ed = ou.quant_q8(X[M - 1])
    assert rel_err(Yh[M - 1], ou.gemv_q4_q8(raw, rows, cols, eq, ed, bias.cpu().numpy())) < 1e-3


def test_gemm_result_does_not_depend_on_M(ctx):
    """Token 0 scored alone, with 3 and with 15 companions: identical bits (step-size invariance)."""
    import torch
    rows, cols = 2048, 1536
    raw, X, w, xq, xd = _setup(ctx, rows, cols, 16, seed=99)
    outs = []
    for M in (1, 4, 16):
        Y = torch.zeros((M, rows), dtype=torch.float32, device="cuda")
        ctx.gemm_q4_q8(w, xq, xd, M, Y)
        ctx.sync()
        outs.append(Y[0].cpu().numpy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_gemm_argument_checks(ctx, pkg):
    import torch
    raw, X, w, xq, xd = _setup(ctx, 64, 64, 2, seed=1)
    Y = torch.zeros((2, 64), device="cuda")
    for bad_m in (0, 17):
        with pytest.raises(pkg.MinferError):
            ctx.gemm_q4_q8(w, xq, xd, bad_m, Y)
    with pytest.raises(pkg.MinferError):
        ctx.gemm_q4_q8(w, None, xd, 2, Y)
    ctx.sync()
