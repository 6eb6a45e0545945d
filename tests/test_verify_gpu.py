"""GPU parity of the M-token step (mi_verify: tcgen05 GEMM projections + M-query attention)
and of the stand-alone split-KV attention entry point (mi_attn_splitkv).

Bars: a token's logits are bit-identical for every M (1..16) and bit-identical to the
single-token persistent decode; greedy ids equal to the q8 oracle and logits within 1e-3
relative of it; attention within 1e-5 relative of a float64 softmax over the same fp16 cache.
"""
import json
from pathlib import Path

import numpy as np
import pytest

import gguf_util as gu
import oracle_util as ou

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
REL_TOL = 1e-3


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = tmp_path_factory.mktemp("vmodels")
    c = json.loads((GOLD / "streams_ref.json").read_text())[1]
    return gu.make_synthetic(d / "tiny.gguf", c["preset"], seed=c["seed"], std=c["std"], extra=["--bias-std", c["bias_std"]])


def run_chunks(m, seq, M, V, pos0=0):
    import torch
    out, lg = [], torch.zeros((len(seq), V), dtype=torch.float32, device="cuda")
    for i in range(0, len(seq), M):
        part = seq[i:i + M]
        o, _ = m.verify(part, pos0 + i, lg[i:i + len(part)])
        out += o
    return out, lg.cpu().numpy()


def test_logits_identical_for_every_m_and_equal_to_decode(ctx, pkg, tiny):
    import torch
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    n = 48
    seq = [int(t) for t in np.random.default_rng(21).integers(0, V, n)]
    m = pkg.Model(ctx, tiny, n + 1)
    ref_logits = torch.zeros((n, V), dtype=torch.float32, device="cuda")
    ref_tok, _ = m.decode(seq, n, 0, ref_logits, pkg.DECODE_PERSISTENT)
    ref = ref_logits.cpu().numpy()
    for M in (1, 2, 3, 4, 8, 16):
        tok, lg = run_chunks(m, seq, M, V)
        assert tok == ref_tok, f"M={M}: greedy ids differ from the single-token decode"
        assert np.array_equal(lg.view(np.uint32), ref.view(np.uint32)), f"M={M}: logits are not bit-identical to the single-token decode"
    orc = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=n + 1)
    worst = 0.0
    for s, t in enumerate(seq):
        tok, lo, _ = orc.forward(t)
        assert tok == ref_tok[s]
        worst = max(worst, rel_err(ref[s], lo))
    assert worst < REL_TOL
    m.free()


def test_prefill_then_decode_continues_the_stream(ctx, pkg, tiny):
    """Prompt through the M-token step, generation through the persistent kernel: same ids as decode alone."""
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    prompt = [int(t) for t in np.random.default_rng(22).integers(0, V, 37)]
    m = pkg.Model(ctx, tiny, 80)
    want, _ = m.generate(prompt, 24)
    first, _ = m.prefill(prompt, 0, chunk=16)
    rest, _ = m.decode([first], 23, len(prompt), None, pkg.DECODE_PERSISTENT)
    assert [first] + rest == want
    m.free()


def test_long_context_chunks_match_decode(ctx, pkg, tiny):
    """Queries whose causal ranges straddle the attention regimes (<= 256, <= 1024, beyond) inside one pass."""
    import torch
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    n = 1072
    seq = [int(t) for t in np.random.default_rng(23).integers(0, V, n)]
    m = pkg.Model(ctx, tiny, n + 1)
    ref_logits = torch.zeros((n, V), dtype=torch.float32, device="cuda")
    ref_tok, _ = m.decode(seq, n, 0, ref_logits, pkg.DECODE_PERSISTENT)
    m2 = pkg.Model(ctx, tiny, n + 1)
    tok, lg = run_chunks(m2, seq, 16, V)
    assert tok == ref_tok
    ref = ref_logits.cpu().numpy()
    for s in (0, 15, 16, 250, 255, 256, 257, 1020, 1023, 1024, 1025, 1039, 1071):
        assert np.array_equal(lg[s].view(np.uint32), ref[s].view(np.uint32)), f"position {s}"
    m.free(); m2.free()


def attention_f64(q, K, V, n_head, n_kv, hd, pos):
    """float64 softmax attention of one query over positions 0..pos of an fp16 cache."""
    out = np.zeros(n_head * hd)
    gq = n_head // n_kv
    for h in range(n_head):
        kv = h // gq
        k = K[:pos + 1, kv * hd:(kv + 1) * hd].astype(np.float64)
        v = V[:pos + 1, kv * hd:(kv + 1) * hd].astype(np.float64)
        s = (k @ q[h * hd:(h + 1) * hd].astype(np.float64)).astype(np.float32) * np.float32(1.0 / np.sqrt(np.float32(hd)))
        s = s.astype(np.float64)
        w = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (w @ v) / w.sum()
    return out


@pytest.mark.parametrize("n_head,n_kv,hd", [(12, 2, 128), (14, 2, 64), (4, 2, 32)])
@pytest.mark.parametrize("pos0,M", [(0, 1), (0, 16), (250, 9), (1017, 16), (3000, 4), (8191, 1), (8191 - 15, 16), (32767, 1), (32767 - 15, 16)])
def test_attn_splitkv_matches_float64_softmax(ctx, pkg, n_head, n_kv, hd, pos0, M):
    import torch
    rng = np.random.default_rng(pos0 * 31 + M + hd)
    npos = pos0 + M
    K = rng.standard_normal((npos, n_kv * hd)).astype(np.float16)
    Vv = rng.standard_normal((npos, n_kv * hd)).astype(np.float16)
    q = rng.standard_normal((M, n_head * hd)).astype(np.float32)
    out = torch.zeros((M, n_head * hd), dtype=torch.float32, device="cuda")
    ctx.attn_splitkv(torch.from_numpy(q).cuda(), torch.from_numpy(K.view(np.uint16).astype(np.int16)).cuda(),
                     torch.from_numpy(Vv.view(np.uint16).astype(np.int16)).cuda(), n_head, n_kv, hd, pos0, M, out)
    ctx.sync()
    got = out.cpu().numpy()
    for i in range(M):
        want = attention_f64(q[i], K, Vv, n_head, n_kv, hd, pos0 + i)
        assert rel_err(got[i], want) < 1e-5, f"query {i} at position {pos0 + i}"


def test_attn_splitkv_rejects_bad_arguments(ctx, pkg):
    import torch
    t = torch.zeros(16, device="cuda")
    with pytest.raises(pkg.MinferError):
        ctx.attn_splitkv(t, t, t, 12, 5, 128, 0, 1, t)       # query heads not a multiple of kv heads
    with pytest.raises(pkg.MinferError):
        ctx.attn_splitkv(t, t, t, 12, 2, 128, 0, 17, t)      # more queries than one call takes
    with pytest.raises(pkg.MinferError):
        ctx.attn_splitkv(t, t, t, 12, 4, 128, 0, 1, t)       # a (head_dim, group) pair that is not instantiated


def test_graph_replay_matches_plain_launches(pkg, ctx, tiny):
    """On a stream of its own the pass is captured into a CUDA graph on the second call with a given M and
    replayed afterwards, with tokens and position read from device memory: same bits as the plain launches
    (the shared `ctx` fixture runs on the legacy default stream, which cannot capture)."""
    import torch
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    n = 64
    seq = [int(t) for t in np.random.default_rng(24).integers(0, V, n)]
    plain = pkg.Model(ctx, tiny, n + 1)
    want_tok, want = run_chunks(plain, seq, 8, V)
    own = pkg.Context(0)                      # the library's own stream
    m = pkg.Model(own, tiny, n + 1)
    torch.cuda.synchronize()
    got_tok, got = run_chunks(m, seq, 8, V)   # pass 1 plain, pass 2 builds the graph, passes 3.. replay it
    assert got_tok == want_tok
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # a split-K GEMV on the same context makes the library grow (and move) the scratch the captured GEMMs point
    # into: the next pass must notice and rebuild its graph instead of replaying the stale one
    rows, cols = 2048, 4096
    raw = ou.quantize_q4_0((np.random.default_rng(5).standard_normal((rows, cols)) * 0.02).astype(np.float32))
    w = own.upload_q4_0(raw, rows, cols)
    xq = torch.zeros(cols, dtype=torch.int8, device="cuda"); xd = torch.ones(cols // 32, dtype=torch.float16, device="cuda")
    y = torch.zeros(rows, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    own.gemv_q4_q8(w, xq, xd, y, ksplit=8)
    own.sync()
    again_tok, again = run_chunks(m, seq, 8, V)
    assert again_tok == want_tok
    assert np.array_equal(again.view(np.uint32), want.view(np.uint32))
    plain.free(); m.free()


@pytest.mark.parametrize("context", [8192, 32768])
def test_m_invariance_at_long_cached_contexts(ctx, pkg, tiny, context):
    """The multi-token configuration's long contexts: the KV cache pre-filled with seeded N(0,1) fp16 for `context`
    positions, then the same 16 drafted tokens scored with M = 1, 2, 4, 8, 16 tokens per weight pass starting at
    position `context`.  Every token's logits must be the same bits whatever M is, and equal to the single-token decode
    kernel's (whose chunked attention walks the same ranges)."""
    import torch
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    seq = [int(t) for t in np.random.default_rng(context).integers(0, V, 16)]
    m = pkg.Model(ctx, tiny, context + 17)
    gen = torch.Generator(device="cuda"); gen.manual_seed(context)
    for name in ("kcache", "vcache"):
        m.state_tensor(name).view(torch.float16).normal_(generator=gen)
    torch.cuda.synchronize()
    ref = None
    for M in (1, 2, 4, 8, 16):
        tok, lg = run_chunks(m, seq, M, V, pos0=context)          # each pass rewrites positions context.. with the same values
        if ref is None:
            ref, ref_tok = lg, tok
        else:
            assert tok == ref_tok, f"M={M}: greedy ids differ"
            assert np.array_equal(lg.view(np.uint32), ref.view(np.uint32)), f"M={M}: logits differ from M=1 at context {context}"
    dl = torch.zeros((16, V), dtype=torch.float32, device="cuda")
    dtok, _ = m.decode(seq, 16, context, dl, pkg.DECODE_PERSISTENT)
    assert dtok == ref_tok and np.array_equal(dl.cpu().numpy().view(np.uint32), ref.view(np.uint32)), "decode kernel differs from the M-token step"
    m.free()
