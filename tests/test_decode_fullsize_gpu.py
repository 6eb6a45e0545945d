"""GPU parity at the benchmark's own sizes (configs 0 and 2 of the benchmark definition):
the Qwen2.5-0.5B and -1.5B shapes with seeded random all-q4_0 weights, against the CPU
oracle in q8_0-activation / fp16-KV mode.  The oracle needs about half a second (0.5B) to a
second and a half (1.5B) per token on the test machine's host cores, so the number of
positions is bounded; the GPU side runs the full prompt + generation of config 0.

Bars: greedy ids identical; logits within 1e-3 relative at every compared position
(0.0 is what the double-carried arithmetic gives in practice)."""
import numpy as np
import pytest

import gguf_util as gu
import oracle_util as ou

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("preset,n_prompt,n_gen,n_logit_pos", [("0.5b", 16, 32, 6), ("1.5b", 8, 6, 3)])
def test_fullsize_decode_matches_q8_oracle(ctx, pkg, tmp_path, preset, n_prompt, n_gen, n_logit_pos):
    import torch
    path = gu.make_synthetic(tmp_path / "m.gguf", preset, seed=2025)
    g = gu.GgufReader(path)
    V = g.config()["n_vocab"]
    prompt = [int(t) for t in np.random.default_rng(2025).integers(0, V, n_prompt)]
    n_steps = n_prompt + n_gen - 1
    m = pkg.Model(ctx, path, n_steps + 1)
    got, _ = m.generate(prompt, n_gen)                                  # persistent engine, config-0 style run
    seq = prompt + got[:-1]
    # the oracle follows the same token sequence (teacher-forced on the GPU's ids) and must predict the same ids
    orc = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=n_steps + 1)
    logits = torch.zeros((n_steps, V), dtype=torch.float32, device="cuda")
    m2 = pkg.Model(ctx, path, n_steps + 1)
    pred, _ = m2.decode(seq, n_steps, 0, logits, pkg.DECODE_PER_PHASE)
    assert pred[n_prompt - 1:] == got                                   # both engines, same stream
    check_at = set(range(n_logit_pos)) | {n_steps - 1}
    worst = 0.0
    for s, t in enumerate(seq):
        want_logits = s in check_at
        tok, lo, _ = orc.forward(t, want_logits=want_logits)
        assert tok == pred[s], f"greedy id differs from the oracle at position {s}"
        if want_logits:
            worst = max(worst, rel_err(logits[s].cpu().numpy(), lo))
    assert worst < 1e-3, f"logits deviate {worst:.2e}"
    m.free(); m2.free()


@pytest.mark.parametrize("preset", ["1.5b", "3b"])
def test_fullsize_engines_and_m_token_step_agree_bit_for_bit(ctx, pkg, tmp_path, preset):
    """The 1.5B shape and the 3B shape (36 layers, hidden 2048, 16 / 2 heads, FFN 11008: the batched configuration's
    model at batch 1): persistent kernel == kernel sequence == M-token step (8 and 16 tokens per weight pass) on the
    logits of every position, as bits.  No oracle here - the CPU side would take minutes at this size."""
    import torch
    path = gu.make_synthetic(tmp_path / "m.gguf", preset, seed=77)
    g = gu.GgufReader(path)
    V = g.config()["n_vocab"]
    n = 24
    seq = [int(t) for t in np.random.default_rng(77).integers(0, V, n)]
    m = pkg.Model(ctx, path, n + 1)
    ref = torch.zeros((n, V), dtype=torch.float32, device="cuda")
    tok_ref, _ = m.decode(seq, n, 0, ref, pkg.DECODE_PERSISTENT)
    lg = torch.zeros_like(ref)
    tok, _ = m.decode(seq, n, 0, lg, pkg.DECODE_PER_PHASE)
    assert tok == tok_ref and torch.equal(lg.view(torch.int32), ref.view(torch.int32)), "kernel sequence differs from the persistent kernel"
    for M in (8, 16):
        lg.zero_()
        tok = []
        for i in range(0, n, M):
            part = seq[i:i + M]
            o, _ = m.verify(part, i, lg[i:i + len(part)])
            tok += o
        assert tok == tok_ref and torch.equal(lg.view(torch.int32), ref.view(torch.int32)), f"M-token step (M={M}) differs from the decode"
    m.free()


def test_config2_window_against_the_oracle(ctx, pkg, tmp_path):
    """The benchmark configuration itself: 1.5B shape, 64-token seeded prompt, 128 generated tokens, KV cache for 4096
    positions.  The GPU generates the window; the oracle then follows the GPU's tokens teacher-forced through all 191
    positions (a tenth of a second each on the test machine) and must predict the same id at every one; logits are
    compared at the last prompt position, at every 16th generated position and at the last.  The kernel-sequence
    engine must give the persistent kernel's bits over the whole window."""
    import torch
    path = gu.make_synthetic(tmp_path / "m.gguf", "1.5b", seed=20251)
    g = gu.GgufReader(path)
    V = g.config()["n_vocab"]
    prompt = [int(t) for t in np.random.default_rng(20251).integers(0, V, 64)]
    n_gen, n_steps = 128, 64 + 128 - 1
    m = pkg.Model(ctx, path, 4096)
    got, _ = m.generate(prompt, n_gen)
    seq = prompt + got[:-1]
    lg = torch.zeros((n_steps, V), dtype=torch.float32, device="cuda")
    pred, _ = m.decode(seq, n_steps, 0, lg, pkg.DECODE_PERSISTENT)
    assert pred[63:] == got
    m2 = pkg.Model(ctx, path, 4096)
    lg2 = torch.zeros((n_steps, V), dtype=torch.float32, device="cuda")
    pred2, _ = m2.decode(seq, n_steps, 0, lg2, pkg.DECODE_PER_PHASE)
    assert pred2 == pred and torch.equal(lg.view(torch.int32), lg2.view(torch.int32)), "kernel sequence differs from the persistent kernel over the window"
    orc = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=n_steps + 1)
    check = {63} | {63 + 16 * k for k in range(1, 8)} | {n_steps - 1}
    worst = 0.0
    for s in range(n_steps):
        tok, lo, _ = orc.forward(seq[s], want_logits=s in check)
        assert tok == pred[s], f"greedy id differs from the oracle at position {s}"
        if s in check:
            worst = max(worst, rel_err(lg[s].cpu().numpy(), lo))
    assert worst < 1e-3, f"logits deviate {worst:.2e}"
    m.free(); m2.free()


@pytest.mark.parametrize("preset", ["1.5b", "3b"])
def test_context_specific_builds_give_the_bits_of_the_general_build(ctx, pkg, tmp_path, monkeypatch, preset):
    """The decode kernel is compiled once with every attention variant and once per context range with only that
    range's variant (short: dedicated attention CTAs; 257..1024 positions; beyond).  Which one a launch gets depends on
    its positions alone; the results must not: same tokens, same logits bits, also for a launch that straddles two
    ranges and therefore runs on the general build."""
    import torch
    path = gu.make_synthetic(tmp_path / "m.gguf", preset, seed=99)
    V = gu.GgufReader(path).config()["n_vocab"]
    rng = np.random.default_rng(5)
    n = 6
    for pos0 in (40, 253, 300, 1020, 1100, 2500):
        res = []
        for general in (False, True):
            if general:
                monkeypatch.setenv("MINFER_NO_LEAN", "1")
            else:
                monkeypatch.delenv("MINFER_NO_LEAN", raising=False)
            m = pkg.Model(ctx, path, 2600)
            # the same arbitrary cache content for both runs
            torch.manual_seed(pos0)
            for name in ("kcache", "vcache"):
                t = m.state_tensor(name).view(torch.float16)
                t.copy_((torch.randn(t.numel(), device="cuda") * 0.5).to(torch.float16))
            logits = torch.zeros((n, V), dtype=torch.float32, device="cuda")
            toks = [int(t) for t in np.random.default_rng(pos0).integers(0, V, 2)]
            out, _ = m.decode(toks, n, pos0, logits)
            res.append((out, logits.cpu().numpy().copy()))
            if pos0 in (253, 1020) and not general:
                # a run that passes a range boundary is two launches: ring entries and margins continue across the cut
                mg = m.margins(n).copy()
                ring = pkg.TokenRing(ctx, n)
                m.decode_run(toks, n, pos0, ring)
                ctx.sync()
                k, rt, rm, _ = ring.peek()
                assert k == n and rt == out and np.array_equal(np.array(rm, dtype=np.float32), mg)
                ring.free()
            m.free()
        assert res[0][0] == res[1][0], f"tokens differ at position {pos0}"
        assert np.array_equal(res[0][1].view(np.uint32), res[1][1].view(np.uint32)), f"logits differ at position {pos0}"
    monkeypatch.delenv("MINFER_NO_LEAN", raising=False)


def test_a_long_run_through_every_context_range_matches_the_general_build(ctx, pkg, tmp_path, monkeypatch):
    """1100 generated tokens after an 8-token prompt pass 256 and 1024 cached positions: three launches of three builds
    on one side, one launch of the general build on the other, the same ids."""
    path = gu.make_synthetic(tmp_path / "m.gguf", "1.5b", seed=4)
    V = gu.GgufReader(path).config()["n_vocab"]
    prompt = [int(t) for t in np.random.default_rng(8).integers(0, V, 8)]
    outs = []
    for general in (False, True):
        if general:
            monkeypatch.setenv("MINFER_NO_LEAN", "1")
        else:
            monkeypatch.delenv("MINFER_NO_LEAN", raising=False)
        m = pkg.Model(ctx, path, 1200)
        out, _ = m.decode(prompt, 1108, 0)
        outs.append(out)
        m.free()
    monkeypatch.delenv("MINFER_NO_LEAN", raising=False)
    assert outs[0] == outs[1]
