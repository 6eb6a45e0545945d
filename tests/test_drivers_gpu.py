"""The driver programs (bin/cuda_infer, bin/mega) are the reference's real boundary: same command line, environment
knobs, stdout and the stderr line shapes its scripts parse.  These tests run the executables on the golden tiny models
and read their output with the very regular expressions of the reference's tools/ab.sh (lines 38-41, 49-51) and
tools/specbench.sh (lines 21, 35); they also cover the token ring and the speculative loop through the C ABI."""
import json
import os
import re
import subprocess
import time
from pathlib import Path

import numpy as np
import pytest

import gguf_util as gu
import oracle_util as ou

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "nano-inference_b200" / "bin"
GOLD = Path(__file__).resolve().parent / "golden"


def run_driver(exe, model, n_gen, ids, **env):
    e = dict(os.environ, RAWIDS="1", WARMUP="1", **{k: str(v) for k, v in env.items()})
    r = subprocess.run([str(BIN / exe), str(model), str(n_gen), *[str(i) for i in ids]], capture_output=True, text=True, env=e, timeout=300)
    assert r.returncode == 0, r.stderr
    return r.stdout, r.stderr


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    d = tmp_path_factory.mktemp("drv")
    out = []
    for i, c in enumerate(json.loads((GOLD / "streams_ref.json").read_text())):
        p = gu.make_synthetic(d / f"m{i}.gguf", c["preset"], seed=c["seed"], std=c["std"], extra=["--bias-std", c["bias_std"]])
        out.append((p, c))
    return out


@pytest.mark.parametrize("exe", ["cuda_infer", "mega"])
def test_stdout_is_the_oracle_stream(cases, exe):
    for path, c in cases:
        g = gu.GgufReader(path)
        want = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=len(c["prompt"]) + c["n_gen"] + 1).generate(c["prompt"], c["n_gen"])
        for spec in (0, 1):
            out, err = run_driver(exe, path, c["n_gen"], c["prompt"], SPEC=spec)
            got = [int(t) for t in out.split()]
            assert got == want, f"{exe} SPEC={spec} on the std-{c['std']} model"
            if c["std"] <= 0.1:
                assert got == c["ref_ids"], "differs from the stream the reference's cpu_infer printed"
            # tools/ab.sh:38 and :40, tools/specbench.sh:21
            assert re.search(r"= ([\d.]+) tok/s", err)
            if exe == "mega":
                assert re.search(r"decode: .*= ([\d.]+) tok/s", err)
                assert "first token after" in err and re.search(r"min logit margin -?[\d.]+ at #\d+", err)


def test_speculation_is_lossless_and_accepts_drafts_where_the_stream_repeats(cases):
    """tools/specbench.sh:33-36: SPEC=1 stdout == SPEC=0 stdout.  The std-0.02 model's greedy stream is one repeated
    token (as the reference's cpu_infer prints it too), so prompt-lookup drafts are accepted there and a step yields
    several tokens; the livelier models exercise rejection."""
    for idx, (path, c) in enumerate(cases):
        outs = {}
        # SPEC=1 lets the loop's cost model pick the draft length (on these two-layer models a pass costs several single
        # steps, so it may pick none); SPEC=2 submits every draft in full, which is what exercises acceptance here
        for spec in (0, 1, 2):
            out, err = run_driver("mega", path, 48, c["prompt"], SPEC=spec, DRAFTK=8, MAXSEQ=128)
            outs[spec] = out
            m = re.search(r"(\d+) generation steps, ([\d.]+) tokens/step \| drafted (\d+), accepted (\d+)", err)      # tools/specbench.sh:35
            assert m, err
            steps, tps, drafted, accepted = int(m.group(1)), float(m.group(2)), int(m.group(3)), int(m.group(4))
            if spec == 0:
                assert "[SPEC=0]" in err and steps == 48 and drafted == 0
            else:
                assert accepted <= drafted and steps <= 48
                if idx == 0 and spec == 2:
                    assert accepted > 0 and steps < 48 and tps > 1.5, f"no draft accepted on a constant stream: {m.group(0)}"
        assert outs[0] == outs[1] == outs[2], f"speculation changed the generated ids on the std-{c['std']} model"


def test_generate_spec_equals_plain_decode_and_counts_accepted_tokens(ctx, pkg, cases):
    path, c = cases[2]
    g = gu.GgufReader(path)
    V = g.config()["n_vocab"]
    m = pkg.Model(ctx, path, 256)
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, V, 20)]
    plain, _ = m.generate(prompt, 100)
    plain_margins = None
    for ngmax, draftk in ((3, 4), (1, 15), (2, 8), (3, -4), (2, -15)):         # negative: every draft submitted in full
        got, st = m.generate_spec(prompt, 100, ngmax=ngmax, draftk=draftk)
        assert got == plain, f"NGMAX={ngmax} DRAFTK={draftk}"
        assert st["accepted"] <= st["drafted"] and st["steps"] <= 100
        if plain_margins is None:
            plain_margins = st["margins"]
        else:
            assert np.array_equal(plain_margins, st["margins"]), "margins depend on how the tokens were grouped into passes"
    got0, st0 = m.generate_spec(prompt, 100, ngmax=3, draftk=0)
    assert got0 == plain and st0["drafted"] == 0 and st0["steps"] == 100
    m.free()


def test_teacher_mode_hash_is_independent_of_tokens_per_pass(cases):
    path, c = cases[1]
    seq = c["prompt"] + c["ref_ids"]
    hashes, lines = set(), []
    for exe in ("mega", "cuda_infer"):
        for tchunk in (1, 8, 16):
            _, err = run_driver(exe, path, 1, seq, TEACHER=len(c["prompt"]), TCHUNK=tchunk)
            line = next(l for l in err.splitlines() if "agreement" in l)
            a = re.sub(r".*: ([0-9]*)/([0-9]*).*", r"\1", line); b = re.sub(r".*/([0-9]*).*", r"\1", line)        # tools/ab.sh:50-51 (sed)
            assert int(b) == len(c["ref_ids"]) and 0 <= int(a) <= int(b)
            hashes.add(re.search(r"logit hash ([0-9a-f]{16})", line).group(1))
            for miss in (l for l in err.splitlines() if l.startswith("  pos ")):
                assert re.match(r"  pos \d+: ref \d+, \w+ \d+ \(\w+ margin -?[\d.]+\)", miss)                   # tools/ab.sh:49
    assert len(hashes) == 1, f"logits differ between engines or tokens per pass: {hashes}"


def test_margins_line_and_segments_parse_like_the_ab_harness(cases):
    path, c = cases[0]
    for spec in (0, 1):
        out, err = run_driver("mega", path, 24, c["prompt"], MARGINS=1, SEGMENTS=8, SPEC=spec)
        ids = [int(t) for t in out.split()]
        # tools/ab.sh:41 - the last stderr line is "i:tok:margin ..."
        marg = dict((int(x.split(":")[0]), (int(x.split(":")[1]), float(x.split(":")[2]))) for x in err.strip().split("\n")[-1].split())
        assert sorted(marg) == list(range(24)) and [marg[i][0] for i in range(24)] == ids
        assert all(v[1] >= 0 for v in marg.values())
        if spec == 0:
            assert re.search(r"tokens\s+0-\s+8 \(pos\s+\d+\): [\d.]+ tok/s", err)


def test_ring_delivers_the_tokens_of_a_plain_decode_while_the_kernel_runs(ctx, pkg, cases):
    path, c = cases[2]
    V = gu.GgufReader(path).config()["n_vocab"]
    m = pkg.Model(ctx, path, 512)
    prompt = [int(t) for t in np.random.default_rng(9).integers(0, V, 8)]
    n = 300
    want, _ = m.decode(prompt, n, 0)
    want_margins = m.margins(n).copy()
    m2 = pkg.Model(ctx, path, 512)
    ring = pkg.TokenRing(ctx, n + 16)
    m2.decode_run(prompt, n, 0, ring)
    seen_partial = False
    t0 = time.time()
    while True:
        k, toks, mar, ns = ring.peek()
        if 0 < k < n:
            seen_partial = True
        if k >= n or time.time() - t0 > 60:
            break
    ctx.sync()
    k, toks, mar, ns = ring.peek()
    assert k == n and toks == want
    assert np.array_equal(np.array(mar, dtype=np.float32), want_margins)
    assert all(b >= a for a, b in zip(ns, ns[1:])), "time stamps must not go backwards"
    # a second run appends; a run that does not fit is refused
    m2.decode_run([want[-1]], 8, n, ring)
    ctx.sync()
    assert ring.peek()[0] == n + 8
    with pytest.raises(pkg.MinferError):
        m2.decode_run([1], 64, n + 8, ring)
    ring.free(); m.free(); m2.free()


# ---- text mode: detokenized output and the end-of-sequence stop -------------------------------------------------------

def _stream(path, prompt, n_gen):
    g = gu.GgufReader(path)
    return g, ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=len(prompt) + n_gen + 1).generate(prompt, n_gen)


def test_stop_token_ends_every_engine_at_the_same_token(ctx, pkg, tmp_path):
    """mi_model_set_stop_token: the run ends after the step that picks the token; forced positions never stop it."""
    path = gu.make_synthetic(tmp_path / "s.gguf", "tiny", seed=21, std=0.1, extra=["--bias-std", 0.05])
    prompt, n_gen = [3, 7, 100, 41], 24
    g, want = _stream(path, prompt, n_gen)
    k = 9                                               # stop at the 10th generated token's first occurrence
    stop = want[k]
    first = want.index(stop)
    m = pkg.Model(ctx, path, max_seq=len(prompt) + n_gen + 1)
    n_steps = len(prompt) + n_gen - 1
    for mode in (pkg.DECODE_PERSISTENT, pkg.DECODE_PER_PHASE):
        m.set_stop_token(stop)
        out, _ = m.decode(prompt, n_steps, 0, None, mode)
        assert m.last_count() == len(prompt) + first, "the step that produced the stop token is the last"
        assert out[len(prompt) - 1:m.last_count()] == want[:first + 1]
        # the cache and the position bookkeeping stay usable: the same call without the rule gives the whole stream
        m.set_stop_token(-1)
        out, _ = m.decode(prompt, n_steps, 0, None, mode)
        assert m.last_count() == n_steps and out[len(prompt) - 1:] == want
    # a forced position whose prediction equals the stop token does not end the run: force the whole stream
    m.set_stop_token(stop)
    seq = prompt + want[:-1]
    out, _ = m.decode(seq, len(seq), 0, None, pkg.DECODE_PERSISTENT)
    assert m.last_count() == len(seq) and out[len(prompt) - 1:] == want
    # the speculative loop stops at the same token
    got, st = m.generate_spec(prompt, n_gen)
    assert m.last_count() == first + 1 and got[:first + 1] == want[:first + 1]
    # a run that reports through the ring: its count is that of the stopped run
    ring = pkg.TokenRing(ctx, n_steps)
    m.decode_run(prompt, n_steps, 0, ring)
    ctx.sync()
    k, toks, _, _ = ring.peek()
    assert k == len(prompt) + first and toks[len(prompt) - 1:] == want[:first + 1]
    ring.free()
    m.set_stop_token(-1)


@pytest.mark.parametrize("exe", ["cuda_infer", "mega"])
@pytest.mark.parametrize("spec", [0, 1])
def test_text_mode_prints_pieces_and_stops_at_eos(tmp_path, pkg, exe, spec):
    prompt, n_gen = [3, 7, 100, 41], 24
    base = gu.make_synthetic(tmp_path / "a.gguf", "tiny", seed=21, std=0.1, extra=["--bias-std", 0.05])
    g, want = _stream(base, prompt, n_gen)
    eos = want[9]
    first = want.index(eos)
    path = gu.make_synthetic(tmp_path / "b.gguf", "tiny", seed=21, std=0.1, extra=["--bias-std", 0.05, "--eos", eos])
    toks = gu.GgufReader(path).tokens
    text = b"".join(pkg.detok_piece(toks[t]) for t in want[:first])          # the end-of-sequence piece is not printed

    def run(**env):
        e = dict(os.environ, WARMUP="1", SPEC=str(spec))
        e.pop("RAWIDS", None)
        e.update({k: str(v) for k, v in env.items()})
        r = subprocess.run([str(BIN / exe), str(path), str(n_gen), *[str(i) for i in prompt]], capture_output=True, env=e, timeout=300)
        assert r.returncode == 0, r.stderr.decode()
        return r.stdout, r.stderr.decode()

    out, err = run()
    assert out == text + b"\n"
    m = re.search(r"(\d+) generation steps", err)
    assert m and int(m.group(1)) <= first + 1
    # with ids asked for, nothing stops early (src/mega.cu:1017: stop_eos = !raw_ids && !teacher)
    out, _ = run(RAWIDS=1)
    assert [int(t) for t in out.split()] == want
