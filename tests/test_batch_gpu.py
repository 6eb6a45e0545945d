"""Batched decode of independent sequences (the batched configuration of the benchmark definition): every sequence of a
batch must get, bit for bit, the ids and logits of its own batch-1 run, whatever shares the weight pass with it."""
import json
from pathlib import Path

import numpy as np
import pytest

import gguf_util as gu
import oracle_util as ou

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = tmp_path_factory.mktemp("bmodels")
    c = json.loads((GOLD / "streams_ref.json").read_text())[2]
    return gu.make_synthetic(d / "tiny.gguf", c["preset"], seed=c["seed"], std=c["std"], extra=["--bias-std", c["bias_std"]])


def run_batch(pkg, ctx, path, prompts, n_gen, max_seq, V, want_logits_at=()):
    """Sequences with ragged prompts advance together, one token per step each: prompt tokens first, then their own
    greedy tokens.  Returns per sequence the generated ids and the logits of the steps in want_logits_at."""
    import torch
    m = pkg.Model(ctx, path, 8)
    bt = pkg.Batch(m, len(prompts), max_seq)
    B = len(prompts)
    cur = [p[0] for p in prompts]
    pos = [0] * B
    gen = [[] for _ in range(B)]
    kept = [dict() for _ in range(B)]
    logits = torch.zeros((B, V), dtype=torch.float32, device="cuda")
    steps = max(len(p) for p in prompts) + n_gen - 1
    for s in range(steps):
        live = [i for i in range(B) if len(gen[i]) < n_gen]
        if not live:
            break
        out, _ = bt.step([cur[i] for i in live], live, [pos[i] for i in live], logits)
        lg = logits.cpu().numpy()
        for j, i in enumerate(live):
            if pos[i] in want_logits_at:
                kept[i][pos[i]] = lg[j].copy()
            pos[i] += 1
            if pos[i] < len(prompts[i]):
                cur[i] = prompts[i][pos[i]]
            else:
                gen[i].append(out[j]); cur[i] = out[j]
    bt.free(); m.free()
    return gen, kept


@pytest.mark.parametrize("B", [3, 16, 21])
def test_every_sequence_of_a_batch_gets_its_batch_1_bits(ctx, pkg, tiny, B):
    import torch
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    rng = np.random.default_rng(B)
    prompts = [[int(t) for t in rng.integers(0, V, int(rng.integers(3, 12)))] for _ in range(B)]
    n_gen = 10
    at = (2, 7, 12)
    gen, kept = run_batch(pkg, ctx, tiny, prompts, n_gen, 40, V, at)
    for i in (0, B // 2, B - 1):                                   # batch-1 runs of three of the sequences, single-token decode kernel
        m = pkg.Model(ctx, tiny, 40)
        n_steps = len(prompts[i]) + n_gen - 1
        lg = torch.zeros((n_steps, V), dtype=torch.float32, device="cuda")
        want, _ = m.generate(prompts[i], n_gen)
        assert gen[i] == want, f"sequence {i} of a batch of {B}"
        seq = prompts[i] + want[:-1]
        m.decode(seq, n_steps, 0, lg, pkg.DECODE_PERSISTENT)
        ref = lg.cpu().numpy()
        for p_, row in kept[i].items():
            assert np.array_equal(row.view(np.uint32), ref[p_].view(np.uint32)), f"sequence {i}, position {p_}: logits differ from the batch-1 run"
        m.free()


def test_two_sequences_against_the_oracle(ctx, pkg, tiny):
    g = gu.GgufReader(tiny)
    V = g.config()["n_vocab"]
    rng = np.random.default_rng(77)
    prompts = [[int(t) for t in rng.integers(0, V, 9)], [int(t) for t in rng.integers(0, V, 5)]]
    gen, _ = run_batch(pkg, ctx, tiny, prompts, 32, 64, V)
    for i, p in enumerate(prompts):
        want = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=64).generate(p, 32)
        assert gen[i] == want, f"sequence {i} differs from the q8 oracle"


def test_batch_argument_checks(ctx, pkg, tiny):
    m = pkg.Model(ctx, tiny, 8)
    bt = pkg.Batch(m, 4, 16)
    with pytest.raises(pkg.MinferError):
        bt.step([1, 2], [0, 0], [0, 0])             # one slot twice
    with pytest.raises(pkg.MinferError):
        bt.step([1], [4], [0])                      # slot out of range
    with pytest.raises(pkg.MinferError):
        bt.step([1], [0], [16])                     # position outside the slab
    bt.free(); m.free()
