"""Loading model files that are not all q4_0: the device re-quantizer against the oracle's restatement of the reference's
host loop (dequantize a row per src/gguf.h:103-140, quantize it per src/mega.cu:924-936), and whole models whose
embedding, lm_head and ffn_down are stored as Q8_0 / Q6_K / Q4_1 like published files.

Bars: q4_0 bytes identical; greedy streams identical to the q8 oracle; logits within 1e-3 relative.
"""
from pathlib import Path

import numpy as np
import pytest

import gguf_util as gu
import oracle_util as ou

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
SHAPE = ["--layers", 2, "--embd", 256, "--ff", 512, "--heads", 4, "--kv-heads", 2, "--vocab", 640, "--bias-std", 0.05]


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("fmt", sorted(ou.BLOCK_FORMATS))
def test_requantizer_reproduces_the_reference_fixture(ctx, fmt):
    """The fixture holds what the reference's own dequant_row and quant_row_q4_0 made of these blocks."""
    import torch
    fx = np.load(GOLD / "requant_ref.npz")
    rows, cols = (int(v) for v in fx["shape"])
    src = torch.from_numpy(fx[f"{fmt}_raw"].copy()).cuda()
    dst = torch.zeros(rows * (cols // 32) * 18, dtype=torch.uint8, device="cuda")
    ctx.requant_q4_0(ou.BLOCK_FORMATS[fmt][0], src, rows, cols, dst)
    ctx.sync()
    assert np.array_equal(dst.cpu().numpy().reshape(rows, -1), fx[f"{fmt}_q4"])


@pytest.mark.parametrize("fmt,rows,cols", [("q4_1", 97, 1536), ("q8_0", 33, 8960), ("q6_k", 64, 1536), ("q6_k", 1, 256), ("q8_0", 1, 32)])
def test_requantizer_matches_the_oracle_on_seeded_blocks(ctx, fmt, rows, cols):
    import torch
    rng = np.random.default_rng(rows * 131 + cols)
    raw = ou.random_blocks(fmt, rows, cols, rng)
    want = ou.requant_q4_0(ou.dequant_rows(fmt, raw, rows, cols))
    dst = torch.zeros(want.size, dtype=torch.uint8, device="cuda")
    ctx.requant_q4_0(ou.BLOCK_FORMATS[fmt][0], torch.from_numpy(raw).cuda(), rows, cols, dst)
    ctx.sync()
    assert np.array_equal(dst.cpu().numpy(), want)


def test_requantizer_all_zero_blocks_and_argument_checks(ctx, pkg):
    import torch
    z = torch.zeros(34 * 4, dtype=torch.uint8, device="cuda")
    dst = torch.full((18 * 4,), 0xEE, dtype=torch.uint8, device="cuda")
    ctx.requant_q4_0(8, z, 1, 128, dst)
    ctx.sync()
    out = dst.cpu().numpy().reshape(4, 18)
    assert np.all(out[:, :2] == 0) and np.all(out[:, 2:] == 0x88)          # scale 0, every value 0
    with pytest.raises(pkg.MinferError):
        ctx.requant_q4_0(14, z, 1, 128, dst)                                # Q6_K rows are multiples of 256
    with pytest.raises(pkg.MinferError):
        ctx.requant_q4_0(2, z, 1, 128, dst)                                 # q4_0 needs no re-quantizer


MIXES = [
    ("published layout: Q8_0 embedding kept, Q6_K head, Q4_1 ffn_down", ["--emb-type", 8, "--head-type", 14, "--down-type", 3]),
    ("tied Q8_0 embedding and head", ["--emb-type", 8, "--head-type", 8]),
    ("tied Q6_K embedding and head, Q8_0 ffn_down", ["--emb-type", 14, "--head-type", 14, "--down-type", 8]),
    ("untied q4_0 head, Q4_1 embedding", ["--emb-type", 3, "--head-type", 2, "--down-type", 14]),
]


@pytest.mark.parametrize("name,extra", MIXES, ids=[m[0].split(":")[0] for m in MIXES])
def test_mixed_type_model_matches_the_oracle(ctx, pkg, tmp_path, name, extra):
    import torch
    path = gu.make_synthetic(tmp_path / "mix.gguf", "tiny", seed=77, std=0.1, extra=SHAPE + extra)
    g = gu.GgufReader(path)
    prompt, n_gen = [5, 17, 300, 9], 20
    n_steps = len(prompt) + n_gen - 1
    want = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=n_steps + 1).generate(prompt, n_gen)
    m = pkg.Model(ctx, path, max_seq=n_steps + 1)
    for mode in (pkg.DECODE_PERSISTENT, pkg.DECODE_PER_PHASE):
        got, _ = m.generate(prompt, n_gen, mode=mode)
        assert got == want, name
    # teacher-forced logits, single-token and M-token paths
    seq = prompt + want[:-1]
    orc = ou.OracleModel(g, act_q8=True, kv_f16=True, max_seq=n_steps + 1)
    ref = np.stack([orc.forward(t)[1] for t in seq])
    logits = torch.zeros((n_steps, g.config()["n_vocab"]), dtype=torch.float32, device="cuda")
    m.decode(seq, n_steps, 0, logits, pkg.DECODE_PERSISTENT)
    assert rel_err(logits.cpu().numpy(), ref) < 1e-3
    lv = torch.zeros((8, g.config()["n_vocab"]), dtype=torch.float32, device="cuda")
    pred, _ = m.verify(seq[:8], 0, lv)
    assert rel_err(lv.cpu().numpy(), ref[:8]) < 1e-3
    assert pred == [int(np.argmax(r)) for r in ref[:8]]


def test_unsupported_matrix_type_is_refused(ctx, pkg, tmp_path):
    """A Q6_K tensor whose rows are not multiples of 256 cannot exist; an F16 matrix is outside this path."""
    path = gu.make_synthetic(tmp_path / "ok.gguf", "tiny", seed=3, std=0.1)
    raw = bytearray(Path(path).read_bytes())
    g = gu.GgufReader(path)
    # patch the stored type of blk.0.ffn_up.weight from 2 (Q4_0) to 1 (F16) in the tensor table
    name = b"blk.0.ffn_up.weight"
    at = raw.find(name) + len(name)
    n_dims = int.from_bytes(raw[at:at + 4], "little")
    tpos = at + 4 + 8 * n_dims
    assert int.from_bytes(raw[tpos:tpos + 4], "little") == 2
    raw[tpos:tpos + 4] = (1).to_bytes(4, "little")
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(bytes(raw))
    with pytest.raises(pkg.MinferError) as e:
        pkg.Model(ctx, str(bad), max_seq=8)
    assert "type 1" in str(e.value)
    del g
