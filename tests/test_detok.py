"""The detokenizer is host code behind the C ABI (mi_detok_piece): it needs the library but no GPU.  Checked against the
published GPT-2 byte-to-unicode table written out here in Python, and on the malformed inputs whose treatment the
reference fixes (src/detok.h:27-41)."""
import pytest

import gguf_util as gu


def byte_to_unicode():
    """GPT-2's table: printable non-space Latin-1 bytes map to themselves, the rest to 256, 257, ... in byte order."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    return table


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


def test_every_byte_round_trips(pkg):
    t = byte_to_unicode()
    assert len(set(t.values())) == 256 and max(ord(c) for c in t.values()) == 323
    for b in range(256):
        assert pkg.detok_piece(t[b]) == bytes([b])
    text = "Hello, wörld!\n\t日本語 🙂 \x00\x7f".encode("utf-8")
    piece = "".join(t[b] for b in text)
    assert pkg.detok_piece(piece) == text
    assert pkg.detok_piece("") == b""


def test_malformed_pieces_follow_the_reference_rules(pkg):
    # stray continuation bytes and bytes that cannot start a sequence are skipped
    assert pkg.detok_piece(b"\x80\xbfA\xf8\xffB") == b"AB"
    # code points outside the table (here U+0144 = 324 and U+20AC) emit nothing
    assert pkg.detok_piece("ańb€c") == b"abc"
    # the last table entry, U+0143 = 323, is byte 0xAD (the last of the 68 remapped bytes)
    assert pkg.detok_piece("Ń") == b"\xad"
    # a sequence cut short by the end of the piece is decoded from what is there: 0xC4 alone is code point 4, not in the table
    assert pkg.detok_piece(b"ok\xc4") == b"ok"
    # a 4-byte sequence maps far outside the table
    assert pkg.detok_piece("x\U0001F642y") == b"xy"


def test_synthetic_vocabulary_spells_bytes_and_words(pkg, tmp_path):
    if not gu.SYNTH.exists():
        pytest.skip("gguf_synth not built")
    g = gu.GgufReader(gu.make_synthetic(tmp_path / "v.gguf", "tiny", seed=1, extra=["--eos", 77]))
    assert int(g.meta["tokenizer.ggml.eos_token_id"]) == 77
    toks = g.tokens
    assert len(toks) == 512
    for b in range(256):
        assert pkg.detok_piece(toks[b]) == bytes([b])
    assert pkg.detok_piece(toks[300]) == b" t300"
