"""Small numpy GGUF reader for the tests, plus a helper that runs the package's
synthetic-model writer.  Parses the same subset as the reference reader
(reference src/gguf.h:183-222)."""
from __future__ import annotations

import struct
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
SYNTH = ROOT / "nano-inference_b200" / "bin" / "gguf_synth"

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
_BLOCK = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 8: (32, 34), 14: (256, 210)}


class GgufReader:
    def __init__(self, path):
        self.path = str(path)
        self.buf = np.memmap(self.path, dtype=np.uint8, mode="r")
        self.mv = memoryview(self.buf)
        self.pos = 0
        self.meta = {}
        self.n_tokens = 0
        self.tokens = []
        self.tensors = {}
        self._parse()

    def _rd(self, fmt):
        v = struct.unpack_from(fmt, self.mv, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def _str(self):
        n = self._rd("<Q")
        s = bytes(self.mv[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def _value(self, vt, key):
        if vt in _SCALAR:
            v = self._rd(_SCALAR[vt])
            if key:
                self.meta[key] = v
        elif vt == 8:
            v = self._str()
            if key:
                self.meta[key] = v
        elif vt == 9:
            et, n = self._rd("<I"), self._rd("<Q")
            keep = key == "tokenizer.ggml.tokens" and et == 8
            if keep:
                self.n_tokens = n
                self.tokens = []
            for _ in range(n):
                if et == 8:
                    ln = self._rd("<Q")
                    if keep and n <= 65536:          # the pieces of small test vocabularies (bytes; large ones are only counted)
                        self.tokens.append(bytes(self.mv[self.pos:self.pos + ln]))
                    self.pos += ln
                else:
                    self._value(et, "")
        else:
            raise ValueError(f"bad metadata type {vt}")

    def _parse(self):
        if self._rd("<I") != 0x46554747:
            raise ValueError("not a GGUF file")
        self._rd("<I")
        n_tensors, n_kv = self._rd("<Q"), self._rd("<Q")
        for _ in range(n_kv):
            key = self._str()
            self._value(self._rd("<I"), key)
        infos = []
        for _ in range(n_tensors):
            name = self._str()
            nd = self._rd("<I")
            ne = [self._rd("<Q") for _ in range(nd)]
            typ, off = self._rd("<I"), self._rd("<Q")
            infos.append((name, ne, typ, off))
        align = int(self.meta.get("general.alignment", 32))
        start = (self.pos + align - 1) // align * align
        for name, ne, typ, off in infos:
            blk, sz = _BLOCK[typ]
            rows = int(np.prod(ne[1:])) if len(ne) > 1 else 1
            nbytes = rows * (ne[0] // blk) * sz
            self.tensors[name] = (typ, ne, start + off, nbytes)

    def config(self):
        m = self.meta
        n_embd, n_head = int(m["qwen2.embedding_length"]), int(m["qwen2.attention.head_count"])
        return dict(n_layer=int(m["qwen2.block_count"]), n_embd=n_embd, n_ff=int(m["qwen2.feed_forward_length"]),
                    n_head=n_head, n_head_kv=int(m["qwen2.attention.head_count_kv"]), head_dim=n_embd // n_head,
                    n_vocab=int(self.n_tokens), rope_base=float(m.get("qwen2.rope.freq_base", 1e6)),
                    rms_eps=float(m.get("qwen2.attention.layer_norm_rms_epsilon", 1e-6)))

    def tensor_bytes(self, name):
        """Contiguous uint8 copy of the tensor's raw bytes (aligned for ctypes use)."""
        typ, ne, off, nbytes = self.tensors[name]
        return np.array(self.buf[off:off + nbytes], dtype=np.uint8, copy=True)

    def tensor_f32(self, name):
        typ, ne, off, nbytes = self.tensors[name]
        assert typ == 0
        return self.tensor_bytes(name).view(np.float32)

    def shape(self, name):
        typ, ne, _, _ = self.tensors[name]
        rows = int(np.prod(ne[1:])) if len(ne) > 1 else 1
        return typ, rows, int(ne[0])


def make_synthetic(path, preset="tiny", seed=1234, std=0.02, extra=()):
    """Write a synthetic GGUF with the package's writer; returns the path."""
    if not SYNTH.exists():
        raise FileNotFoundError(f"{SYNTH} not built: run `python nano-inference_b200/build.py`")
    cmd = [str(SYNTH), str(path), "--preset", preset, "--seed", str(seed), "--std", str(std), *[str(e) for e in extra]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("gguf_synth failed: " + r.stderr)
    return str(path)
