"""ctypes access to the CPU checker: oracle/_build/liboracle.so (the C restatement)
and, where it was built, oracle/_ref/libref_ops.so (the reference's own functions).

Test infrastructure only: nothing on the product path imports this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_SO = ROOT / "oracle" / "_build" / "liboracle.so"
REF_OPS_SO = ROOT / "oracle" / "_ref" / "libref_ops.so"
REF_CPU_INFER = ROOT / "oracle" / "_ref" / "cpu_infer"

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        if not ORACLE_SO.exists():
            r = subprocess.run(["make", "-C", str(ROOT / "oracle"), "all"], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("cannot build the oracle:\n" + r.stdout + r.stderr)
        L = C.CDLL(str(ORACLE_SO))
        L.orc_fp16_to_fp32.restype, L.orc_fp16_to_fp32.argtypes = _f32, [C.c_uint16]
        L.orc_fp32_to_fp16.restype, L.orc_fp32_to_fp16.argtypes = C.c_uint16, [_f32]
        L.orc_dequant_row_q4_0.argtypes = [_vp, _i64, _vp]
        L.orc_quantize_row_q4_0.argtypes = [_vp, _i64, _vp]
        L.orc_dequant_row_t.restype, L.orc_dequant_row_t.argtypes = _i32, [_i32, _vp, _i64, _vp]
        L.orc_requant_row_q4_0.argtypes = [_vp, _i64, _vp]
        L.orc_quant_q8.argtypes = [_vp, _i64, _vp, _vp]
        L.orc_block_isums.argtypes = [_vp, _i64, _i64, _vp, _vp]
        L.orc_gemv_q4_q8.argtypes = [_vp, _i64, _i64, _vp, _vp, _vp, _vp]
        L.orc_matvec_f32.argtypes = [_vp, _i64, _i64, _vp, _vp]
        L.orc_rmsnorm.argtypes = [_vp, _vp, _i32, _f32, _vp]
        L.orc_rope.argtypes = [_vp, _i32, _i32, _i32, _f32]
        L.orc_attention.argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]
        L.orc_state_new.restype, L.orc_state_new.argtypes = _vp, [_vp, _i32, _i32, _i32]
        L.orc_state_free.argtypes = [_vp]
        L.orc_forward.restype, L.orc_forward.argtypes = _i32, [_vp, _vp, _i32, _i32, _vp, _vp]
        L.orc_num_threads.restype = _i32
        L.orc_state_kc.restype, L.orc_state_kc.argtypes = C.POINTER(C.c_float), [_vp]
        L.orc_state_vc.restype, L.orc_state_vc.argtypes = C.POINTER(C.c_float), [_vp]
        _lib = L
    return _lib


def have_ref():
    return REF_OPS_SO.exists() and REF_CPU_INFER.exists()


def ref():
    """The reference's own functions (only where oracle/_ref was built)."""
    global _ref
    if _ref is None:
        R = C.CDLL(str(REF_OPS_SO))
        R.ref_matvec_q4_0.argtypes = [_vp, _i64, _i64, _vp, _vp]
        R.ref_dequant_row_q4_0.argtypes = [_vp, _i64, _i64, _i64, _vp]
        R.ref_rmsnorm.argtypes = [_vp, _vp, _i32, _f32, _vp]
        R.ref_rope.argtypes = [_vp, _i32, _i32, _i32, _f32]
        R.ref_add_bias.argtypes = [_vp, _vp, _i32]
        R.ref_fp16_to_fp32.restype, R.ref_fp16_to_fp32.argtypes = _f32, [C.c_uint16]
        R.ref_dequant_row.argtypes = [C.c_uint32, _vp, _i64, _i64, _i64, _vp]
        _ref = R
    return _ref


def _p(a):
    return a.ctypes.data if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---- numpy-level wrappers of the restatement ----------------------------------

def quantize_q4_0(W):
    """fp32 [rows, cols] -> raw GGUF q4_0 bytes, uint8 [rows*(cols/32)*18]."""
    W = _c(W, np.float32)
    rows, cols = W.shape
    out = np.empty(rows * (cols // 32) * 18, dtype=np.uint8)
    lib().orc_quantize_row_q4_0(_p(W), rows * cols, _p(out))
    return out


def dequant_q4_0(raw, rows, cols):
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_dequant_row_q4_0(_p(raw), rows * (cols // 32), _p(out))
    return out


def quant_q8(x):
    x = _c(x, np.float32).reshape(-1)
    xq = np.empty(x.size, dtype=np.int8)
    xd = np.empty(x.size // 32, dtype=np.uint16)
    lib().orc_quant_q8(_p(x), x.size, _p(xq), _p(xd))
    return xq, xd


def block_isums(raw, rows, cols, xq):
    out = np.empty((rows, cols // 32), dtype=np.int32)
    lib().orc_block_isums(_p(raw), rows, cols, _p(xq), _p(out))
    return out


def gemv_q4_q8(raw, rows, cols, xq, xd, bias=None):
    y = np.empty(rows, dtype=np.float32)
    b = _c(bias, np.float32) if bias is not None else None
    lib().orc_gemv_q4_q8(_p(raw), rows, cols, _p(xq), _p(xd), _p(b), _p(y))
    return y


def matvec_f32(raw, rows, cols, x):
    y = np.empty(rows, dtype=np.float32)
    x = _c(x, np.float32)
    lib().orc_matvec_f32(_p(raw), rows, cols, _p(x), _p(y))
    return y


def rmsnorm(x, w, eps):
    x, w = _c(x, np.float32), _c(w, np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), x.size, eps, _p(out))
    return out


def rope(v, n_head, hd, pos, base):
    v = _c(v, np.float32).copy()
    lib().orc_rope(_p(v), n_head, hd, pos, base)
    return v


def attention(q, kc, vc, pos, n_head, n_head_kv, hd):
    q, kc, vc = _c(q, np.float32), _c(kc, np.float32), _c(vc, np.float32)
    att = np.empty(n_head * hd, dtype=np.float32)
    lib().orc_attention(_p(q), _p(kc), _p(vc), pos, n_head, n_head_kv, hd, _p(att))
    return att


def f16_bits_to_f32(bits):
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


# ---- whole model ---------------------------------------------------------------

class _OrcModel(C.Structure):
    _fields_ = [(n, _i32) for n in ("n_layer", "n_embd", "n_ff", "n_head", "n_head_kv", "head_dim", "n_vocab")] + \
               [("rope_base", _f32), ("rms_eps", _f32), ("tok_emb", _vp), ("out_w", _vp), ("out_norm", _vp)] + \
               [(n, _vp) for n in ("attn_norm", "ffn_norm", "wq", "wk", "wv", "wo", "bq", "bk", "bv", "wg", "wu", "wd")] + \
               [("tok_emb_type", _i32)]


class OracleModel:
    """Runs the restated forward pass on the tensors of a parsed GGUF file
    (tests/gguf_util.GgufReader).  Matrices stored as Q4_1, Q8_0 or Q6_K are re-quantized to q4_0 the way the reference's
    loader does (src/mega.cu:986-993); a Q8_0 token embedding is read as it is (src/mega.cu:1110-1111)."""

    def __init__(self, g, act_q8, kv_f16, max_seq):
        self.g = g
        cfg = g.config()
        self.cfg = cfg
        L = cfg["n_layer"]
        self._keep = []

        def arr(name, keep_q8=False):
            a = g.tensor_bytes(name)
            typ, rows, cols = g.shape(name)
            if typ not in (0, 2) and not (keep_q8 and typ == 8):
                fmt = {t: f for f, (t, _, _) in BLOCK_FORMATS.items()}[typ]
                a = requant_q4_0(dequant_rows(fmt, a, rows, cols))
            self._keep.append(a)
            return a.ctypes.data

        def parr(fmt):
            pa = (_vp * L)(*[arr(fmt.format(i)) for i in range(L)])
            self._keep.append(pa)
            return C.cast(pa, _vp)

        m = _OrcModel()
        for k in ("n_layer", "n_embd", "n_ff", "n_head", "n_head_kv", "head_dim", "n_vocab"):
            setattr(m, k, cfg[k])
        m.rope_base, m.rms_eps = cfg["rope_base"], cfg["rms_eps"]
        m.tok_emb, m.out_w, m.out_norm = arr("token_embd.weight", True), arr("output.weight"), arr("output_norm.weight")
        m.tok_emb_type = g.shape("token_embd.weight")[0]
        m.attn_norm, m.ffn_norm = parr("blk.{}.attn_norm.weight"), parr("blk.{}.ffn_norm.weight")
        m.wq, m.wk, m.wv, m.wo = (parr(f"blk.{{}}.attn_{n}.weight") for n in ("q", "k", "v", "output"))
        m.bq, m.bk, m.bv = (parr(f"blk.{{}}.attn_{n}.bias") for n in ("q", "k", "v"))
        m.wg, m.wu, m.wd = (parr(f"blk.{{}}.ffn_{n}.weight") for n in ("gate", "up", "down"))
        self.m = m
        self.state = lib().orc_state_new(C.byref(m), max_seq, int(act_q8), int(kv_f16))
        self.pos = 0

    def forward(self, token, want_logits=True, want_hidden=False):
        cfg = self.cfg
        logits = np.empty(cfg["n_vocab"], dtype=np.float32) if want_logits else None
        hidden = np.empty((cfg["n_layer"], cfg["n_embd"]), dtype=np.float32) if want_hidden else None
        tok = lib().orc_forward(C.byref(self.m), self.state, int(token), self.pos, _p(logits), _p(hidden))
        self.pos += 1
        return tok, logits, hidden

    def kv_cache(self, max_seq):
        """(K, V) caches as [layer][max_seq][kv_dim] float32 views."""
        cfg = self.cfg
        shape = (cfg["n_layer"], max_seq, cfg["n_head_kv"] * cfg["head_dim"])
        n = int(np.prod(shape))
        return (np.ctypeslib.as_array(lib().orc_state_kc(self.state), shape=(n,)).reshape(shape),
                np.ctypeslib.as_array(lib().orc_state_vc(self.state), shape=(n,)).reshape(shape))

    def generate(self, prompt, n_gen):
        """Greedy continuation exactly as the reference CLI prints it: n_gen ids,
        the first being the prediction after the last prompt token."""
        nxt = -1
        for t in prompt:
            nxt, _, _ = self.forward(t, want_logits=False)
        out = []
        for _ in range(n_gen):
            out.append(nxt)
            nxt, _, _ = self.forward(nxt, want_logits=False)
        return out

    def close(self):
        if self.state:
            lib().orc_state_free(self.state)
            self.state = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def run_ref_cpu_infer(gguf_path, n_gen, prompt, threads=None, timeout=3600):
    """Run the reference's unmodified cpu_infer program; returns (ids, wall seconds)."""
    import os
    import time
    env = dict(os.environ)
    if threads:
        env["OMP_NUM_THREADS"] = str(threads)
    t0 = time.time()
    r = subprocess.run([str(REF_CPU_INFER), str(gguf_path), str(n_gen), *[str(t) for t in prompt]],
                       capture_output=True, text=True, env=env, timeout=timeout)
    dt = time.time() - t0
    if r.returncode != 0:
        raise RuntimeError("cpu_infer failed: " + r.stderr)
    return [int(t) for t in r.stdout.split()], dt


# ---- other block formats (real model files): bytes per block, elements per block, ggml type id
BLOCK_FORMATS = {"q4_1": (3, 20, 32), "q8_0": (8, 34, 32), "q6_k": (14, 210, 256)}


def random_blocks(fmt, rows, cols, rng):
    """Random but well-formed raw blocks of a format: random quant bytes, small positive fp16 scales (and small mins)."""
    tid, bpb, epb = BLOCK_FORMATS[fmt]
    nblk = rows * (cols // epb)
    raw = rng.integers(0, 256, size=(nblk, bpb), dtype=np.uint8)
    sc = np.float16(rng.uniform(0.001, 0.02, nblk)).view(np.uint16)
    if fmt == "q4_1":
        raw[:, 0:2] = sc.view(np.uint8).reshape(-1, 2)
        raw[:, 2:4] = np.float16(rng.uniform(-0.1, 0.0, nblk)).view(np.uint8).reshape(-1, 2)
    elif fmt == "q8_0":
        raw[:, 0:2] = sc.view(np.uint8).reshape(-1, 2)
    else:
        raw[:, 208:210] = np.float16(rng.uniform(1e-4, 1e-3, nblk)).view(np.uint8).reshape(-1, 2)
    return np.ascontiguousarray(raw.reshape(-1))


def dequant_rows(fmt, raw, rows, cols):
    """The oracle's dequantization of every row (float32 [rows][cols])."""
    tid, bpb, epb = BLOCK_FORMATS[fmt]
    out = np.empty((rows, cols), np.float32)
    rb = cols // epb * bpb
    for r in range(rows):
        assert lib().orc_dequant_row_t(tid, raw[r * rb:].ctypes.data, cols, out[r].ctypes.data) == 0
    return out


def requant_q4_0(y):
    """The reference's q4_0 re-quantizer (amax/7, lrintf + 8) as restated by the oracle: float32 [rows][cols] -> raw q4_0 bytes."""
    y = np.ascontiguousarray(y, np.float32)
    rows, cols = y.shape
    out = np.empty(rows * (cols // 32) * 18, np.uint8)
    for r in range(rows):
        lib().orc_requant_row_q4_0(y[r].ctypes.data, cols, out[r * (cols // 32) * 18:].ctypes.data)
    return out
