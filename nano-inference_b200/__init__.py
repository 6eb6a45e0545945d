"""ctypes binding of libminfer_b200.so, the B200-native (sm_100a) quantized decode path.

The product is the CUDA library behind the C ABI of include/minfer_b200.h; this
module only loads it and passes device pointers.  PyTorch is used by callers for
device memory and streams, never for the arithmetic.  There is no CPU fallback:
if the library has not been built, or no GPU is present, calls fail loudly.

The directory name contains a hyphen, so load it with importlib (the repository's
__graft_entry__.load_package() does this) under the module name nano_inference_b200.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libminfer_b200.so"
BIN_DIR = PKG_DIR / "bin"

MI_OK = 0
STATUS_NAMES = {0: "MI_OK", 1: "MI_ERR_INVALID", 2: "MI_ERR_CUDA", 3: "MI_ERR_NOMEM", 4: "MI_ERR_TIMEOUT",
                5: "MI_ERR_IO", 6: "MI_ERR_FORMAT", 7: "MI_ERR_UNSUPPORTED", 8: "MI_ERR_LIMIT"}


class MinferError(RuntimeError):
    def __init__(self, status, where, detail=""):
        self.status = status
        super().__init__(f"{where}: {STATUS_NAMES.get(status, status)} {detail}".strip())


_lib = None

_vp, _i32, _i64 = C.c_void_p, C.c_int, C.c_int64
# name -> (restype, argtypes); every symbol include/minfer_b200.h declares
SIGNATURES = {
    "mi_version": (C.c_char_p, []),
    "mi_strerror": (C.c_char_p, [_i32]),
    "mi_ctx_create": (_i32, [_i32, C.POINTER(_vp)]),
    "mi_ctx_destroy": (_i32, [_vp]),
    "mi_ctx_set_stream": (_i32, [_vp, _vp]),
    "mi_ctx_sync": (_i32, [_vp]),
    "mi_last_error": (C.c_char_p, [_vp]),
    "mi_ctx_set_wait_budget_ns": (_i32, [_vp, C.c_uint64]),
    "mi_probe_read_bw": (_i32, [_vp, C.c_size_t, _i32, _i32, C.POINTER(C.c_float)]),
    "mi_probe_hop_ns": (_i32, [_vp, _i32, C.POINTER(C.c_float)]),
    "mi_model_debug_drop_phase": (_i32, [_vp, _i32]),
    "mi_ctx_sm_count": (_i32, [_vp]),
    "mi_device_malloc": (_i32, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "mi_device_free": (_i32, [_vp, _vp]),
    "mi_memcpy_to_device": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mi_memcpy_to_host": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mi_weight_upload_q4_0": (_i32, [_vp, _vp, _i64, _i64, _i64, C.POINTER(_vp)]),
    "mi_weight_repack_q4_0_dev": (_i32, [_vp, _vp, _i64, _i64, _i64, C.POINTER(_vp)]),
    "mi_weight_download_q4_0": (_i32, [_vp, _vp, _vp]),
    "mi_requant_q4_0": (_i32, [_vp, _i32, _vp, _i64, _i64, _vp]),
    "mi_detok_piece": (_i64, [C.c_char_p, _i64, C.c_char_p, _i64]),
    "mi_model_set_stop_token": (_i32, [_vp, _i32]),
    "mi_model_last_count": (_i32, [_vp]),
    "mi_weight_free": (_i32, [_vp, _vp]),
    "mi_weight_info": (_i32, [_vp, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "mi_quant_q8": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp]),
    "mi_gemv_q4_q8": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "mi_gemv_q4_q8_ex": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32]),
    "mi_gemv_q4_q8_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "mi_gemm_q4_q8": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _vp]),
    "mi_block_isums_q4_q8": (_i32, [_vp, _vp, _vp, _vp]),
    "mi_gemv_q4_f32_host": (_i32, [_vp, _vp, _vp, _vp, _vp]),
    "mi_model_load_gguf": (_i32, [_vp, C.c_char_p, _i32, C.POINTER(_vp)]),
    "mi_model_free": (_i32, [_vp, _vp]),
    "mi_model_info": (_i32, [_vp, _vp]),
    "mi_model_state_ptr": (_i32, [_vp, _i32, C.POINTER(_vp), C.POINTER(_i64)]),
    "mi_decode": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _i32, C.POINTER(C.c_float)]),
    "mi_decode_phases": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32]),
    "mi_decode_margins": (_i32, [_vp, _vp, _i32, _vp]),
    "mi_ring_create": (_i32, [_vp, _i32, C.POINTER(_vp)]),
    "mi_ring_destroy": (_i32, [_vp, _vp]),
    "mi_ring_reset": (_i32, [_vp, _vp]),
    "mi_ring_peek": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp)]),
    "mi_decode_run": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "mi_verify": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp, _vp, C.POINTER(C.c_float)]),
    "mi_generate_spec": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "mi_verify_margins": (_i32, [_vp, _vp, _i32, _vp]),
    "mi_batch_create": (_i32, [_vp, _vp, _i32, _i32, C.POINTER(_vp)]),
    "mi_batch_free": (_i32, [_vp, _vp]),
    "mi_batch_step": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, C.POINTER(C.c_float)]),
    "mi_attn_splitkv": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]),
    "mi_tp_partition": (None, [_i32, _i32, _i32, C.POINTER(_i32), C.POINTER(_i32)]),
    "mi_model_load_gguf_tp": (_i32, [_vp, C.c_char_p, _i32, _i32, _i32, C.POINTER(_vp)]),
    "mi_model_tp_region": (_i32, [_vp, _i32, _i32, C.POINTER(_vp), C.POINTER(_i64)]),
    "mi_decode_launch": (_i32, [_vp, _vp, _i32, _i32, _i32]),
    "mi_decode_launch_fused": (_i32, [_vp, _vp, _i32, _i32, _i32]),
    "mi_model_set_token": (_i32, [_vp, _vp, _i32]),
    "mi_model_set_pos": (_i32, [_vp, _vp, _i32]),
    "mi_model_advance_pos": (_i32, [_vp, _vp, _i32]),
    "mi_model_get_token": (_i32, [_vp, _vp, C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    "mi_tp_pick": (_i32, [_vp, _vp, _vp, _i32]),
    "mi_tp_ipc_handles": (_i32, [_vp, _vp, _vp]),
    "mi_tp_ipc_open": (_i32, [_vp, _vp, _vp]),
    "mi_tp_exchange": (_i32, [_vp, _vp, _i32, _i32]),
}
TP_QKV, TP_PART_O, TP_ACT, TP_PART_DOWN, TP_BEST = range(5)

DECODE_PERSISTENT, DECODE_PER_PHASE = 0, 1
POS_DEVICE = -1          # mi_decode_launch: use the model's device-resident position
STATE = {"h": 0, "q": 1, "att": 2, "kcache": 3, "vcache": 4, "act_q": 5, "act_d": 6, "profile": 7, "h_mid": 8}


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "n_ff", "n_head", "n_head_kv", "head_dim", "n_vocab",
                                          "max_seq", "tied_lm_head", "grid_ctas")] + \
               [("rope_base", C.c_float), ("rms_eps", C.c_float),
                ("q4_weight_bytes_per_token", C.c_int64), ("kv_bytes_per_position", C.c_int64)]


def load_library(path=None):
    """Load libminfer_b200.so and attach argument types.  Raises if it is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else LIB_PATH
    if not p.exists():
        raise FileNotFoundError(f"{p} not built: run `python nano-inference_b200/build.py` (needs nvcc); there is no fallback path")
    lib = C.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library does not export a declared symbol
        fn.restype, fn.argtypes = res, args
    if path is None:
        _lib = lib
    return lib


def detok_piece(piece):
    """Text bytes of one vocabulary piece of a byte-level BPE tokenizer (bytes or str in, bytes out).  Host only."""
    raw = piece.encode("utf-8") if isinstance(piece, str) else bytes(piece)
    buf = C.create_string_buffer(max(len(raw), 1))
    n = load_library().mi_detok_piece(raw, len(raw), buf, len(raw))
    if n < 0:
        raise ValueError("mi_detok_piece: bad argument")
    return buf.raw[:n]


def _ptr(t):
    """Device (or host) address of a torch tensor / numpy array / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    if hasattr(t, "ctypes"):
        return t.ctypes.data
    raise TypeError(f"cannot take the address of {type(t)}")


class Context:
    """One GPU: wraps mi_ctx."""

    def __init__(self, device=0):
        self.lib = load_library()
        h = _vp()
        st = self.lib.mi_ctx_create(device, C.byref(h))
        if st != MI_OK:
            raise MinferError(st, "mi_ctx_create", "(no usable sm_100 CUDA device?)")
        self.h = h
        self.device = device

    def check(self, st, where):
        if st != MI_OK:
            raise MinferError(st, where, self.lib.mi_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            self.lib.mi_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def sm_count(self):
        return self.lib.mi_ctx_sm_count(self.h)

    def set_stream(self, cuda_stream_ptr):
        self.check(self.lib.mi_ctx_set_stream(self.h, cuda_stream_ptr), "mi_ctx_set_stream")

    def use_torch_stream(self):
        import torch
        h = torch.cuda.current_stream().cuda_stream
        self.set_stream(h if h else 1)          # handle 0 is the legacy default stream: pass its alias

    def sync(self):
        self.check(self.lib.mi_ctx_sync(self.h), "mi_ctx_sync")

    def probe_read_bw(self, nbytes, variant=0, repeats=3):
        """Read-only streaming GB/s over a freshly allocated buffer of nbytes (variant 0: 16-byte loads, 1: bulk-copy ring)."""
        v = C.c_float()
        self.check(self.lib.mi_probe_read_bw(self.h, int(nbytes), variant, repeats, C.byref(v)), "mi_probe_read_bw")
        return v.value

    def probe_hop_ns(self, iters=2000):
        """One-way store-to-load latency between two SMs, nanoseconds."""
        v = C.c_float()
        self.check(self.lib.mi_probe_hop_ns(self.h, iters, C.byref(v)), "mi_probe_hop_ns")
        return v.value

    def set_wait_budget_ns(self, ns):
        """Time budget of the decode kernel's device-side waits (default 2 s)."""
        self.check(self.lib.mi_ctx_set_wait_budget_ns(self.h, int(ns)), "mi_ctx_set_wait_budget_ns")

    # ---- weights
    def upload_q4_0(self, raw_host, rows, cols, count=1):
        """raw_host: numpy uint8 array of count*rows*(cols/32)*18 bytes in GGUF block order."""
        h = _vp()
        self.check(self.lib.mi_weight_upload_q4_0(self.h, _ptr(raw_host), rows, cols, count, C.byref(h)), "mi_weight_upload_q4_0")
        return Weight(self, h)

    def repack_q4_0_dev(self, raw_dev, rows, cols, count=1):
        h = _vp()
        self.check(self.lib.mi_weight_repack_q4_0_dev(self.h, _ptr(raw_dev), rows, cols, count, C.byref(h)), "mi_weight_repack_q4_0_dev")
        return Weight(self, h)

    def requant_q4_0(self, ggml_type, src_dev, rows, cols, dst_dev):
        """Q4_1 (3), Q8_0 (8) or Q6_K (14) blocks on the device -> row-major q4_0 blocks on the device (uint8 tensors)."""
        self.check(self.lib.mi_requant_q4_0(self.h, ggml_type, _ptr(src_dev), rows, cols, _ptr(dst_dev)), "mi_requant_q4_0")

    # ---- kernels (device pointers: torch CUDA tensors)
    def quant_q8(self, x, xq, xd, n=None, M=1):
        n = x.shape[-1] if n is None else n
        self.check(self.lib.mi_quant_q8(self.h, _ptr(x), n, M, _ptr(xq), _ptr(xd)), "mi_quant_q8")

    def gemv_q4_q8(self, w, xq, xd, y, bias=None, ksplit=0, variant=0):
        self.check(self.lib.mi_gemv_q4_q8_ex(self.h, w.h, _ptr(xq), _ptr(xd), _ptr(bias), _ptr(y), ksplit, variant), "mi_gemv_q4_q8")

    def gemv_q4_q8_noalloc(self, w, xq, xd, y, bias=None):
        """The GEMV through the entry point that never allocates (fixed built-in scratch)."""
        self.check(self.lib.mi_gemv_q4_q8_noalloc(self.h, w.h, _ptr(xq), _ptr(xd), _ptr(bias), _ptr(y)), "mi_gemv_q4_q8_noalloc")

    def gemm_q4_q8(self, w, xq, xd, M, y, bias=None):
        """M token vectors per weight pass on the tensor cores; y is [M][rows]."""
        self.check(self.lib.mi_gemm_q4_q8(self.h, w.h, _ptr(xq), _ptr(xd), M, _ptr(bias), _ptr(y)), "mi_gemm_q4_q8")

    def attn_splitkv(self, q, kcache, vcache, n_head, n_head_kv, head_dim, pos0, M, out):
        """Causal GQA attention of M consecutive queries over an fp16 cache [positions][n_head_kv*head_dim]."""
        self.check(self.lib.mi_attn_splitkv(self.h, _ptr(q), _ptr(kcache), _ptr(vcache), n_head, n_head_kv, head_dim, pos0, M, _ptr(out)),
                   "mi_attn_splitkv")

    def block_isums(self, w, xq, isum):
        self.check(self.lib.mi_block_isums_q4_q8(self.h, w.h, _ptr(xq), _ptr(isum)), "mi_block_isums_q4_q8")

    def gemv_q4_f32_host(self, w, x_host, y_host, bias=None):
        self.check(self.lib.mi_gemv_q4_f32_host(self.h, w.h, _ptr(x_host), _ptr(bias), _ptr(y_host)), "mi_gemv_q4_f32_host")


class Weight:
    """A q4_0 matrix stack in the tiled device layout: wraps mi_weight."""

    def __init__(self, ctx, h):
        self.ctx, self.h = ctx, h
        r, c, n, b = _i64(), _i64(), _i64(), _i64()
        ctx.lib.mi_weight_info(h, C.byref(r), C.byref(c), C.byref(n), C.byref(b))
        self.rows, self.cols, self.count, self.device_bytes = r.value, c.value, n.value, b.value

    def download(self, out_host):
        self.ctx.check(self.ctx.lib.mi_weight_download_q4_0(self.ctx.h, self.h, _ptr(out_host)), "mi_weight_download_q4_0")

    def free(self):
        if self.h and self.ctx.h:
            self.ctx.lib.mi_weight_free(self.ctx.h, self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Batch:
    """KV slabs for sequences decoded together, one step per call: wraps mi_batch."""

    def __init__(self, model, n_slots, max_seq):
        self.ctx, self.model = model.ctx, model
        h = _vp()
        self.ctx.check(self.ctx.lib.mi_batch_create(self.ctx.h, model.h, n_slots, max_seq, C.byref(h)), "mi_batch_create")
        self.h = h

    def step(self, tokens, slots, positions, logits=None):
        """One decode step of len(tokens) sequences; returns (next greedy token of each, device milliseconds)."""
        import numpy as np
        t = np.ascontiguousarray(tokens, dtype=np.int32); s = np.ascontiguousarray(slots, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        out = np.empty(t.size, dtype=np.int32)
        ms = C.c_float(0)
        self.ctx.check(self.ctx.lib.mi_batch_step(self.ctx.h, self.h, t.size, _ptr(t), _ptr(s), _ptr(p), _ptr(out), _ptr(logits), C.byref(ms)), "mi_batch_step")
        return out.tolist(), ms.value

    def free(self):
        if self.h and self.ctx.h:
            self.ctx.lib.mi_batch_free(self.ctx.h, self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class TokenRing:
    """Host-mapped ring a running generation publishes its tokens into: wraps mi_token_ring."""

    def __init__(self, ctx, capacity):
        self.ctx = ctx
        h = _vp()
        ctx.check(ctx.lib.mi_ring_create(ctx.h, capacity, C.byref(h)), "mi_ring_create")
        self.h = h

    def peek(self):
        """(count, tokens, margins, ns) of the entries valid right now, as lists."""
        n, t, g, s = _i32(), _vp(), _vp(), _vp()
        self.ctx.check(self.ctx.lib.mi_ring_peek(self.h, C.byref(n), C.byref(t), C.byref(g), C.byref(s)), "mi_ring_peek")
        k = n.value
        toks = list((C.c_int32 * k).from_address(t.value)) if k else []
        mar = list((C.c_float * k).from_address(g.value)) if k else []
        ns = list((C.c_uint64 * k).from_address(s.value)) if k else []
        return k, toks, mar, ns

    def reset(self):
        self.ctx.check(self.ctx.lib.mi_ring_reset(self.ctx.h, self.h), "mi_ring_reset")

    def free(self):
        if self.h and self.ctx.h:
            self.ctx.lib.mi_ring_destroy(self.ctx.h, self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Model:
    """A loaded GGUF model with its KV cache and decode state: wraps mi_model."""

    def __init__(self, ctx, path, max_seq, tp_rank=0, tp_world=1):
        self.ctx = ctx
        self.tp_rank, self.tp_world = tp_rank, tp_world
        h = _vp()
        ctx.check(ctx.lib.mi_model_load_gguf_tp(ctx.h, str(path).encode(), max_seq, tp_rank, tp_world, C.byref(h)), "mi_model_load_gguf_tp")
        self.h = h
        self.config = ModelConfig()
        ctx.check(ctx.lib.mi_model_info(h, C.byref(self.config)), "mi_model_info")

    def decode(self, in_tokens, n_steps, pos0=0, logits=None, mode=DECODE_PERSISTENT):
        """Returns (greedy tokens after each step, device milliseconds)."""
        import numpy as np
        toks = np.ascontiguousarray(in_tokens, dtype=np.int32)
        out = np.empty(max(n_steps, 1), dtype=np.int32)
        ms = C.c_float(0)
        self.ctx.check(self.ctx.lib.mi_decode(self.ctx.h, self.h, _ptr(toks) if toks.size else None, toks.size, n_steps, pos0,
                                              _ptr(out), _ptr(logits), mode, C.byref(ms)), "mi_decode")
        return out[:n_steps].tolist(), ms.value

    def set_stop_token(self, token):
        """End runs of whole steps after the step that picks `token` as the next input (-1: never)."""
        self.ctx.check(self.ctx.lib.mi_model_set_stop_token(self.h, token), "mi_model_set_stop_token")

    def last_count(self):
        """Tokens the last decode / generate_spec call produced (fewer than asked after a stop)."""
        return int(self.ctx.lib.mi_model_last_count(self.h))

    def margins(self, n):
        """Top-1 minus top-2 logit of the first n steps of the last decode call (numpy float32)."""
        import numpy as np
        out = np.empty(max(n, 1), dtype=np.float32)
        self.ctx.check(self.ctx.lib.mi_decode_margins(self.ctx.h, self.h, n, _ptr(out)), "mi_decode_margins")
        return out[:n]

    def decode_run(self, in_tokens, n_steps, pos0, ring):
        """Asynchronous persistent decode whose tokens arrive in `ring` (a TokenRing) while the kernel runs."""
        import numpy as np
        toks = np.ascontiguousarray(in_tokens, dtype=np.int32)
        self.ctx.check(self.ctx.lib.mi_decode_run(self.ctx.h, self.h, _ptr(toks) if toks.size else None, toks.size, n_steps, pos0, ring.h), "mi_decode_run")

    def verify(self, tokens, pos0=0, logits=None):
        """One M-token pass (M = len(tokens) <= 16): returns (greedy token after each, device milliseconds)."""
        import numpy as np
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty(toks.size, dtype=np.int32)
        ms = C.c_float(0)
        self.ctx.check(self.ctx.lib.mi_verify(self.ctx.h, self.h, _ptr(toks), toks.size, pos0, _ptr(out), _ptr(logits), C.byref(ms)), "mi_verify")
        return out.tolist(), ms.value

    def generate_spec(self, prompt, n_gen, ngmax=3, draftk=4):
        """Greedy generation with lossless n-gram speculation; returns (ids, stats dict)."""
        import numpy as np
        toks = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(max(n_gen, 1), dtype=np.int32)
        st = np.zeros(4, dtype=np.int64)
        mg = np.zeros(max(n_gen, 1), dtype=np.float32)
        self.ctx.check(self.ctx.lib.mi_generate_spec(self.ctx.h, self.h, _ptr(toks), toks.size, n_gen, ngmax, draftk, _ptr(out), _ptr(mg), _ptr(st)), "mi_generate_spec")
        return out[:n_gen].tolist(), {"steps": int(st[0]), "drafted": int(st[1]), "accepted": int(st[2]), "spec_steps": int(st[3]),
                                      "margins": mg[:n_gen]}

    def prefill(self, tokens, pos0=0, chunk=16):
        """Prompt processing through the M-token step, `chunk` tokens per weight pass; returns (token after the last one, ms)."""
        total, last = 0.0, None
        for i in range(0, len(tokens), chunk):
            out, ms = self.verify(tokens[i:i + chunk], pos0 + i)
            total += ms
            last = out[-1]
        return last, total

    def generate(self, prompt, n_gen, mode=DECODE_PERSISTENT):
        """The reference CLI's output: n_gen greedy ids, the first predicted after the last prompt token."""
        out, ms = self.decode(prompt, len(prompt) + n_gen - 1, 0, None, mode)
        return out[len(prompt) - 1:], ms

    # ---- tensor parallelism: asynchronous launches + the exchanged buffers as torch tensors
    def tp_region(self, which, layer=0):
        """uint8 torch tensor aliasing one exchanged buffer (no copy)."""
        p, n = _vp(), _i64()
        self.ctx.check(self.ctx.lib.mi_model_tp_region(self.h, which, layer, C.byref(p), C.byref(n)), "mi_model_tp_region")
        return _as_cuda_tensor(p.value, n.value)

    def launch(self, pos, ph0, ph1):
        self.ctx.check(self.ctx.lib.mi_decode_launch(self.ctx.h, self.h, pos, ph0, ph1), "mi_decode_launch")

    def tp_ipc_handles(self):
        """192 bytes: CUDA IPC handles of this rank's exchanged buffers (numpy uint8)."""
        import numpy as np
        out = np.zeros(192, dtype=np.uint8)
        self.ctx.check(self.ctx.lib.mi_tp_ipc_handles(self.ctx.h, self.h, _ptr(out)), "mi_tp_ipc_handles")
        return out

    def tp_ipc_open(self, all_handles):
        """all_handles: numpy uint8 [world * 192], every rank's handles in rank order."""
        self.ctx.check(self.ctx.lib.mi_tp_ipc_open(self.ctx.h, self.h, _ptr(all_handles)), "mi_tp_ipc_open")

    def tp_exchange(self, which, layer=0):
        self.ctx.check(self.ctx.lib.mi_tp_exchange(self.ctx.h, self.h, which, layer), "mi_tp_exchange")

    def launch_fused(self, pos, ph0, ph1):
        self.ctx.check(self.ctx.lib.mi_decode_launch_fused(self.ctx.h, self.h, pos, ph0, ph1), "mi_decode_launch_fused")

    def set_pos(self, pos):
        self.ctx.check(self.ctx.lib.mi_model_set_pos(self.ctx.h, self.h, int(pos)), "mi_model_set_pos")

    def advance_pos(self, delta=1):
        self.ctx.check(self.ctx.lib.mi_model_advance_pos(self.ctx.h, self.h, int(delta)), "mi_model_advance_pos")

    def set_token(self, tok):
        self.ctx.check(self.ctx.lib.mi_model_set_token(self.ctx.h, self.h, int(tok)), "mi_model_set_token")

    def get_token(self):
        t, v = C.c_int32(), C.c_float()
        self.ctx.check(self.ctx.lib.mi_model_get_token(self.ctx.h, self.h, C.byref(t), C.byref(v)), "mi_model_get_token")
        return t.value, v.value

    def tp_pick(self, gathered, world):
        self.ctx.check(self.ctx.lib.mi_tp_pick(self.ctx.h, self.h, _ptr(gathered), world), "mi_tp_pick")

    def debug_drop_phase(self, phase):
        """Test hook: the producers of `phase` publish nothing (its consumers' waits then run out); -1 = normal."""
        self.ctx.check(self.ctx.lib.mi_model_debug_drop_phase(self.h, int(phase)), "mi_model_debug_drop_phase")

    def run_phases(self, token, pos, ph0, ph1):
        self.ctx.check(self.ctx.lib.mi_decode_phases(self.ctx.h, self.h, token, pos, ph0, ph1), "mi_decode_phases")

    def state_tensor(self, name):
        """uint8 torch tensor aliasing a whole state buffer (no copy), e.g. to fill the KV cache for a benchmark."""
        p, n = _vp(), _i64()
        self.ctx.check(self.ctx.lib.mi_model_state_ptr(self.h, STATE[name], C.byref(p), C.byref(n)), "mi_model_state_ptr")
        return _as_cuda_tensor(p.value, n.value)

    def state(self, name, dtype, count):
        """Copy of a state buffer as a numpy array."""
        import numpy as np
        p, n = _vp(), _i64()
        self.ctx.check(self.ctx.lib.mi_model_state_ptr(self.h, STATE[name], C.byref(p), C.byref(n)), "mi_model_state_ptr")
        self.ctx.sync()
        nbytes = min(n.value, count * np.dtype(dtype).itemsize)
        return _as_cuda_tensor(p.value, nbytes).cpu().numpy().view(dtype).copy()

    def free(self):
        if self.h and self.ctx.h:
            self.ctx.lib.mi_model_free(self.ctx.h, self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _as_cuda_tensor(ptr, nbytes):
    """A torch uint8 CUDA tensor aliasing raw device memory (no copy)."""
    import torch

    class _Holder:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}
    return torch.as_tensor(_Holder(), device="cuda")
