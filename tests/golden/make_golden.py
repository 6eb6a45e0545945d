"""Generates the golden fixtures in this directory from the REFERENCE itself.

Run where the reference checkout is present and oracle/_ref has been built
(`make -C oracle ref`):

    python tests/golden/make_golden.py

It calls the reference's own functions (matvec, rmsnorm, rope, dequant_row from
src/cpu_infer.cpp / src/gguf.h, through oracle/_ref/libref_ops.so) and the
unmodified cpu_infer program on seeded inputs, and stores inputs + outputs:

    ops_ref.npz        q4_0 matrix bytes, x, reference matvec / dequant / rmsnorm / rope results
    streams_ref.json   gguf_synth arguments, prompts and the greedy ids cpu_infer printed

The fixtures are small (a few tens of KB) and are what the CPU test-suite and
the GPU parity tests compare against where the reference cannot travel.
"""
import json
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import gguf_util as gu      # noqa: E402
import oracle_util as ou    # noqa: E402


def main():
    if not ou.have_ref():
        raise SystemExit("oracle/_ref is not built: run `make -C oracle ref` where the reference is present")
    R = ou.ref()
    rng = np.random.default_rng(20240607)
    fx = {}
    # --- matvec on three shapes (last one has a row count that is not a multiple of 32)
    for tag, rows, cols in (("a", 96, 256), ("b", 64, 896), ("c", 50, 1536)):
        W = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
        raw = ou.quantize_q4_0(W)             # bytes are the input; how they were made does not matter
        x = rng.standard_normal(cols).astype(np.float32)
        y = np.empty(rows, np.float32)
        R.ref_matvec_q4_0(raw.ctypes.data, rows, cols, x.ctypes.data, y.ctypes.data)
        deq = np.empty((rows, cols), np.float32)
        for r in range(rows):
            R.ref_dequant_row_q4_0(raw.ctypes.data, rows, cols, r, deq[r].ctypes.data)
        fx[f"mv_{tag}_raw"], fx[f"mv_{tag}_x"], fx[f"mv_{tag}_y"] = raw, x, y
        fx[f"mv_{tag}_shape"] = np.array([rows, cols])
        fx[f"mv_{tag}_deq_row0"] = deq[0].copy()
        fx[f"mv_{tag}_deq_rowlast"] = deq[-1].copy()
    # --- rmsnorm, rope
    x = rng.standard_normal(896).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(896)).astype(np.float32)
    out = np.empty_like(x)
    R.ref_rmsnorm(x.ctypes.data, w.ctypes.data, 896, 1e-6, out.ctypes.data)
    fx["rms_x"], fx["rms_w"], fx["rms_out"] = x, w, out
    v = rng.standard_normal(4 * 64).astype(np.float32)
    for pos in (0, 1, 77, 4095):
        vv = v.copy()
        R.ref_rope(vv.ctypes.data, 4, 64, pos, 1e6)
        fx[f"rope_out_{pos}"] = vv
    fx["rope_in"] = v
    # --- fp16 table: every half value through the reference's converter
    allh = np.arange(65536, dtype=np.uint16)
    fx["fp16_all"] = np.array([R.ref_fp16_to_fp32(int(h)) for h in allh], dtype=np.float32).view(np.uint32)
    np.savez_compressed(HERE / "ops_ref.npz", **fx)

    # --- greedy streams of the unmodified cpu_infer on synthetic models
    streams = []
    with tempfile.TemporaryDirectory() as td:
        for preset, seed, std, prompt, n_gen in (
            ("tiny", 5, 0.02, [1, 2, 3, 4, 5, 6, 7], 16),
            ("tiny", 5, 0.1, [1, 2, 3, 4, 5, 6, 7], 16),
            ("tiny", 11, 0.3, [500, 3, 77, 12, 12, 401], 24),
        ):
            p = gu.make_synthetic(Path(td) / "m.gguf", preset, seed=seed, std=std, extra=["--bias-std", std])
            ids, _ = ou.run_ref_cpu_infer(p, n_gen, prompt)
            streams.append(dict(preset=preset, seed=seed, std=std, bias_std=std, prompt=prompt, n_gen=n_gen, ref_ids=ids))
    (HERE / "streams_ref.json").write_text(json.dumps(streams, indent=1))
    print("wrote", HERE / "ops_ref.npz", HERE / "streams_ref.json")


if __name__ == "__main__":
    main()
