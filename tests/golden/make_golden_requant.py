"""Generates requant_ref.npz from the REFERENCE itself: the block formats other than q4_0 that real model files carry.

Run where the reference checkout is present and oracle/_ref has been built (`make -C oracle ref`; the q4_0 re-quantizer
needs nvcc because it lives in the reference's src/mega.cu):

    python tests/golden/make_golden_requant.py

For Q4_1, Q8_0 and Q6_K it stores seeded well-formed raw blocks, the rows the reference's GGUF::dequant_row
(src/gguf.h:103-140) makes of them, and the q4_0 bytes the reference's quant_row_q4_0 (src/mega.cu:924-936) makes of those
rows.  The CPU tests pin the oracle's restatement to these; the GPU test compares the library's load-time re-quantizer with
the oracle.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import oracle_util as ou    # noqa: E402


def main():
    mega_so = ou.ROOT / "oracle" / "_ref" / "libref_mega.so"
    if not ou.have_ref() or not mega_so.exists():
        raise SystemExit("oracle/_ref is not complete: run `make -C oracle ref` where the reference and nvcc are present")
    R = ou.ref()
    M = C.CDLL(str(mega_so))
    M.ref_quant_row_q4_0.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    rng = np.random.default_rng(20240611)
    fx = {}
    rows, cols = 5, 768
    for fmt, (tid, bpb, epb) in ou.BLOCK_FORMATS.items():
        raw = ou.random_blocks(fmt, rows, cols, rng)
        deq = np.empty((rows, cols), np.float32)
        q4 = np.empty((rows, cols // 32 * 18), np.uint8)
        for r in range(rows):
            R.ref_dequant_row(tid, raw.ctypes.data, rows, cols, r, deq[r].ctypes.data)
            M.ref_quant_row_q4_0(deq[r].ctypes.data, cols, q4[r].ctypes.data)
        fx[f"{fmt}_raw"], fx[f"{fmt}_deq"], fx[f"{fmt}_q4"] = raw, deq.view(np.uint32), q4
    # edge rows for the re-quantizer alone: zeros, one spike, values at the rounding ties of lrintf
    edge = np.zeros((3, 64), np.float32)
    edge[1, 5] = -3.5
    edge[2] = np.linspace(-7.0, 7.0, 64, dtype=np.float32) * 0.5
    q4e = np.empty((3, 36), np.uint8)
    for r in range(3):
        M.ref_quant_row_q4_0(edge[r].ctypes.data, 64, q4e[r].ctypes.data)
    fx["edge_y"], fx["edge_q4"] = edge, q4e
    fx["shape"] = np.array([rows, cols])
    np.savez_compressed(HERE / "requant_ref.npz", **fx)
    print("wrote", HERE / "requant_ref.npz")


if __name__ == "__main__":
    main()
