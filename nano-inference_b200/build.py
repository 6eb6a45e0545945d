"""Builds the native parts in-tree: the CUDA library for sm_100a and the host programs.

    python nano-inference_b200/build.py [--force]

Outputs (all git-ignored, next to the sources so that they travel with the tree):
    nano-inference_b200/lib/libminfer_b200.so     CUDA kernels + C ABI
    nano-inference_b200/bin/gguf_synth            synthetic model writer
    nano-inference_b200/bin/cuda_infer, mega      driver programs (same command line as the reference's)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
LIB = PKG / "lib" / "libminfer_b200.so"
BIN = PKG / "bin"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--shared",
]
GXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed ({r.returncode}): {' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")
    return r


def cuda_sources():
    return sorted(CSRC.glob("*.cu"))


def build_library(force=False, verbose=False, extra_flags=()):
    """Each .cu becomes an object under build/ (recompiled only when it or a header
    changed, several at a time), then one shared library is linked."""
    from concurrent.futures import ThreadPoolExecutor
    srcs = cuda_sources()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(HOST.glob("*.hpp")) + [ROOT / "include" / "minfer_b200.h"]
    objdir = PKG / "build"
    objdir.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "--shared"]
    jobs = []
    for s in srcs:
        o = objdir / (s.stem + ".o")
        if force or _newer(o, [s] + headers):
            jobs.append([_nvcc(), *flags, "-ccbin", GXX, *extra_flags, "-I", ROOT / "include", "-I", HOST, "-c", "-o", o, s])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    objs = [objdir / (s.stem + ".o") for s in srcs]
    if force or jobs or _newer(LIB, objs):
        _run([_nvcc(), "--shared", "-ccbin", GXX, "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs], verbose)
    return LIB


def build_host(force=False, verbose=False):
    BIN.mkdir(parents=True, exist_ok=True)
    out = []
    synth = BIN / "gguf_synth"
    if force or _newer(synth, [HOST / "gguf_synth.cpp"]):
        _run([GXX, "-O2", "-std=c++17", "-pthread", "-o", synth, HOST / "gguf_synth.cpp"], verbose)
    out.append(synth)
    for name in ("cuda_infer", "mega"):
        src = HOST / f"{name}.cpp"
        if not src.exists():
            continue
        exe = BIN / name
        if force or _newer(exe, [src, LIB, HOST / "driver_common.hpp", ROOT / "include" / "minfer_b200.h"]):
            _run([GXX, "-O2", "-std=c++17", "-I", ROOT / "include", "-I", HOST, "-o", exe, src,
                  "-L", LIB.parent, "-lminfer_b200", "-Wl,-rpath,$ORIGIN/../lib"], verbose)
        out.append(exe)
    return out


def build_all(force=False, verbose=False):
    lib = build_library(force, verbose)
    exes = build_host(force, verbose)
    return lib, exes


if __name__ == "__main__":
    lib, exes = build_all(force="--force" in sys.argv, verbose=True)
    print(lib)
    for e in exes:
        print(e)
