"""CPU: the C-ABI library loads and exports every symbol the header declares;
source hygiene checks that need no GPU."""
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "minfer_b200.h"
PKG = ROOT / "nano-inference_b200"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"MI_API\s+[\w\s\*]+?\b(mi_\w+)\s*\(", text)))


def test_header_declares_symbols():
    syms = declared_symbols()
    assert "mi_gemv_q4_q8" in syms and "mi_ctx_create" in syms and len(syms) >= 15


def test_library_exports_every_declared_symbol(pkg):
    if not pkg.LIB_PATH.exists():
        pytest.fail(f"{pkg.LIB_PATH} is not built: run `python nano-inference_b200/build.py`")
    lib = pkg.load_library()
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} is declared in the header but not exported"
        assert s in pkg.SIGNATURES, f"{s} has no ctypes signature in the binding"
    assert b"sm_100a" in lib.mi_version()


def test_status_strings(pkg):
    lib = pkg.load_library()
    assert lib.mi_strerror(0) == b"ok"
    assert b"wait" in lib.mi_strerror(4)
    assert lib.mi_strerror(12345) == b"unknown status"


def test_ctx_create_fails_loudly_without_gpu(pkg):
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert pkg.load_library().mi_ctx_create(0, C.byref(h)) != 0     # no fallback device
    with pytest.raises(pkg.MinferError):
        pkg.Context(0)


def test_no_cluster_multicast_loads_in_cuda_sources():
    """Every kernel here also runs in multi-GPU jobs: bulk/TMA loads must not use cluster multicast."""
    for f in list(PKG.rglob("*.cu")) + list(PKG.rglob("*.cuh")):
        assert "multicast" not in f.read_text(), f"{f} mentions multicast"


def test_product_does_not_touch_the_oracle():
    """The oracle is a checker: nothing under the package may include, link or load it."""
    for f in PKG.rglob("*"):
        if f.is_file() and f.suffix in (".cu", ".cuh", ".cpp", ".hpp", ".h", ".py"):
            t = f.read_text()
            assert "oracle" not in t.lower() or f.name == "__init__.py" and "oracle" not in t, f"{f} refers to the oracle"
