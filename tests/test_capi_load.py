"""The C-ABI library builds, loads without a GPU and exports every symbol include/vexel_cuda.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vexel_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib_built):
    dll = ctypes.CDLL(lib_built)
    names = declared_symbols()
    assert len(names) > 60
    missing = [n for n in names if not hasattr(dll, n)]
    assert not missing, missing


def test_binding_covers_the_header(lib_built):
    from vexel_b200 import capi
    assert set(capi.SIGNATURES) == set(declared_symbols())
    capi.Lib.get()


def test_no_cpu_fallback(lib_built):
    """Without a CUDA device vx_init must fail; with one it must succeed."""
    dll = ctypes.CDLL(lib_built)
    h = ctypes.c_void_p()
    rc = dll.vx_init(0, ctypes.byref(h))
    import torch
    if torch.cuda.is_available():
        assert rc == 0
        dll.vx_destroy(h)
    else:
        assert rc == 2 and not h.value


def test_product_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "vexel_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle|vexel_oracle|libvexel_oracle", src, flags=re.M), f"{f} uses the oracle"
