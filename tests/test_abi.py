"""CPU checks of the boundary: the shared object loads, exports every symbol that
include/ane_cuda.h declares, and refuses to work without a GPU instead of falling back."""
import os
import re

from ane_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ane_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ane_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = _declared()
    assert len(names) >= 45
    assert sorted(lib.PROTOTYPES) == names


def test_library_exports_every_declared_symbol():
    L = lib.load()
    for name in _declared():
        assert hasattr(L, name), name
    assert L.ane_cuda_version() == 100


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        return
    L = lib.load()
    assert L.ane_cuda_init(0) == lib.ERR_CUDA
    assert b"no CPU path" in L.ane_cuda_last_error()
    # operators refuse to run before a successful init
    assert L.ane_cuda_residual_dev(None, lib.F32, 4, 1, 1, 1, 1.0) == lib.ERR_NOT_INIT


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: nothing under ane_b200/ may reference it."""
    for dirpath, _, files in os.walk(os.path.join(ROOT, "ane_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in src, os.path.join(dirpath, f)
