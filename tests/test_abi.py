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


def test_host_mirrors_refuse_arrays_that_do_not_match_their_size_arguments():
    """The reference's functions trust the caller with the sizes; the Python mirrors check every array against them before
    anything reaches C (no GPU needed: the check comes first)."""
    import numpy as np
    import pytest
    import torch
    from ane_b200 import cpu_ops, host_ops
    x, w = np.zeros((8, 4), np.float32), np.ones(8, np.float32)
    with pytest.raises(ValueError, match="out"):
        cpu_ops.rmsnorm(np.zeros((8, 3), np.float32), x, w, 8, 4)
    with pytest.raises(ValueError, match="w"):
        cpu_ops.rmsnorm(np.zeros_like(x), x, np.ones(7, np.float32), 8, 4)
    with pytest.raises(TypeError):
        cpu_ops.rmsnorm(np.zeros_like(x), x.astype(np.float64), w, 8, 4)
    with pytest.raises(TypeError):
        cpu_ops.rmsnorm(np.zeros_like(x), x.T, w, 4, 8)                       # not C-contiguous
    with pytest.raises(ValueError):
        cpu_ops.rmsnorm(np.zeros_like(x), x, w, 8, 0)
    with pytest.raises(ValueError, match="targets"):
        cpu_ops.cross_entropy_loss(np.zeros((5, 4), np.float32), np.zeros((5, 4), np.float32), np.zeros(3, np.uint16), 5, 4)
    with pytest.raises(ValueError, match="head width"):
        cpu_ops.rope_backward_inplace(np.zeros((12, 4), np.float32), 4, 12, 5)
    st = cpu_ops.AdamState(8)
    with pytest.raises(ValueError, match="g"):
        cpu_ops.adam_update(np.zeros(8, np.float32), np.zeros(9, np.float32), st, 1, 1e-3, 0.9, 0.999, 1e-8)
    with pytest.raises(ValueError, match="from 1"):
        cpu_ops.adam_update(np.zeros(8, np.float32), np.zeros(8, np.float32), st, 0, 1e-3, 0.9, 0.999, 1e-8)
    t = torch.zeros(2, 8, 4)
    with pytest.raises(ValueError, match="out"):
        host_ops.rmsnorm(torch.zeros(2, 8, 3), t, torch.ones(8))
    with pytest.raises(ValueError, match="w"):
        host_ops.rmsnorm(torch.zeros(2, 8, 4), t, torch.ones(9))
    with pytest.raises(ValueError, match="heads"):
        host_ops.qknorm_rope(torch.zeros(2, 8, 4), t, torch.ones(3), 3)
    with pytest.raises(ValueError, match="dy"):
        host_ops.rmsnorm_bwd(torch.zeros(2, 8, 4), torch.zeros(8), torch.zeros(2, 8, 4, dtype=torch.bfloat16), t, torch.ones(8))


def test_chain_and_library_memory_calls_refuse_to_run_before_init():
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        return
    L = lib.load()
    assert not L.ane_cuda_chain_create(None, 1, None)
    assert b"ane_cuda_init" in L.ane_cuda_last_error()
    assert L.ane_cuda_chain_step(None, None) == lib.ERR_NOT_INIT
    assert L.ane_cuda_chain_sync(None) == lib.ERR_NOT_INIT
    assert L.ane_cuda_chain_h2d_bytes(None) == 0 and L.ane_cuda_chain_d2h_bytes(None) == 0
    assert not L.ane_cuda_chain_compute_stream(None)
    L.ane_cuda_chain_destroy(None)                                   # a null chain is ignored
    for rc in (L.ane_cuda_reserve_workspace(1 << 20), L.ane_cuda_freeze(1), L.ane_cuda_release_caches(),
               L.ane_cuda_zero_dev(None, None, 16), L.ane_cuda_copy_dev(None, None, None, 16)):
        assert rc == lib.ERR_NOT_INIT
    sz = C.c_size_t()
    assert L.ane_cuda_ckpt_tensor_offset(None, 0, 0, 0, C.byref(sz), C.byref(sz)) == lib.ERR_INVALID
    assert L.ane_cuda_ckpt_flat_decay_count(None) == 0
