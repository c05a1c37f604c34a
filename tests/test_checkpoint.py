"""Checkpoint reader / writer (ane_cuda_ckpt_*) against files laid out the way the reference's save_checkpoint writes
them (training/train_large.m:109-145, training/training_dynamic/train.m:104-138)."""
import os

import numpy as np
import pytest

from ane_b200 import checkpoint as ck
from ane_b200 import lib
from oracle import ckpt_format as fmt

CASES = {
    "v4_gqa": dict(version=4, n_layers=3, vocab_size=50, dim=16, hidden_dim=40, n_heads=4, seq_len=32, kv_heads=2, head_dim=8, q_dim=32),
    "v2_square": dict(version=2, n_layers=2, vocab_size=33, dim=12, hidden_dim=20, n_heads=3, seq_len=16),
}


def _make(tmp_path, name):
    c = dict(CASES[name], step=7, total_steps=100, lr=3e-4, loss=2.5, cum_compile=1.5, cum_train=12.25, cum_wall=20.0, cum_steps=7,
             cum_batches=3, adam_t=7)
    rng = np.random.default_rng(len(name))
    sz = fmt.sizes(c["version"], c["n_layers"], c["vocab_size"], c["dim"], c["hidden_dim"], c["n_heads"], c.get("kv_heads", 0),
                   c.get("head_dim", 0), c.get("q_dim", 0))
    trip = lambda n: tuple(rng.standard_normal(n).astype(np.float32) for _ in range(3))
    layers = [[trip(n) for n in sz] for _ in range(c["n_layers"])]
    rms_final, embed = trip(c["dim"]), trip(c["vocab_size"] * c["dim"])
    path = str(tmp_path / f"{name}.bin")
    fmt.write(path, c, layers, rms_final, embed)
    return path, c, layers, rms_final, embed


@pytest.mark.parametrize("name", list(CASES))
def test_header_is_read_without_a_gpu(tmp_path, name):
    path, c, layers, rms_final, embed = _make(tmp_path, name)
    h = ck.read_header(path)
    assert C_sizeof(h) == 96
    for k in ("version", "step", "total_steps", "n_layers", "vocab_size", "dim", "hidden_dim", "n_heads", "seq_len", "cum_steps", "adam_t"):
        assert getattr(h, k) == c[k], k
    assert abs(h.lr - c["lr"]) < 1e-9 and h.cum_train == c["cum_train"] and h.cum_wall == c["cum_wall"]
    n = ck.param_count(h)
    assert n == fmt.weight_order(layers, rms_final, embed, 0).size
    assert os.path.getsize(path) == 96 + 3 * 4 * n
    assert [s for _, s in ck.layer_tensors(h)] == fmt.sizes(c["version"], c["n_layers"], c["vocab_size"], c["dim"], c["hidden_dim"],
                                                            c["n_heads"], c.get("kv_heads", 0), c.get("head_dim", 0), c.get("q_dim", 0))


def C_sizeof(obj):
    import ctypes
    return ctypes.sizeof(obj)


def test_bad_files_are_refused(tmp_path):
    p = tmp_path / "short.bin"
    p.write_bytes(b"\x00" * 10)
    with pytest.raises(lib.AneCudaError):
        ck.read_header(str(p))
    p = tmp_path / "magic.bin"
    p.write_bytes(b"\x01" * 96)
    with pytest.raises(lib.AneCudaError):
        ck.read_header(str(p))
    with pytest.raises(lib.AneCudaError):
        ck.read_header(str(tmp_path / "missing.bin"))


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_load_and_save_round_trip(tmp_path, name):
    import torch
    assert torch.cuda.is_available(), "needs a CUDA device"
    lib.init(0)
    path, c, layers, rms_final, embed = _make(tmp_path, name)
    h, w, m, v = ck.load(path)
    for which, t in enumerate((w, m, v)):
        assert np.array_equal(t.cpu().numpy(), fmt.weight_order(layers, rms_final, embed, which))       # bit-exact
    h2, w_only, m2, v2 = ck.load(path, with_moments=False)
    assert m2 is None and torch.equal(w_only, w)
    out = str(tmp_path / "again.bin")
    ck.save(out, h, w, m, v)
    assert open(out, "rb").read() == open(path, "rb").read()                                          # byte-identical file
    # a buffer of the wrong size is refused before anything is copied
    with pytest.raises(lib.AneCudaError):
        lib.check(lib.load().ane_cuda_ckpt_save(out.encode(), __import__("ctypes").byref(h), w.data_ptr(), m.data_ptr(), v.data_ptr(), w.numel() - 1))
