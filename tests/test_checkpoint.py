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


# ------------------------------------------------------------------ optimizer order, truncated files, llama2.c files
def test_tensor_offsets_in_both_arrangements(tmp_path):
    """ane_cuda_ckpt_tensor_offset (no GPU): every tensor's range in weight order and in optimizer order equals its
    place in the numpy statements of the two arrangements."""
    path, c, layers, rms_final, embed = _make(tmp_path, "v4_gqa")
    h = ck.read_header(path)
    for flat, ref in ((False, fmt.weight_order(layers, rms_final, embed, 0)), (True, fmt.optimizer_order(layers, rms_final, embed, 0))):
        for L in range(c["n_layers"]):
            for i, name in enumerate(ck.TENSORS[:9]):
                off, cnt = ck.tensor_range(h, name, L, flat)
                assert np.array_equal(ref[off:off + cnt], layers[L][i][0])
        off, cnt = ck.tensor_range(h, "rms_final", 0, flat)
        assert np.array_equal(ref[off:off + cnt], rms_final[0])
        off, cnt = ck.tensor_range(h, "embed", 0, flat)
        assert np.array_equal(ref[off:off + cnt], embed[0])
    n_matrix = sum(t[0].size for tensors in layers for t in tensors[:7])
    assert ck.flat_decay_count(h) == n_matrix + embed[0].size
    with pytest.raises(lib.AneCudaError):
        ck.tensor_range(h, "Wq", c["n_layers"], True)


def _llama2c(tmp_path, n_heads=4, n_kv_heads=4, shared=True, cut=0):
    dim, hidden, n_layers, vocab, seq = 16, 40, 3, 50, 32
    kv = dim * n_kv_heads // n_heads
    rng = np.random.default_rng(n_kv_heads)
    sz = [dim * dim, kv * dim, kv * dim, dim * dim, hidden * dim, dim * hidden, hidden * dim, dim, dim]
    layers = [[rng.standard_normal(n).astype(np.float32) for n in sz] for _ in range(n_layers)]
    rms_final, embed = rng.standard_normal(dim).astype(np.float32), rng.standard_normal(vocab * dim).astype(np.float32)
    path = str(tmp_path / f"model_{n_kv_heads}_{int(shared)}_{cut}.bin")
    fmt.write_llama2c(path, dim, hidden, n_layers, n_heads, n_kv_heads, vocab, seq, layers, rms_final, embed, shared,
                      trailing=b"\x07" * 300)
    if cut:
        data = open(path, "rb").read()
        open(path, "wb").write(data[:len(data) - 300 - cut])
    trip = lambda a: (a, a, a)
    return path, [[trip(t) for t in tensors] for tensors in layers], trip(rms_final), trip(embed)


def test_llama2c_config_is_read_without_a_gpu(tmp_path):
    path, *_ = _llama2c(tmp_path, shared=False)
    c = ck.llama2c_read_config(path)
    assert (c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.vocab_size, c.seq_len) == (16, 40, 3, 4, 4, -50, 32)
    import ctypes
    h = ck.CkptHeader()
    lib.check(lib.load().ane_cuda_llama2c_to_header(ctypes.byref(c), ctypes.byref(h)))
    assert (h.version, h.vocab_size, h.dim, h.n_layers) == (2, 50, 16, 3)          # |vocab_size|, train_large.m:25
    p = tmp_path / "short_model.bin"
    p.write_bytes(b"\x01" * 20)
    with pytest.raises(lib.AneCudaError):
        ck.llama2c_read_config(str(p))


@pytest.mark.gpu
@pytest.mark.parametrize("n_kv_heads,shared", [(4, True), (4, False), (2, True)])
def test_llama2c_weights_load_into_both_arrangements(tmp_path, n_kv_heads, shared):
    """The file order of training/train_large.m:28-50 lands tensor by tensor where the checkpoint writer and the flat
    optimizer expect it; saving the result gives a reference checkpoint whose weights read back the same."""
    import torch
    lib.init(0)
    path, layers, rms_final, embed = _llama2c(tmp_path, n_kv_heads=n_kv_heads, shared=shared)
    h, w = ck.llama2c_load(path)
    assert h.version == (2 if n_kv_heads == 4 else 4)
    assert np.array_equal(w.cpu().numpy(), fmt.weight_order(layers, rms_final, embed, 0))
    h2, wf = ck.llama2c_load(path, flat=True, out=torch.full((w.numel() + 24,), 7.0, device="cuda"))
    assert np.array_equal(wf[:w.numel()].cpu().numpy(), fmt.optimizer_order(layers, rms_final, embed, 0))
    assert bool((wf[w.numel():] == 7.0).all())                                           # extras untouched
    out = str(tmp_path / "from_llama2c.ckpt")
    z = torch.zeros_like(w)
    ck.save(out, h, w, z, z)
    h3, w3, m3, _ = ck.load(out)
    assert torch.equal(w3, w) and not bool(m3.any()) and h3.version == h.version
    # config mismatch and truncated files are refused (train_large.m:20-23)
    bad = ck.Llama2cConfig(dim=16, hidden_dim=41, n_layers=3)
    with pytest.raises(lib.AneCudaError, match="mismatch"):
        ck.llama2c_load(path, expect=bad)
    short, *_ = _llama2c(tmp_path, n_kv_heads=n_kv_heads, shared=shared, cut=8)
    with pytest.raises(lib.AneCudaError, match="truncated"):
        ck.llama2c_load(short)


@pytest.mark.gpu
def test_truncated_checkpoint_body_is_refused(tmp_path):
    import torch
    lib.init(0)
    path, c, layers, rms_final, embed = _make(tmp_path, "v4_gqa")
    data = open(path, "rb").read()
    for keep in (96 + 40, len(data) // 2, len(data) - 4):
        cut = str(tmp_path / f"cut_{keep}.bin")
        open(cut, "wb").write(data[:keep])
        with pytest.raises(lib.AneCudaError, match="truncated"):
            ck.load(cut)
        with pytest.raises(lib.AneCudaError, match="truncated"):
            ck.load_flat(cut, torch.empty(len(data) // 12, device="cuda"))


@pytest.mark.gpu
def test_checkpoint_to_flat_params_adam_step_and_back(tmp_path, oracle):
    """A version-4 file loaded in optimizer order into layer_chain.FlatParams, one optimizer step through ShardedAdam
    (weight decay on matrices and embedding, none on the norm weights, train.m:837-869), saved again: every tensor of the
    new file equals the oracle's per-tensor adam_update of the old one, and the QK-norm weights that the file does not
    hold survive the load untouched."""
    import torch
    from ane_b200.layer_chain import ChainConfig, FlatParams
    from ane_b200.sharded import ShardedAdam
    lib.init(0)
    path, c, layers, rms_final, embed = _make(tmp_path, "v4_gqa")
    cfg = ChainConfig(layers=c["n_layers"], dim=c["dim"], hidden=c["hidden_dim"], heads=c["n_heads"], kv_heads=c["kv_heads"],
                      head_dim=c["head_dim"], seq=c["seq_len"], vocab=c["vocab_size"], dtype=torch.float32)
    p = FlatParams(cfg, "cuda")
    p.init_random(seed=1)
    qk_before = p.w[p.off_wq:p.n].clone()
    p.v.fill_(0.5)
    h = ck.load_flat(path, p.w, p.m, p.v)
    p.v.abs_()                                                       # the synthetic moments are signed; v must not be
    assert ck.param_count(h) == p.off_wq and ck.flat_decay_count(h) == p.n_decay
    assert torch.equal(p.w[p.off_wq:p.n], qk_before)
    assert torch.equal(p.norm_w("ffn", 1), torch.from_numpy(layers[1][8][0]).cuda())
    assert torch.equal(p.embed().reshape(-1), torch.from_numpy(embed[0]).cuda())
    g = torch.Generator(device="cuda").manual_seed(9)
    p.g.normal_(0.0, 1e-3, generator=g)
    opt = ShardedAdam(p.w, p.g, p.m, p.v, p.n_decay, p.n, lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=0.0)
    opt.step(c["adam_t"] + 1, 1.0)
    h.adam_t += 1
    out = str(tmp_path / "after.bin")
    ck.save_flat(out, h, p.w, p.m, p.v)
    h2, w2, m2, v2 = ck.load(out)
    assert h2.adam_t == c["adam_t"] + 1
    gh = p.g.cpu().numpy()
    for L in range(c["n_layers"]):
        for i, name in enumerate(ck.TENSORS[:9]):
            fo, cnt = ck.tensor_range(h, name, L, True)
            wo, _ = ck.tensor_range(h, name, L, False)
            w, m, v = (a.copy() for a in layers[L][i])
            v = np.abs(v)
            oracle.adam(w, gh[fo:fo + cnt].copy(), m, v, c["adam_t"] + 1, 3e-4, 0.9, 0.95, 1e-8, wd=0.1 if i < 7 else 0.0, variant=1)
            for got, want in ((w2, w), (m2, m), (v2, v)):
                err = np.abs(got[wo:wo + cnt].cpu().numpy() - want).max() / max(np.abs(want).max(), 1e-30)
                assert err <= 1e-5, (name, L)
