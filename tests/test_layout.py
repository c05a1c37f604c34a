"""Layout helpers around the operator set: GQA head tile / head sum (training_dynamic/io.h:327-351), fp32 <-> 16-bit
casts and the packed "activations + weights" surface (stories_io.h:41-58, io.h:33-50,79-95), vocabulary compaction
(cpu_ops.h:96-148).

CPU tests pin the oracle: the vocabulary functions against the reference's own code compiled from its headers, the
rest (whose reference lives in an Objective-C header that does not compile here) against numpy statements of the
same formulas.  GPU tests compare the CUDA entry points with the oracle: bit-exact for copies, casts, index maps and
fp32 sums; 16-bit head sums within one rounding of the fp32 sum."""
import numpy as np
import pytest

from oracle.oracle import Oracle, Reference, reference_available


@pytest.fixture(scope="module")
def orc():
    return Oracle()


def _tokens(rng, n, vocab, used):
    ids = rng.choice(vocab, size=used, replace=False)
    return ids[rng.integers(0, used, size=n)].astype(np.int32)


# ------------------------------------------------------------------------------------------------ CPU: oracle pins
def test_oracle_gqa_matches_numpy(orc):
    rng = np.random.default_rng(1)
    B, kv, ratio, hd, S = 2, 3, 4, 8, 10
    x = rng.standard_normal((B, kv * hd, S)).astype(np.float32)
    t = orc.gqa_tile(x, kv, ratio)
    want = np.repeat(x.reshape(B, kv, 1, hd, S), ratio, axis=2).reshape(B, kv * ratio * hd, S)
    assert np.array_equal(t, want)
    y = rng.standard_normal((B, kv * ratio * hd, S)).astype(np.float32)
    r = orc.gqa_reduce(y, kv, ratio)
    acc = np.zeros((B, kv, hd, S), np.float32)
    for q in range(ratio):                              # same order of fp32 additions
        acc = acc + y.reshape(B, kv, ratio, hd, S)[:, :, q]
    assert np.array_equal(r, acc.reshape(B, kv * hd, S))
    # reduce(tile(x)) = ratio * x exactly for a power-of-two ratio
    assert np.array_equal(orc.gqa_reduce(t, kv, ratio), ratio * x)


def test_oracle_casts_and_pack_match_numpy(orc):
    rng = np.random.default_rng(2)
    x = np.concatenate([rng.standard_normal(5000).astype(np.float32) * 10.0 ** rng.integers(-6, 5, 5000),
                        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, -7e4, np.inf], np.float32)]).astype(np.float32)
    h = orc.cvt_f32_f16(x)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    assert np.array_equal(h.view(np.uint16), want.view(np.uint16))                      # round to nearest even, overflow to inf
    assert np.array_equal(orc.cvt_f16_f32(h), h.astype(np.float32))
    act = rng.standard_normal((7, 12)).astype(np.float32)
    W = rng.standard_normal((7, 5)).astype(np.float32)
    packed = orc.pack_dyn(act, W)
    assert np.array_equal(packed.view(np.uint16), np.concatenate([act, W], axis=1).astype(np.float16).view(np.uint16))


@pytest.mark.skipif(not reference_available(), reason="the reference's headers are not present on this machine")
def test_oracle_vocab_rows_match_compiled_reference(orc):
    ref = Reference()
    rng = np.random.default_rng(3)
    V, dim, n = 500, 24, 2000
    tok = _tokens(rng, n, V, 173)
    cv, f2c, c2f = orc.vocab_map_build(tok, V)
    cv_r, f2c_r, c2f_r = ref.vocab_map_build(tok.astype(np.uint16), V)
    assert cv == cv_r == 173 and np.array_equal(f2c, f2c_r) and np.array_equal(c2f[:cv], c2f_r[:cv])
    full = rng.standard_normal((V, dim)).astype(np.float32)
    comp = rng.standard_normal((cv, dim)).astype(np.float32)
    assert np.array_equal(orc.vocab_compact_embed(full, c2f, cv), ref.vocab_rows("compact_embed", np.zeros((cv, dim), np.float32), full, c2f_r, cv))
    assert np.array_equal(orc.vocab_scatter_grads(full, comp, c2f, cv), ref.vocab_rows("scatter_grads", full, comp, c2f_r, cv))
    assert np.array_equal(orc.vocab_update_full(full, comp, c2f, cv), ref.vocab_rows("update_full", full, comp, c2f_r, cv))


# ------------------------------------------------------------------------------------------------ GPU parity
def _cuda():
    import torch
    from ane_b200 import lib
    assert torch.cuda.is_available(), "needs a CUDA device"
    lib.init(0)
    return torch


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("shape", [(2, 8, 2, 128, 256), (1, 3, 4, 8, 10), (3, 2, 1, 5, 7), (1, 1, 6, 2, 3)])
def test_gqa_tile_and_reduce(orc, dtype, shape):
    torch = _cuda()
    from ane_b200 import dev_ops as ops
    B, kv, ratio, hd, S = shape
    tdt = getattr(torch, dtype)
    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.standard_normal((B, kv * hd, S)).astype(np.float32)).to(tdt).cuda()
    t = ops.gqa_tile(x, kv, ratio)
    want = orc.gqa_tile(x.float().cpu().numpy(), kv, ratio)
    assert np.array_equal(t.float().cpu().numpy(), want)                               # a copy: bit-exact in every type
    y = torch.from_numpy(rng.standard_normal((B, kv * ratio * hd, S)).astype(np.float32)).to(tdt).cuda()
    r = ops.gqa_reduce(y, kv, ratio)
    want = orc.gqa_reduce(y.float().cpu().numpy(), kv, ratio)
    if dtype == "float32":
        assert np.array_equal(r.cpu().numpy(), want)                                   # same fp32 additions in the same order
    else:
        # fp32 sum of the 16-bit inputs, one rounding on store
        assert np.array_equal(r.float().cpu().numpy(), torch.from_numpy(want).to(tdt).float().numpy())


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 7, 8, 4096 + 3, 1 << 20])
def test_convert_matches_oracle(orc, n):
    torch = _cuda()
    from ane_b200 import dev_ops as ops
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n).astype(np.float32) * 10.0 ** rng.integers(-6, 5, n)).astype(np.float32)
    if n >= 8:
        x[:8] = np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, -7e4, np.inf], np.float32)
    xd = torch.from_numpy(x).cuda()
    h = ops.convert(xd, torch.float16)
    assert np.array_equal(h.cpu().numpy().view(np.uint16), orc.cvt_f32_f16(x).view(np.uint16))
    back = ops.convert(h, torch.float32)
    assert np.array_equal(back.cpu().numpy().view(np.uint32), orc.cvt_f16_f32(h.cpu().numpy()).view(np.uint32))
    # bfloat16 has no counterpart in the reference; the cast must agree with round-to-nearest-even
    b = ops.convert(xd, torch.bfloat16)
    assert torch.equal(b, xd.to(torch.bfloat16))
    # unaligned views take the element-wise path
    if n > 9:
        h2 = ops.convert(xd[3:], torch.float16)            # a view 12 bytes past a 16-byte boundary
        assert np.array_equal(h2.cpu().numpy().view(np.uint16), orc.cvt_f32_f16(x[3:]).view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(64, 256, 64), (7, 12, 5), (1, 1, 1), (33, 1000, 129)])
def test_pack_dyn_matches_oracle(orc, shape):
    torch = _cuda()
    from ane_b200 import dev_ops as ops
    ic, seq, oc = shape
    rng = np.random.default_rng(5)
    act = rng.standard_normal((ic, seq)).astype(np.float32)
    W = rng.standard_normal((ic, oc)).astype(np.float32)
    got = ops.pack_dyn(torch.from_numpy(act).cuda(), torch.from_numpy(W).cuda())
    assert np.array_equal(got.cpu().numpy().view(np.uint16), orc.pack_dyn(act, W).view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(500, 24, 2000, 173, "int32"), (32000, 768, 65536, 9200, "uint16"), (151936, 1024, 65536, 40000, "int32"),
                                  (10, 3, 5, 1, "int32")])
def test_vocab_compaction_matches_oracle(orc, case):
    torch = _cuda()
    from ane_b200 import dev_ops as ops, lib
    V, dim, n, used, idt = case
    rng = np.random.default_rng(V)
    tok = _tokens(rng, n, V, used)
    cv, f2c_o, c2f_o = orc.vocab_map_build(tok, V)
    tok_d = torch.from_numpy(tok).cuda() if idt == "int32" else torch.from_numpy(tok.astype(np.uint16).view(np.int16)).cuda()
    f2c, c2f, cnt = ops.vocab_map_build(tok_d, V)
    assert int(cnt.item()) == cv
    assert np.array_equal(f2c.cpu().numpy(), f2c_o)                                    # index work: bit-exact
    assert np.array_equal(c2f.cpu().numpy()[:cv], c2f_o[:cv])
    full = rng.standard_normal((V, dim)).astype(np.float32)
    comp = rng.standard_normal((cv, dim)).astype(np.float32)
    full_d, comp_d = torch.from_numpy(full).cuda(), torch.from_numpy(comp).cuda()
    ce = ops.vocab_compact_embed(full_d, c2f, cnt, cv)
    assert np.array_equal(ce.cpu().numpy(), orc.vocab_compact_embed(full, c2f_o, cv))
    g = ops.vocab_scatter_grads(full_d.clone(), comp_d, c2f, cnt, cv)
    assert np.array_equal(g.cpu().numpy(), orc.vocab_scatter_grads(full, comp, c2f_o, cv))
    u = ops.vocab_update_full(full_d.clone(), comp_d, c2f, None, cv)                   # row count given by the host
    assert np.array_equal(u.cpu().numpy(), orc.vocab_update_full(full, comp, c2f_o, cv))
    # compact-vocabulary round trip: gather, change, write back, gather again
    assert torch.equal(ops.vocab_compact_embed(u, c2f, cnt, cv), comp_d)
    assert lib.poll_status().oor_ids == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bfloat16", "float32", "float16"])
@pytest.mark.parametrize("case", [(2, 8, 2, 128, 256), (1, 2, 4, 128, 192), (3, 4, 2, 64, 128), (1, 1, 4, 64, 64)])
def test_head_sum_folded_into_k_backward(orc, dtype, case):
    """ane_cuda_rope_qknorm_bwd_gqa_dev equals gqa_reduce followed by rope_qknorm_bwd bit for bit (dx and dw), and the
    unfused pair equals the oracle's gqa_reduce + rope_qknorm_bwd within the storage type's tolerance."""
    torch = _cuda()
    from ane_b200 import dev_ops as ops
    B, kv, ratio, hd, S = case
    tdt = getattr(torch, dtype)
    rng = np.random.default_rng(31)
    x = torch.from_numpy(rng.standard_normal((B, kv * hd, S)).astype(np.float32)).to(tdt).cuda()
    dyt = torch.from_numpy(rng.standard_normal((B, kv * ratio * hd, S)).astype(np.float32)).to(tdt).cuda()
    w = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).cuda()
    dw_a, dw_b = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda")
    fused = ops.rope_qknorm_bwd_gqa(dyt, x, w, dw_a, hd, ratio)
    dk = ops.gqa_reduce(dyt, kv, ratio)
    plain = ops.rope_qknorm_bwd(dk, x, w, dw_b, hd)
    assert torch.equal(fused, plain)
    assert torch.equal(dw_a, dw_b)
    # and the pair against the oracle
    rdk = torch.from_numpy(orc.gqa_reduce(dyt.float().cpu().numpy(), kv, ratio)).to(tdt).float().numpy()
    rdx, rdw = orc.rope_qknorm_bwd(rdk, x.float().cpu().numpy(), w.cpu().numpy(), hd, eps=1e-6, base=1e6)
    got = fused.float().cpu().numpy()
    scale = np.abs(rdx).max()
    tol = 1e-5 if dtype == "float32" else (2.0 ** -8 if dtype == "bfloat16" else 2.0 ** -11)
    assert np.abs(got - rdx).max() <= tol * scale
    assert np.abs(dw_a.cpu().numpy() - rdw).max() <= (1e-5 if dtype == "float32" else 1e-4) * np.abs(rdw).max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("case", [(2, 8, 2, 128, 256), (1, 2, 4, 128, 192), (3, 4, 3, 64, 128)])
def test_k_forward_written_into_the_tiled_layout(dtype, case):
    """ane_cuda_qknorm_rope_tiled_dev equals qknorm_rope followed by gqa_tile bit for bit."""
    torch = _cuda()
    from ane_b200 import dev_ops as ops
    B, kv, ratio, hd, S = case
    tdt = getattr(torch, dtype)
    rng = np.random.default_rng(41)
    x = torch.from_numpy(rng.standard_normal((B, kv * hd, S)).astype(np.float32)).to(tdt).cuda()
    w = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).cuda()
    fused = ops.qknorm_rope_tiled(x, w, hd, ratio)
    assert torch.equal(fused, ops.gqa_tile(ops.qknorm_rope(x, w, hd), kv, ratio))


# More (token tile, KV head) items than the persistent grid of the TMA kernels holds (296 blocks over 64-token tiles):
# every block steps through several full rounds and the ragged last round is shared out head by head.
GQA_ROUNDS = [(10, 8, 2, 128, 2048), (19, 4, 4, 128, 2048), (21, 2, 2, 128, 1024 + 72)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("case", GQA_ROUNDS)
def test_gqa_fused_k_side_over_several_rounds_against_the_oracle(orc, dtype, case):
    """ane_cuda_qknorm_rope_tiled_dev and ane_cuda_rope_qknorm_bwd_gqa_dev at Qwen3's sequence length (base 1e6,
    positions to 2047) with 320 to 608 token tiles, each against the oracle's own sequence of operators
    (qknorm_rope then gqa_tile; gqa_reduce then rope_qknorm_bwd), in both forms of the norm backward."""
    torch = _cuda()
    from ane_b200 import dev_ops as ops
    from ane_b200 import lib
    B, kv, ratio, hd, S = case
    tdt = getattr(torch, dtype)
    rng = np.random.default_rng(43)
    x = torch.from_numpy(rng.standard_normal((B, kv * hd, S)).astype(np.float32)).to(tdt).cuda()
    dyt = torch.from_numpy(rng.standard_normal((B, kv * ratio * hd, S)).astype(np.float32)).to(tdt).cuda()
    w_np = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    w = torch.from_numpy(w_np).cuda()
    xr = x.float().cpu().numpy()
    tol = 1e-5 if dtype == "float32" else 2.0 ** -8
    lib.poll_status(reset=True)

    fwd = ops.qknorm_rope_tiled(x, w, hd, ratio).float().cpu().numpy()
    want = orc.gqa_tile(orc.qknorm_rope(xr, w_np, hd, 1e-6, 1e6, 0), kv, ratio)
    assert np.abs(fwd - want).max() <= tol * np.abs(want).max()
    if dtype != "float32":
        l2 = np.sqrt(((fwd - want).astype(np.float64) ** 2).sum() / (want.astype(np.float64) ** 2).sum())
        assert l2 <= 2e-3

    rdk = torch.from_numpy(orc.gqa_reduce(dyt.float().cpu().numpy(), kv, ratio)).to(tdt).float().numpy()
    for exact in (False, True):
        dw = torch.zeros(hd, device="cuda")
        got = ops.rope_qknorm_bwd_gqa(dyt, x, w, dw, hd, ratio, exact=exact).float().cpu().numpy()
        rdx, rdw = orc.rope_qknorm_bwd(rdk, xr, w_np, hd, eps=1e-6, base=1e6, exact=exact)
        assert np.abs(got - rdx).max() <= tol * np.abs(rdx).max()
        assert np.abs(dw.cpu().numpy() - rdw).max() <= (1e-5 if dtype == "float32" else 1e-4) * np.abs(rdw).max()
    assert lib.poll_status().wait_giveups == 0
