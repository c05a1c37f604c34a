"""CPU tests that pin the oracle (the C restatement in oracle/oracle_ops.c).

Pins, strongest first:
 * the committed golden vectors -- outputs of the reference's own functions
   (training/stories_cpu_ops.h, training/training_dynamic/cpu_ops.h) on the seeded fixtures of
   training/test_rmsnorm_bwd.m:26-33 and training/test_classifier.m:25-27,132-134 and on
   PCG64 inputs;
 * where oracle/_ref is built, the reference functions themselves, run live.
Tolerance for fp32: 1e-5 of the tensor's max magnitude (the figure the library is held to);
index/byte work is bit-exact.
"""
import ctypes

import numpy as np
import pytest

from tests.conftest import rel_err
from tests.golden import gen_inputs as gi

TOL = 1e-5


def _sampled(g, name, full):
    s = int(g[name + "_stride"])
    return np.ascontiguousarray(full).reshape(-1)[::s], g[name]


def test_drand48_matches_libc():
    libc = ctypes.CDLL("libc.so.6")
    libc.drand48.restype = ctypes.c_double
    libc.srand48(999)
    ref = np.array([libc.drand48() for _ in range(9000)])
    assert np.array_equal(ref, gi.Drand48(999).next(9000))


def test_bf16_round_helpers():
    a = np.array([1.0, 1.00390625, 1.005859375, -3.14159, 65504.0, 1e-40], np.float32)
    r = gi.round_bf16(a)
    import torch
    t = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(r, t)


@pytest.mark.parametrize("variant", ["stories", "dynamic"])
def test_rmsnorm_bwd_reference_fixture(golden, oracle, variant):
    x, dy, w = gi.fixture_rmsnorm_bwd()
    dx, dw = oracle.rmsnorm_bwd(dy, x, w)
    got, want = _sampled(golden, f"rmsbwd_fixture_{variant}_dx", dx)
    assert rel_err(got, want) <= TOL
    assert rel_err(dw, golden[f"rmsbwd_fixture_{variant}_dw"]) <= TOL
    assert abs(dx.astype(np.float64).sum() - golden[f"rmsbwd_fixture_{variant}_dx_sum"]) <= 1e-5 * golden[
        f"rmsbwd_fixture_{variant}_dx_abssum"]


@pytest.mark.parametrize("variant", ["stories", "dynamic"])
def test_rmsnorm_fwd_reference_fixture(golden, oracle, variant):
    x, w = gi.fixture_rmsnorm_fwd()
    got, want = _sampled(golden, f"rms_fixture_{variant}_out", oracle.rmsnorm(x, w))
    assert rel_err(got, want) <= TOL


def test_rmsnorm_bwd_is_the_reference_form_not_the_analytic_one(oracle):
    """The reference multiplies both dx terms by w (stories_cpu_ops.h:42-46); with w != 1 this
    is far from the analytic gradient, which `exact` selects (ane_rmsnorm_bwd.h:56,70-74)."""
    x, dy, w = gi.fixture_rmsnorm_bwd()
    dx_ref, dw_ref = oracle.rmsnorm_bwd(dy, x, w)
    dx_ex, dw_ex = oracle.rmsnorm_bwd(dy, x, w, exact=True)
    assert rel_err(dx_ex, dx_ref) > 1e-3
    assert np.array_equal(dw_ex, dw_ref)
    # analytic form against a float64 derivation
    xd, dyd, wd = x.astype(np.float64), dy.astype(np.float64), w.astype(np.float64)
    rr = 1.0 / np.sqrt((xd * xd).mean(axis=0) + 1e-5)
    dot = (dyd * xd * wd[:, None]).sum(axis=0) * rr * rr / x.shape[0]
    want = (dyd * wd[:, None] - xd * dot) * rr
    assert rel_err(dx_ex, want) <= TOL


def test_cfg1_golden(golden, oracle):
    x, w, dy = gi.cfg1()
    got, want = _sampled(golden, "cfg1_rms_out", oracle.rmsnorm(x[0], w))
    assert rel_err(got, want) <= TOL
    dx, dw = oracle.rmsnorm_bwd(dy[0], x[0], w)
    got, want = _sampled(golden, "cfg1_rmsbwd_dx", dx)
    assert rel_err(got, want) <= TOL
    assert rel_err(dw, golden["cfg1_rmsbwd_dw"]) <= TOL


@pytest.mark.parametrize("variant", ["stories", "dynamic"])
def test_cross_entropy_reference_fixture(golden, oracle, variant):
    logits = gi.fixture_softmax_logits()
    tg = golden["ce_fixture_targets"].astype(np.int32)
    loss, dl, oor = oracle.cross_entropy(logits, tg)
    assert oor == 0
    assert abs(float(loss[0]) - float(golden[f"ce_fixture_{variant}_loss"])) <= TOL * abs(
        float(golden[f"ce_fixture_{variant}_loss"]))
    got, want = _sampled(golden, f"ce_fixture_{variant}_dlogits", dl)
    assert rel_err(got, want) <= TOL
    # probabilities of the first four positions sum to one (training/test_classifier.m:173-185)
    assert np.allclose(golden[f"ce_fixture_{variant}_psum4"], 1.0, atol=1e-4)


@pytest.mark.parametrize("name,wd,b2,variant", [("stories", 0.0, 0.999, 0), ("dynamic", 0.1, 0.95, 1)])
def test_adam_golden(golden, oracle, name, wd, b2, variant):
    w, g, m, v = gi.adam_inputs()
    for t in (1, 2, 3):
        oracle.adam(w, g, m, v, t, 3e-4, 0.9, b2, 1e-8, wd=wd, variant=variant)
    for arr, key in ((w, "w"), (m, "m"), (v, "v")):
        got, want = _sampled(golden, f"adam_{name}_{key}", arr)
        assert rel_err(got, want) <= TOL


def test_embed_golden_bit_exact(golden, oracle):
    r = gi.rng(77)
    tok = r.integers(0, 32000, size=256).astype(np.uint16)
    tok[10:20] = tok[0]
    assert np.array_equal(tok, golden["embed_tokens"])
    table = gi.normal(r, (32000, 768), 0.02)
    x, oor = oracle.embed_lookup(table, tok.astype(np.int32)[None])
    assert oor == 0
    got, want = _sampled(golden, "embed_lookup_x", x[0])
    assert np.array_equal(got, want)          # gather is a bit-exact copy
    dxe = gi.normal(r, (768, 256))
    dE, _ = oracle.embed_backward(np.zeros((32000, 768), np.float32), dxe[None], tok.astype(np.int32)[None])
    rows = dE[tok[:32].astype(np.int64)][:, ::7]
    assert np.array_equal(rows, golden["embed_backward_rows"])   # same sequential order -> same bits


def test_embed_out_of_range_is_skipped(oracle):
    table = gi.normal(gi.rng(5), (100, 8))
    tok = np.array([[3, 100, -1, 99]], np.int32)
    init = np.full((1, 8, 4), 7.0, np.float32)
    x, oor = oracle.embed_lookup(table, tok, x_init=init)
    assert oor == 2
    assert np.all(x[0, :, 1] == 7.0) and np.all(x[0, :, 2] == 7.0)   # stale columns (stories_cpu_ops.h:115)
    assert np.array_equal(x[0, :, 0], table[3]) and np.array_equal(x[0, :, 3], table[99])


@pytest.mark.parametrize("name,dim,hd", [("hd64", 768, 64), ("hd128", 2048, 128)])
def test_rope_bwd_golden(golden, oracle, name, dim, hd):
    d = gi.normal(gi.rng(88), (dim, 256))
    got, want = _sampled(golden, f"ropebwd_{name}", oracle.rope(d, hd, base=10000.0, inverse=True))
    assert rel_err(got, want) <= TOL


def test_rope_forward_then_backward_is_identity(oracle):
    d = gi.normal(gi.rng(3), (2, 256, 64))
    y = oracle.rope(d, 64, base=1e6, pos0=5)
    z = oracle.rope(y, 64, base=1e6, pos0=5, inverse=True)
    assert rel_err(z, d) <= 1e-6
    # against the row-major statement of training/forward.h:55-70 in float64
    S, hd = 64, 64
    i = np.arange(hd // 2)
    freq = 1.0 / np.power(np.float32(1e6), (2.0 * i / hd).astype(np.float32)).astype(np.float32)
    th = (np.arange(S)[None, :] + 5).astype(np.float32) * freq[:, None].astype(np.float32)
    c, s = np.cos(th.astype(np.float64)), np.sin(th.astype(np.float64))
    x4 = d.astype(np.float64).reshape(2, 4, hd // 2, 2, S)
    a, b = x4[:, :, :, 0], x4[:, :, :, 1]
    want = np.stack([a * c - b * s, a * s + b * c], axis=3).reshape(d.shape)
    assert rel_err(y, want) <= TOL


def test_swiglu_matches_float64(oracle):
    h1, h3, d, _, _ = gi.cfg2()
    out = oracle.swiglu(h1, h3)
    h1d, h3d, dd = h1.astype(np.float64), h3.astype(np.float64), d.astype(np.float64)
    sig = 1.0 / (1.0 + np.exp(-h1d))
    assert rel_err(out, h1d * sig * h3d) <= TOL
    dh1, dh3 = oracle.swiglu_bwd(h1, h3, d)
    assert rel_err(dh3, dd * h1d * sig) <= TOL
    assert rel_err(dh1, dd * h3d * sig * (1 + h1d * (1 - sig))) <= TOL   # training/backward.h:44-47


def test_residual_and_grad_post(oracle):
    _, _, _, x, f = gi.cfg2()
    alpha = np.float32(1.0 / np.sqrt(np.float32(2.0 * 12)))          # train.m:188
    assert np.array_equal(oracle.residual(x, f, alpha), f * alpha + x)
    g = gi.normal(gi.rng(9), (100000,), 0.5)
    nsq = oracle.grad_norm_sq(g, 1.0 / 2560.0)
    assert abs(nsq - float(((g.astype(np.float64) / 2560.0) ** 2).sum())) <= 1e-6 * nsq
    assert oracle.clip_factor(4.0, 1.0) == pytest.approx(0.5)
    assert oracle.clip_factor(0.25, 1.0) == 1.0
    assert oracle.clip_factor(4.0, 0.0) == 1.0


def test_qknorm_is_per_head_rmsnorm(oracle):
    q, k, wq, wk, dq, dk = gi.cfg3(seq=64)
    y = oracle.qknorm(q, wq, 128)
    for h in (0, 7, 15):
        want = oracle.rmsnorm(q[0, h * 128:(h + 1) * 128], wq, eps=1e-6)
        assert np.array_equal(y[0, h * 128:(h + 1) * 128], want)
    fused = oracle.qknorm_rope(q, wq, 128)
    assert np.array_equal(fused, oracle.rope(y, 128, base=1e6))
    dx, dw = oracle.rope_qknorm_bwd(dq, q, wq, 128)
    gq = oracle.rope(dq, 128, base=1e6, inverse=True)
    dx2, dw2 = oracle.qknorm_bwd(gq, q, wq, 128)
    assert np.array_equal(dx, dx2) and np.array_equal(dw, dw2)


def test_vocab_map_golden(golden, oracle):
    data = gi.rng(99).integers(0, 32000, size=20000).astype(np.uint16)
    cv, f2c, c2f = oracle.vocab_map_build(data, 32000)
    assert cv == int(golden["vocab_cv"])
    assert np.array_equal(c2f[:64], golden["vocab_c2f_head"])
    assert int(f2c.astype(np.int64).sum()) == int(golden["vocab_f2c_sum"])


# ------------------------------------------------------------------ live reference (when built)
def _reference():
    from oracle.oracle import Reference, reference_available
    if not reference_available():
        pytest.skip("oracle/_ref not built on this box")
    return Reference()


def test_live_reference_norms_and_ce(oracle):
    ref = _reference()
    x, w, dy = gi.cfg1(seed=4321)
    for variant in ("stories", "dynamic"):
        assert rel_err(oracle.rmsnorm(x[0], w), ref.rmsnorm(x[0], w, variant)) <= TOL
        dx, dw = oracle.rmsnorm_bwd(dy[0], x[0], w)
        rdx, rdw = ref.rmsnorm_bwd(dy[0], x[0], w, variant=variant)
        assert rel_err(dx, rdx) <= TOL and rel_err(dw, rdw) <= TOL
    logits = gi.cfg4_logits(B=1, vocab=9000, seq=64)[0]
    tg = gi.rng(1).integers(0, 9000, size=64).astype(np.uint16)
    for variant in ("stories", "dynamic"):
        rl, rdl = ref.cross_entropy_loss(logits, tg, variant)
        loss, dl, _ = oracle.cross_entropy(logits, tg.astype(np.int32))
        assert abs(loss[0] - rl) <= TOL * abs(rl)
        assert rel_err(dl, rdl) <= TOL


def test_live_reference_ce_out_of_range_quirk(oracle):
    """stories_cpu_ops.h:94-103: an out-of-range target leaves the plain softmax in the column."""
    ref = _reference()
    logits = gi.cfg4_logits(B=1, vocab=500, seq=8)[0]
    tg = np.array([1, 2, 600, 3, 4, 5, 6, 7], np.uint16)
    rl, rdl = ref.cross_entropy_loss(logits, tg, "stories")
    loss, dl, oor = oracle.cross_entropy(logits, tg.astype(np.int32))
    assert oor == 1
    assert abs(loss[0] - rl) <= TOL * abs(rl)
    assert rel_err(dl, rdl) <= TOL
    assert abs(dl[:, 2].sum() - 1.0) < 1e-4


# ------------------------------------------------------------------ the reference's inline blocks, compiled by line range
def _grad_post_by_oracle(oracle):
    """Scale, norm and clip the way the library folds them: norm of the scaled gradient, one clip factor, g*gsc*factor."""
    layers, fin, emb = gi.grad_post_inputs()
    flat = gi.grad_post_flat(layers, fin, emb)
    nsq = oracle.grad_norm_sq(flat, gi.GRAD_POST_GSC)
    cf = oracle.clip_factor(np.float32(nsq), 1.0)
    return (flat * np.float32(gi.GRAD_POST_GSC)) * np.float32(cf), nsq, cf


def test_inline_blocks_golden(golden, oracle):
    """SwiGLU fwd / bwd, the DeepNet residual, RoPE forward and the gradient scale / norm / clip chain against the
    committed outputs of the reference's own statements (training_dynamic/train.m:460,538-554,754-825,
    training/forward.h:55-70,101,149-151)."""
    h1, h3, d, x, f = (a[0] for a in gi.cfg2())
    dh1, dh3 = oracle.swiglu_bwd(h1, h3, d)
    for name, got in (("inline_swiglu_bwd_dh1", dh1), ("inline_swiglu_bwd_dh3", dh3), ("inline_swiglu", oracle.swiglu(h1, h3))):
        assert rel_err(got.reshape(-1)[::int(golden[name + "_stride"])], golden[name]) <= TOL
    for name, alpha in (("a25", np.float32(24.0 ** -0.25)), ("a50", np.float32(1.0) / np.sqrt(np.float32(24.0)))):
        got = oracle.residual(x, f, alpha)
        assert np.array_equal(got.reshape(-1)[::int(golden[f"inline_residual_{name}_stride"])], golden[f"inline_residual_{name}"])
    q = gi.cfg3()[0][0]
    for name, arr, hd in (("inline_rope_hd128", q, 128), ("inline_rope_hd64", np.ascontiguousarray(q[:768]), 64)):
        got = oracle.rope(arr, hd, base=10000.0)
        assert rel_err(got.reshape(-1)[::int(golden[name + "_stride"])], golden[name]) <= TOL
    flat, nsq, cf = _grad_post_by_oracle(oracle)
    assert cf < 1.0                                                       # the clip branch ran
    assert abs(np.sqrt(nsq) - float(golden["inline_grad_norm"])) <= TOL * float(golden["inline_grad_norm"])
    assert rel_err(flat[::int(golden["inline_grad_flat_stride"])], golden["inline_grad_flat"]) <= TOL


def _reference_inline():
    from oracle.oracle import ReferenceInline, reference_inline_available
    if not reference_inline_available():
        pytest.skip("oracle/_ref/libref_inline.so not built on this box")
    return ReferenceInline()


def test_live_reference_swiglu(oracle):
    """train.m:538-554 (13 vDSP passes) and forward.h:101,149-151 compiled, on other seeds and a ragged size."""
    ref = _reference_inline()
    for seed, hidden, seq in ((7, 2048, 256), (8, 33, 5)):
        h1, h3, d, _, _ = (a[0] for a in gi.cfg2(seed=seed, hidden=hidden, seq=seq))
        dh1, dh3 = oracle.swiglu_bwd(h1, h3, d)
        rdh1, rdh3 = ref.swiglu_bwd(h1, h3, d)
        assert rel_err(dh1, rdh1) <= TOL and rel_err(dh3, rdh3) <= TOL
        assert rel_err(oracle.swiglu(h1, h3), ref.swiglu(h1, h3)) <= TOL


def test_live_reference_residual(oracle):
    """train.m:460 compiled: x + alpha*f, bit for bit, for the alpha of train.m:188, the benchmark's and 1."""
    ref = _reference_inline()
    _, _, _, x, f = (a[0] for a in gi.cfg2(seed=9))
    for alpha in (np.float32(1.0) / np.sqrt(np.float32(24.0)), np.float32(24.0 ** -0.25), np.float32(1.0)):
        assert np.array_equal(oracle.residual(x, f, alpha), ref.residual(x, f, alpha))


def test_live_reference_rope_forward(oracle):
    """forward.h:55-70 compiled (row-major, base 10000) against the channel-first restatement."""
    ref = _reference_inline()
    q = gi.cfg3(seed=10)[0][0]
    assert rel_err(oracle.rope(q, 128, base=10000.0), ref.rope_channel_first(q, 128)) <= TOL
    q64 = np.ascontiguousarray(q[:768, :100])
    assert rel_err(oracle.rope(q64, 64, base=10000.0), ref.rope_channel_first(q64, 64)) <= TOL


def test_live_reference_grad_scale_norm_clip(oracle):
    """train.m:754-767 (scale), :770-788 (norm), :809-825 (clip) compiled, against the folded form the library uses
    (norm of the scaled gradient, then g * gscale * factor inside Adam); with and without the clip triggering."""
    ref = _reference_inline()
    for clip in (1.0, 1e9, 0.0):
        layers, fin, emb = gi.grad_post_inputs(seed=77)
        flat0 = gi.grad_post_flat(layers, fin, emb)
        norm, nsq = ref.grad_scale_norm_clip(layers, fin, emb, gi.GRAD_POST_GSC, clip)
        want_nsq = oracle.grad_norm_sq(flat0, gi.GRAD_POST_GSC)
        assert abs(nsq - want_nsq) <= TOL * want_nsq
        cf = oracle.clip_factor(np.float32(want_nsq), clip)
        assert (cf < 1.0) == (clip == 1.0)
        want = (flat0 * np.float32(gi.GRAD_POST_GSC)) * np.float32(cf)
        assert rel_err(gi.grad_post_flat(layers, fin, emb), want) <= TOL
