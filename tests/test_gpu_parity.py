"""GPU parity tests: every operator of libane_cuda, called through its C ABI, against the CPU
oracle (oracle/oracle_ops.c) on the same seeded inputs.

Tolerances:
  * fp32 operators               max |got - ref| / max |ref| <= 1e-5 per tensor
  * bf16 / fp16 variants         against the fp32 oracle run on the rounded inputs:
                                 relative L2 error <= 2e-3, max-norm error within the unit
                                 roundoff of the storage type (2^-8 bf16, 2^-11 fp16: one
                                 correctly rounded store of a value that is itself within
                                 1e-5), and all but a handful of elements bit-identical to
                                 the oracle's result rounded to the storage type
  * gathers, token indexing and the scatter-add (same addition order as the reference loop)
                                 bit-exact
Shapes cover the reference's own (DIM 768, SEQ 256, VOCAB 32000), the benchmark configurations
at sizes the oracle finishes in seconds, and ragged / tiny cases that break every alignment the
vector paths rely on.
"""
import ctypes as C

import numpy as np
import pytest

from tests.conftest import rel_err
from tests.golden import gen_inputs as gi

pytestmark = pytest.mark.gpu

TOL32 = 1e-5
TOL16 = 2e-3


@pytest.fixture(scope="module")
def dev():
    import torch
    from ane_b200 import dev_ops, lib
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    lib.init(0)
    return dev_ops


def _torch():
    import torch
    return torch


DT = {"f32": "float32", "bf16": "bfloat16", "f16": "float16"}


def up(a, dt="f32"):
    """numpy fp32 -> device tensor of dtype dt; also returns the rounded values as fp32 numpy."""
    torch = _torch()
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda().to(getattr(torch, DT[dt])).contiguous()
    return t, t.float().cpu().numpy()


def down(t):
    return t.float().cpu().numpy()


def tol(dt):
    return TOL32 if dt == "f32" else TOL16


UNIT_ROUNDOFF = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11}


def close(got, ref, dt):
    """True when `got` (fp32 view of the device result) matches the fp32 oracle result `ref`
    within the tolerance of storage type dt (see the module docstring)."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    if dt == "f32":
        return rel_err(got, ref) <= TOL32
    den = float(np.sqrt((ref * ref).sum())) or 1.0
    l2 = float(np.sqrt(((got - ref) ** 2).sum())) / den
    mx = rel_err(got, ref)
    rounded = gi.round_bf16(ref.astype(np.float32)) if dt == "bf16" else gi.round_f16(ref.astype(np.float32))
    mismatch = float(np.mean(rounded.astype(np.float64) != got)) if ref.size else 0.0
    l2_tol = TOL16 if ref.size >= 256 else UNIT_ROUNDOFF[dt] * 1.01     # the L2 figure is statistical
    ok = l2 <= l2_tol and mx <= UNIT_ROUNDOFF[dt] * 1.01 and mismatch <= max(2e-3, 2.0 / max(ref.size, 1))
    if not ok:
        print(f"close({dt}): rel L2 {l2:.3e}, max-norm {mx:.3e}, non-identical fraction {mismatch:.3e}")
    return ok


NORM_SHAPES = [(1, 768, 256), (3, 7, 5), (2, 128, 257), (1, 1, 1), (2, 1024, 64), (1, 2, 3), (5, 33, 48), (1, 300, 8),
               (2, 129, 64), (1, 3000, 32), (1, 3200, 40), (1, 64, 2048)]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_rmsnorm_fwd(dev, oracle, shape, dt):
    B, Cn, S = shape
    x, w, _ = gi.cfg1(seed=11, B=B, dim=Cn, seq=S)
    xd, xr = up(x, dt)
    wd, _ = up(w)
    got = down(dev.rmsnorm(xd, wd, 1e-5))
    assert close(got, oracle.rmsnorm(xr, w, 1e-5), dt)


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_rmsnorm_bwd(dev, oracle, shape, dt, exact):
    torch = _torch()
    B, Cn, S = shape
    x, w, dy = gi.cfg1(seed=12, B=B, dim=Cn, seq=S)
    xd, xr = up(x, dt)
    dyd, dyr = up(dy, dt)
    wd, _ = up(w)
    dw0 = gi.normal(gi.rng(5), (Cn,), 0.1)
    dwd, _ = up(dw0)
    dx = down(dev.rmsnorm_bwd(dyd, xd, wd, dwd, eps=1e-5, exact=exact))
    rdx, rdw = oracle.rmsnorm_bwd(dyr, xr, w, dw=dw0, eps=1e-5, exact=exact)
    assert close(dx, rdx, dt)
    assert rel_err(down(dwd), rdw) <= (TOL32 if dt == "f32" else 1e-4)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_rmsnorm_bwd_fused_add_and_determinism(dev, oracle, dt):
    torch = _torch()
    B, Cn, S = 4, 768, 256
    x, w, dy = gi.cfg1(seed=13, B=B, dim=Cn, seq=S)
    add = gi.normal(gi.rng(6), (B, Cn, S))
    xd, xr = up(x, dt)
    dyd, dyr = up(dy, dt)
    ad, ar = up(add, dt)
    wd, _ = up(w)
    dw1 = torch.zeros(Cn, device="cuda")
    dx1 = dev.rmsnorm_bwd(dyd, xd, wd, dw1, add=ad)
    rdx, rdw = oracle.rmsnorm_bwd(dyr, xr, w)
    assert close(down(dx1), oracle.add(rdx, ar), dt)          # train.m:590,721
    assert rel_err(down(dw1), rdw) <= (TOL32 if dt == "f32" else 1e-4)
    dw2 = torch.zeros(Cn, device="cuda")
    dx2 = dev.rmsnorm_bwd(dyd, xd, wd, dw2, add=ad)
    assert torch.equal(dx1, dx2) and torch.equal(dw1, dw2)              # bit-stable run to run


RING_SHAPES = [(1, 768, 256), (2, 1024, 64), (1, 3000, 32), (1, 3200, 40), (3, 257, 72), (2, 1024, 2048 + 8), (40, 1024, 512),
               (150, 256, 512)]


@pytest.mark.parametrize("knob", [0, 8, 9, 10, 11, 12])
@pytest.mark.parametrize("with_add", [False, True])
@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", RING_SHAPES)
def test_rmsnorm_bwd_cluster_of_four_kernels(dev, oracle, shape, dt, exact, with_add, knob):
    """Every persistent form of the backward (tuning knob norm_bwd = 0: two sweeps per tile, the second from L2;
    8: pair of blocks; 9: cluster of four, 64-byte rows, double-buffered strips; 10: cluster of four, 128-byte rows;
    11: cluster of eight, 256-byte rows; 12: cluster of eight, 128-byte rows, double-buffered strips): ragged channel parts (C = 257, 3000), ragged token tiles, more tiles than resident
    blocks, pairs or clusters (the last two shapes: 320 to 2400 tiles, so every block steps through several
    rounds and the last round is ragged), and the same bits from two runs."""
    torch = _torch()
    from ane_b200 import lib
    B, Cn, S = shape
    x, w, dy = gi.cfg1(seed=15, B=B, dim=Cn, seq=S)
    add = gi.normal(gi.rng(16), (B, Cn, S)) if with_add else None
    xd, xr = up(x, dt)
    dyd, dyr = up(dy, dt)
    wd, _ = up(w)
    ad, ar = up(add, dt) if with_add else (None, None)
    dw0 = gi.normal(gi.rng(5), (Cn,), 0.1)
    rdx, rdw = oracle.rmsnorm_bwd(dyr, xr, w, dw=dw0, eps=1e-5, exact=exact)
    if with_add:
        rdx = oracle.add(rdx, ar)
    lib.set_tuning("norm_bwd", knob)
    try:
        outs = []
        for _ in range(2):
            dwd, _ = up(dw0)
            dx = dev.rmsnorm_bwd(dyd, xd, wd, dwd, eps=1e-5, exact=exact, add=ad)
            outs.append((dx, dwd))
        assert close(down(outs[0][0]), rdx, dt)
        assert rel_err(down(outs[0][1]), rdw) <= (TOL32 if dt == "f32" else 1e-4)
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    finally:
        lib.clear_tuning("norm_bwd")


def test_rmsnorm_reference_fixtures_on_gpu(dev, golden):
    """The reference tests' own inputs (test_rmsnorm_bwd.m:26-33, test_classifier.m:25-27)
    against the committed outputs of the reference functions."""
    torch = _torch()
    x, dy, w = gi.fixture_rmsnorm_bwd()
    dw = torch.zeros(768, device="cuda")
    dx = down(dev.rmsnorm_bwd(up(dy)[0], up(x)[0], up(w)[0], dw))
    s = int(golden["rmsbwd_fixture_stories_dx_stride"])
    assert rel_err(dx.reshape(-1)[::s], golden["rmsbwd_fixture_stories_dx"]) <= TOL32
    assert rel_err(down(dw), golden["rmsbwd_fixture_stories_dw"]) <= TOL32
    x, w = gi.fixture_rmsnorm_fwd()
    out = down(dev.rmsnorm(up(x)[0], up(w)[0]))
    s = int(golden["rms_fixture_stories_out_stride"])
    assert rel_err(out.reshape(-1)[::s], golden["rms_fixture_stories_out"]) <= TOL32


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("n,off", [(2048 * 256, 0), (1, 0), (1023, 0), (4099, 1), (768 * 256, 3)])
def test_elementwise(dev, oracle, n, off, dt):
    """residual (train.m:460), scale (train.m:523), SwiGLU fwd (forward.h:101) and bwd
    (train.m:537-554); off > 0 shifts the pointers off 16-byte alignment."""
    torch = _torch()
    r = gi.rng(21)
    arrs = [gi.normal(r, (n + off,)) for _ in range(3)]
    (h1d, h1), (h3d, h3), (dd, d) = [up(a, dt) for a in arrs]
    h1d, h3d, dd = h1d[off:], h3d[off:], dd[off:]
    h1, h3, d = (np.ascontiguousarray(a[off:]) for a in (h1, h3, d))
    alpha = float(np.float32((2.0 * 12) ** -0.25))
    assert close(down(dev.residual(h1d, h3d, alpha, out=torch.empty_like(h1d))), oracle.residual(h1, h3, alpha), dt)
    assert close(down(dev.scale(h1d, alpha, out=torch.empty_like(h1d))), oracle.scale(h1, alpha), dt)
    assert close(down(dev.swiglu(h1d, h3d, out=torch.empty_like(h1d))), oracle.swiglu(h1, h3), dt)
    g1, g3 = dev.swiglu_bwd(h1d, h3d, dd, dh1=torch.empty_like(h1d), dh3=torch.empty_like(h1d))
    r1, r3 = oracle.swiglu_bwd(h1, h3, d)
    assert close(down(g1), r1, dt) and close(down(g3), r3, dt)


@pytest.mark.parametrize("exact", [0, 1])
def test_swiglu_over_the_whole_exponent_range(dev, oracle, exact):
    """SwiGLU forward and backward with h1 from -100 to 100 (exp(-h1) from 0 to overflow), both forms of the sigmoid: the
    default one from the hardware's ex2 / rcp approximations and the literal expf-and-division one (knob swiglu_exact).
    Element by element within 1e-5 of the oracle (train.m:537-554, forward.h:101), no NaN where the oracle has none.  The
    default form flushes a sigmoid below the normal range (h1 < -87.3: values under 1.2e-38) to zero, hence the absolute
    floor of 1e-34 on products of such a value with h1, h3 and d."""
    from ane_b200 import lib
    r = gi.rng(23)
    h1 = np.concatenate([np.linspace(-100, 100, 20001), gi.normal(r, (12000,), 3.0), [0.0, -0.0, 88.7, -88.7, 104.0, -104.0]]).astype(np.float32)
    h3 = gi.normal(r, h1.shape)
    d = gi.normal(r, h1.shape)
    lib.set_tuning("swiglu_exact", exact)
    try:
        out = down(dev.swiglu(up(h1)[0], up(h3)[0]))
        g1, g3 = (down(t) for t in dev.swiglu_bwd(up(h1)[0], up(h3)[0], up(d)[0]))
    finally:
        lib.clear_tuning("swiglu_exact")
    r1, r3 = oracle.swiglu_bwd(h1, h3, d)
    # dh1 = (d*h3) * sig * (1 + h1*(1 - sig)) cancels near h1 = -1.278: its error is measured against the size of its terms
    with np.errstate(over="ignore"):
        sig = 1.0 / (1.0 + np.exp(-h1.astype(np.float64)))
    terms1 = np.abs(d.astype(np.float64) * h3) * sig * (1.0 + np.abs(h1) * (1.0 - sig))
    ro = oracle.swiglu(h1, h3)
    for got, ref, size in ((out, ro, np.abs(ro)), (g1, r1, terms1), (g3, r3, np.abs(r3))):
        assert np.array_equal(np.isnan(got), np.isnan(ref))
        ok = np.abs(got.astype(np.float64) - ref) <= 1e-5 * size + 1e-34
        assert ok.all(), (int((~ok).sum()), h1[~ok][:5], got[~ok][:5], ref[~ok][:5])


def test_residual_alpha_of_the_reference(dev, oracle):
    """alpha = 1/sqrt(2*NLAYERS) (train.m:188) and alpha = 1 (train_large.m:427): bit-exact."""
    _, _, _, x, f = gi.cfg2()
    for alpha in (float(np.float32(1.0) / np.sqrt(np.float32(24.0))), 1.0):
        got = down(dev.residual(up(x)[0], up(f)[0], alpha))
        assert np.array_equal(got, oracle.residual(x, f, alpha))


def test_inline_reference_blocks_golden_on_gpu(dev, golden):
    """The reference's own inline statements (training_dynamic/train.m:460 residual, :538-554 SwiGLU backward,
    :754-825 gradient scale / norm / clip; training/forward.h:55-70 RoPE forward, :101,149-151 SwiGLU gate), compiled
    where the reference is and committed as golden vectors, against the device operators."""
    torch = _torch()

    def sampled(t, name):
        return down(t).reshape(-1)[::int(golden[name + "_stride"])]

    h1, h3, d, x, f = (a[0] for a in gi.cfg2())
    g1, g3 = dev.swiglu_bwd(up(h1)[0], up(h3)[0], up(d)[0])
    assert rel_err(sampled(g1, "inline_swiglu_bwd_dh1"), golden["inline_swiglu_bwd_dh1"]) <= TOL32
    assert rel_err(sampled(g3, "inline_swiglu_bwd_dh3"), golden["inline_swiglu_bwd_dh3"]) <= TOL32
    assert rel_err(sampled(dev.swiglu(up(h1)[0], up(h3)[0]), "inline_swiglu"), golden["inline_swiglu"]) <= TOL32
    for name, alpha in (("a25", np.float32(24.0 ** -0.25)), ("a50", np.float32(1.0) / np.sqrt(np.float32(24.0)))):
        got = dev.residual(up(x)[0], up(f)[0], float(alpha))
        assert np.array_equal(sampled(got, f"inline_residual_{name}"), golden[f"inline_residual_{name}"])
    q = gi.cfg3()[0][0]
    for name, arr, hd in (("inline_rope_hd128", q, 128), ("inline_rope_hd64", np.ascontiguousarray(q[:768]), 64)):
        assert rel_err(sampled(dev.rope(up(arr)[0], hd, base=10000.0), name), golden[name]) <= TOL32
    # scale / norm / clip: the library folds the scale and the clip factor into Adam; here the same factors are applied
    # with the scale operator so that the gradient itself can be compared
    layers, fin, emb = gi.grad_post_inputs()
    flat = torch.from_numpy(gi.grad_post_flat(layers, fin, emb)).cuda()
    nsq = dev.grad_norm_sq(flat, gi.GRAD_POST_GSC)
    assert abs(float(nsq[0]) - float(golden["inline_grad_norm_sq"])) <= TOL32 * float(golden["inline_grad_norm_sq"])
    cf = dev.clip_factor(nsq, 1.0)
    assert float(cf[0]) < 1.0
    got = dev.scale(dev.scale(flat, gi.GRAD_POST_GSC), float(cf[0]))
    assert rel_err(sampled(got, "inline_grad_flat"), golden["inline_grad_flat"]) <= TOL32


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [(1, 768, 256), (2, 1024, 128), (3, 7, 5), (2, 100, 37)])
def test_residual_rmsnorm_fused(dev, oracle, shape, dt):
    B, Cn, S = shape
    r = gi.rng(31)
    x, f = gi.normal(r, shape), gi.normal(r, shape)
    w = gi.normal(r, (Cn,), 0.02, 1.0)
    alpha = float(np.float32((2.0 * 28) ** -0.5))
    (xd, xr), (fd, fr) = up(x, dt), up(f, dt)
    x2, x2n = dev.residual_rmsnorm(xd, fd, up(w)[0], alpha, 1e-5)
    assert close(down(x2), oracle.residual(xr, fr, alpha), dt)
    # the norm is taken over the stored (rounded) x2, which is what the backward pass will read
    assert close(down(x2n), oracle.rmsnorm(down(x2), w, 1e-5), dt)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,heads,hd,S,base,pos0", [(1, 16, 128, 256, 1e4, 0), (2, 8, 128, 64, 1e6, 0), (1, 12, 64, 256, 1e4, 0),
                                                     (2, 3, 8, 37, 1e6, 11), (1, 2, 2, 1, 1e4, 0), (1, 4, 128, 2048, 1e6, 0)])
def test_rope_fwd_and_inverse(dev, oracle, B, heads, hd, S, base, pos0, dt):
    x = gi.normal(gi.rng(41), (B, heads * hd, S))
    xd, xr = up(x, dt)
    for inverse in (False, True):
        got = down(dev.rope(xd, hd, base=base, pos0=pos0, inverse=inverse))
        assert close(got, oracle.rope(xr, hd, base=base, pos0=pos0, inverse=inverse), dt)
    # in place
    y = xd.clone()
    dev.rope(y, hd, base=base, pos0=pos0, out=y)
    assert close(down(y), oracle.rope(xr, hd, base=base, pos0=pos0), dt)


def test_rope_bwd_golden_on_gpu(dev, golden):
    """training_dynamic/cpu_ops.h:168 on the committed reference outputs."""
    for name, (dim, hd) in (("hd64", (768, 64)), ("hd128", (2048, 128))):
        d = gi.normal(gi.rng(88), (dim, 256))
        got = down(dev.rope(up(d)[0], hd, base=10000.0, inverse=True))
        s = int(golden[f"ropebwd_{name}_stride"])
        assert rel_err(got.reshape(-1)[::s], golden[f"ropebwd_{name}"]) <= TOL32


QK_CASES = [(1, 16, 128, 256), (2, 8, 128, 64), (1, 12, 64, 128), (2, 3, 8, 37), (1, 2, 32, 5), (3, 16, 128, 40)]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,heads,hd,S", QK_CASES)
def test_qknorm_and_fusions_fwd(dev, oracle, B, heads, hd, S, dt):
    r = gi.rng(51)
    x = gi.normal(r, (B, heads * hd, S))
    w = gi.normal(r, (hd,), 0.02, 1.0)
    xd, xr = up(x, dt)
    wd, _ = up(w)
    assert close(down(dev.qknorm(xd, wd, hd, 1e-6)), oracle.qknorm(xr, w, hd, 1e-6), dt)
    got = down(dev.qknorm_rope(xd, wd, hd, 1e-6, 1e6, 3))
    assert close(got, oracle.qknorm_rope(xr, w, hd, 1e-6, 1e6, 3), dt)


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,heads,hd,S", QK_CASES)
def test_qknorm_and_fusions_bwd(dev, oracle, B, heads, hd, S, dt, exact):
    torch = _torch()
    r = gi.rng(52)
    x = gi.normal(r, (B, heads * hd, S))
    dy = gi.normal(r, (B, heads * hd, S))
    w = gi.normal(r, (hd,), 0.02, 1.0)
    (xd, xr), (dyd, dyr) = up(x, dt), up(dy, dt)
    wd, _ = up(w)
    dwtol = TOL32 if dt == "f32" else 1e-4
    dw = torch.zeros(hd, device="cuda")
    dx = down(dev.qknorm_bwd(dyd, xd, wd, dw, hd, 1e-6, exact=exact))
    rdx, rdw = oracle.qknorm_bwd(dyr, xr, w, hd, eps=1e-6, exact=exact)
    assert close(dx, rdx, dt) and rel_err(down(dw), rdw) <= dwtol
    dw = torch.zeros(hd, device="cuda")
    dx = down(dev.rope_qknorm_bwd(dyd, xd, wd, dw, hd, 1e-6, 1e6, 3, exact=exact))
    rdx, rdw = oracle.rope_qknorm_bwd(dyr, xr, w, hd, eps=1e-6, base=1e6, pos0=3, exact=exact)
    assert close(dx, rdx, dt) and rel_err(down(dw), rdw) <= dwtol


# More (token tile, head) items than the persistent grid of the TMA kernels holds (296 blocks over 64-token
# tiles): 320 tiles = one full round and 24 left-over tiles shared out head by head, 608 tiles = two rounds and
# 16 left over, 1216 tiles of 8 heads, and a 64-wide head shape; S = 2048 with base 1e6 is the Qwen3 attention
# prep as configured (positions to 2047, where one ulp of a frequency already moves the angle by 1e-4).
QK_ROUNDS = [(10, 16, 128, 2048), (19, 8, 128, 2048), (5, 16, 128, 2048 + 64 + 8), (12, 12, 64, 2048), (38, 2, 128, 2048)]


@pytest.mark.parametrize("pipe", [0, 1])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,heads,hd,S", QK_ROUNDS)
def test_qk_kernels_over_several_rounds_fwd(dev, oracle, B, heads, hd, S, dt, pipe):
    from ane_b200 import lib
    lib.set_tuning("qk_fwd_pipe", pipe)                  # one block barrier per item, or two
    try:
        _qk_rounds_fwd(dev, oracle, B, heads, hd, S, dt)
    finally:
        lib.clear_tuning("qk_fwd_pipe")


def _qk_rounds_fwd(dev, oracle, B, heads, hd, S, dt):
    from ane_b200 import lib
    r = gi.rng(53)
    x = gi.normal(r, (B, heads * hd, S))
    w = gi.normal(r, (hd,), 0.02, 1.0)
    xd, xr = up(x, dt)
    wd, _ = up(w)
    lib.poll_status(reset=True)
    assert close(down(dev.qknorm(xd, wd, hd, 1e-6)), oracle.qknorm(xr, w, hd, 1e-6), dt)
    assert close(down(dev.qknorm_rope(xd, wd, hd, 1e-6, 1e6, 0)), oracle.qknorm_rope(xr, w, hd, 1e-6, 1e6, 0), dt)
    assert close(down(dev.rope(xd, hd, base=1e6)), oracle.rope(xr, hd, base=1e6), dt)
    assert lib.poll_status().wait_giveups == 0


# Q and K of one layer in one call: (B, heads_q, heads_k, hd, S) -- one block round and several, a ragged last round, both head
# widths, a shape the side-by-side form does not cover (hd 32: the two calls run one after the other)
QK_PAIRS = [(2, 4, 2, 128, 256), (10, 16, 8, 128, 2048), (5, 16, 8, 128, 2048 + 64 + 8), (7, 12, 4, 64, 2048), (3, 3, 1, 128, 520),
            (2, 4, 2, 32, 96)]


@pytest.mark.parametrize("pair", [1, 0])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("B,hq,hk,hd,S", QK_PAIRS)
def test_qk_pair_equals_the_two_calls_and_the_oracle(dev, oracle, B, hq, hk, hd, S, dt, pair):
    """ane_cuda_qknorm_rope_pair_dev / ane_cuda_rope_qknorm_bwd_pair_dev: outputs and dx carry the bits of the separate
    calls (and match the oracle), dw matches the oracle and is bit-stable from call to call; knob qk_pair = 0 makes the
    two calls one after the other."""
    torch = _torch()
    from ane_b200 import lib
    r = gi.rng(97)
    q, k = gi.normal(r, (B, hq * hd, S)), gi.normal(r, (B, hk * hd, S))
    dyq, dyk = gi.normal(r, (B, hq * hd, S)), gi.normal(r, (B, hk * hd, S))
    wq, wk = gi.normal(r, (hd,), 0.05, 1.0), gi.normal(r, (hd,), 0.05, 1.0)
    (qd, qr), (kd, kr), (dyqd, dyqr), (dykd, dykr) = up(q, dt), up(k, dt), up(dyq, dt), up(dyk, dt)
    wqd, wkd = up(wq)[0], up(wk)[0]
    lib.poll_status(reset=True)
    lib.set_tuning("qk_pair", pair)
    try:
        oq, ok = dev.qknorm_rope_pair(qd, kd, wqd, wkd, hd, 1e-6, 1e6, 0)
        dwq, dwk = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda")
        dq, dk = dev.rope_qknorm_bwd_pair(dyqd, dykd, qd, kd, wqd, wkd, dwq, dwk, hd, 1e-6, 1e6, 0)
        dwq2, dwk2 = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda")
        dq2, dk2 = dev.rope_qknorm_bwd_pair(dyqd, dykd, qd, kd, wqd, wkd, dwq2, dwk2, hd, 1e-6, 1e6, 0)
    finally:
        lib.clear_tuning("qk_pair")
    assert torch.equal(oq, dev.qknorm_rope(qd, wqd, hd, 1e-6, 1e6, 0)) and torch.equal(ok, dev.qknorm_rope(kd, wkd, hd, 1e-6, 1e6, 0))
    sq, sk = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda")
    assert torch.equal(dq, dev.rope_qknorm_bwd(dyqd, qd, wqd, sq, hd, 1e-6, 1e6, 0))
    assert torch.equal(dk, dev.rope_qknorm_bwd(dykd, kd, wkd, sk, hd, 1e-6, 1e6, 0))
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dwq, dwq2) and torch.equal(dwk, dwk2)
    assert close(down(oq), oracle.qknorm_rope(qr, wq, hd, 1e-6, 1e6, 0), dt) and close(down(ok), oracle.qknorm_rope(kr, wk, hd, 1e-6, 1e6, 0), dt)
    rdq, rdwq = oracle.rope_qknorm_bwd(dyqr, qr, wq, hd, eps=1e-6, base=1e6)
    rdk, rdwk = oracle.rope_qknorm_bwd(dykr, kr, wk, hd, eps=1e-6, base=1e6)
    assert close(down(dq), rdq, dt) and close(down(dk), rdk, dt)
    dwtol = TOL32 if dt == "f32" else 1e-4
    assert rel_err(down(dwq), rdwq) <= dwtol and rel_err(down(dwk), rdwk) <= dwtol
    assert rel_err(down(sq), rdwq) <= dwtol and rel_err(down(sk), rdwk) <= dwtol
    assert lib.poll_status().wait_giveups == 0


def test_qk_pair_in_a_replayed_graph(dev):
    """The pair forks to a stream of the library and joins again inside the call: captured into a graph, the replay gives
    the bits of the eager call."""
    torch = _torch()
    B, hq, hk, hd, S = 6, 16, 8, 128, 1024
    gen = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, hq * hd, S, device="cuda", generator=gen).bfloat16()
    k = torch.randn(B, hk * hd, S, device="cuda", generator=gen).bfloat16()
    dyq, dyk = torch.randn_like(q), torch.randn_like(k)
    wq = (1 + 0.1 * torch.randn(hd, device="cuda", generator=gen)).float()
    wk = (1 + 0.1 * torch.randn(hd, device="cuda", generator=gen)).float()
    oq, ok, dq, dk = torch.empty_like(q), torch.empty_like(k), torch.empty_like(q), torch.empty_like(k)
    dwq, dwk = torch.zeros(hd, device="cuda"), torch.zeros(hd, device="cuda")

    def run():
        dev.qknorm_rope_pair(q, k, wq, wk, hd, out_q=oq, out_k=ok)
        dev.rope_qknorm_bwd_pair(dyq, dyk, oq, ok, wq, wk, dwq, dwk, hd, out_q=dq, out_k=dk)

    run()
    torch.cuda.synchronize()
    want = [t.clone() for t in (oq, ok, dq, dk, dwq, dwk)]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(2):
        for t in (oq, ok, dq, dk, dwq, dwk):
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip((oq, ok, dq, dk, dwq, dwk), want):
            assert torch.equal(a, b)


@pytest.mark.parametrize("pipe", [0, 1])
@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,heads,hd,S", QK_ROUNDS)
def test_qk_kernels_over_several_rounds_bwd(dev, oracle, B, heads, hd, S, dt, exact, pipe):
    torch = _torch()
    from ane_b200 import lib
    lib.set_tuning("qk_bwd_pipe", pipe)                  # one block barrier per item, or two
    try:
        _qk_rounds_bwd(dev, oracle, B, heads, hd, S, dt, exact)
    finally:
        lib.clear_tuning("qk_bwd_pipe")


def _qk_rounds_bwd(dev, oracle, B, heads, hd, S, dt, exact):
    torch = _torch()
    from ane_b200 import lib
    r = gi.rng(54)
    x = gi.normal(r, (B, heads * hd, S))
    dy = gi.normal(r, (B, heads * hd, S))
    w = gi.normal(r, (hd,), 0.02, 1.0)
    (xd, xr), (dyd, dyr) = up(x, dt), up(dy, dt)
    wd, _ = up(w)
    dwtol = TOL32 if dt == "f32" else 1e-4
    lib.poll_status(reset=True)
    dw = torch.zeros(hd, device="cuda")
    dx = down(dev.qknorm_bwd(dyd, xd, wd, dw, hd, 1e-6, exact=exact))
    rdx, rdw = oracle.qknorm_bwd(dyr, xr, w, hd, eps=1e-6, exact=exact)
    assert close(dx, rdx, dt) and rel_err(down(dw), rdw) <= dwtol
    outs = []
    for _ in range(2):
        dw = torch.zeros(hd, device="cuda")
        outs.append((dev.rope_qknorm_bwd(dyd, xd, wd, dw, hd, 1e-6, 1e6, 0, exact=exact), dw))
    rdx, rdw = oracle.rope_qknorm_bwd(dyr, xr, w, hd, eps=1e-6, base=1e6, pos0=0, exact=exact)
    assert close(down(outs[0][0]), rdx, dt) and rel_err(down(outs[0][1]), rdw) <= dwtol
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])     # bit-stable run to run
    assert lib.poll_status().wait_giveups == 0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("idt", ["int32", "uint16"])
@pytest.mark.parametrize("B,D,S,V", [(1, 768, 256, 32000), (2, 1024, 64, 151936), (3, 5, 7, 11), (1, 100, 33, 70000)])
def test_embed_lookup_bit_exact(dev, oracle, B, D, S, V, idt, dt):
    torch = _torch()
    from ane_b200 import lib
    if idt == "uint16" and V > 65536:
        pytest.skip("uint16 ids cannot address this vocabulary")
    r = gi.rng(61)
    table = gi.normal(r, (V, D), 0.02)
    tok = r.integers(0, V, size=(B, S)).astype(np.int32)
    tabd, tabr = up(table, dt)
    tokd = torch.from_numpy(tok.astype(np.uint16 if idt == "uint16" else np.int32)).cuda()
    lib.poll_status(reset=True)
    got = down(dev.embed_lookup(tabd, tokd))
    want, _ = oracle.embed_lookup(tabr, tok)
    assert np.array_equal(got, want)
    assert lib.poll_status().oor_ids == 0


def test_embed_lookup_out_of_range(dev, oracle):
    torch = _torch()
    from ane_b200 import lib
    table = gi.normal(gi.rng(62), (100, 40))
    tok = np.array([[3, 100, -1, 99, 5]], np.int32)
    tabd, _ = up(table)
    lib.poll_status(reset=True)
    init = torch.full((1, 40, 5), 7.0, device="cuda")
    got = down(dev.embed_lookup(tabd, torch.from_numpy(tok).cuda(), out=init.clone()))
    want, oor = oracle.embed_lookup(table, tok, x_init=np.full((1, 40, 5), 7.0, np.float32))
    assert np.array_equal(got, want)                       # stale columns kept (stories_cpu_ops.h:115)
    assert lib.poll_status().oor_ids == oor == 2
    got = down(dev.embed_lookup(tabd, torch.from_numpy(tok).cuda(), out=init.clone(), zero_oor=True))
    assert np.all(got[0, :, 1] == 0) and np.all(got[0, :, 2] == 0)
    lib.poll_status(reset=True)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,D,S,V,dup", [(1, 768, 256, 32000, 10), (2, 1024, 64, 151936, 0), (3, 5, 7, 11, 0),
                                         (2, 96, 130, 50, 0), (1, 64, 300, 1000, 300), (2, 256, 512, 5000, 100), (3, 1024, 256, 400, 40),
                                         (2, 1536, 64, 30, 0)])
def test_embed_backward_bit_exact_and_deterministic(dev, oracle, B, D, S, V, dup, dt):
    """fp32 additions happen in the reference's order (increasing (b, t) per row), so the result
    equals the sequential CPU sum bit for bit.  The cases cover every way a run's positions get ordered: runs of
    2-32 positions (sorted in registers), up to 256 (ranked by counting), beyond (a walk over the token array)."""
    torch = _torch()
    r = gi.rng(63)
    tok = r.integers(0, V, size=(B, S)).astype(np.int32)
    if dup:
        tok[0, :dup] = tok[0, 0]
    dx = gi.normal(r, (B, D, S))
    dE0 = gi.normal(r, (V, D), 0.01)
    dxd, dxr = up(dx, dt)
    tokd = torch.from_numpy(tok).cuda()
    want, _ = oracle.embed_backward(dE0, dxr, tok)
    outs = []
    for _ in range(2):
        dE = torch.from_numpy(dE0).cuda()
        dev.embed_backward(dE, dxd, tokd)
        outs.append(dE)
    assert torch.equal(outs[0], outs[1])
    assert np.array_equal(down(outs[0]), want)


@pytest.mark.parametrize("sorted_path", [0, 1])
def test_embed_backward_skewed_ids(dev, oracle, sorted_path):
    """Ids drawn from a heavy-tailed distribution (a few ids take thousands of positions, most occur once or never), as
    token streams of real text are: still the sequential sum, bit for bit, through both forms of the scatter-add."""
    torch = _torch()
    from ane_b200 import lib
    r = gi.rng(65)
    B, D, S, V = 8, 512, 1024, 20000
    tok = np.minimum((r.pareto(0.9, size=(B, S)) * 3).astype(np.int64), V - 1).astype(np.int32)
    assert np.bincount(tok.reshape(-1)).max() > 300
    dx = gi.normal(r, (B, D, S))
    dE0 = gi.normal(r, (V, D), 0.01)
    dxd, dxr = up(dx, "bf16")
    want, _ = oracle.embed_backward(dE0, dxr, tok)
    lib.set_tuning("embed_sort", sorted_path)
    try:
        dE = torch.from_numpy(dE0).cuda()
        dev.embed_backward(dE, dxd, torch.from_numpy(tok).cuda())
        assert np.array_equal(down(dE), want)
    finally:
        lib.clear_tuning("embed_sort")


def test_embed_backward_skips_out_of_range(dev, oracle):
    torch = _torch()
    from ane_b200 import lib
    tok = np.array([[1, 50, 2, -3, 1]], np.int32)
    dx = gi.normal(gi.rng(64), (1, 16, 5))
    dE = torch.zeros(50, 16, device="cuda")
    lib.poll_status(reset=True)
    dev.embed_backward(dE, up(dx)[0], torch.from_numpy(tok).cuda())
    want, oor = oracle.embed_backward(np.zeros((50, 16), np.float32), dx, tok)
    assert np.array_equal(down(dE), want)
    assert lib.poll_status().oor_ids == oor == 2
    lib.poll_status(reset=True)


@pytest.mark.parametrize("idt", ["int32", "uint16"])
@pytest.mark.parametrize("B,V,S,gs", [(1, 32000, 256, 1.0), (2, 1000, 37, 256.0), (1, 151936, 64, 1.0), (3, 17, 4, 1.0), (1, 9200, 256, 1.0),
                                       (5, 9200, 256, 1.0), (2, 32000, 520, 256.0)])   # the last two take the whole-grid wave kernel
def test_cross_entropy(dev, oracle, B, V, S, gs, idt):
    torch = _torch()
    if idt == "uint16" and V > 65536:
        pytest.skip("uint16 ids cannot address this vocabulary")
    r = gi.rng(71)
    logits = gi.normal(r, (B, V, S))
    tg = r.integers(0, V, size=(B, S)).astype(np.int32)
    ld, _ = up(logits)
    tgd = torch.from_numpy(tg.astype(np.uint16 if idt == "uint16" else np.int32)).cuda()
    loss, dl = dev.cross_entropy(ld, tgd, grad_scale=gs)
    rloss, rdl, _ = oracle.cross_entropy(logits, tg, grad_scale=gs)
    assert rel_err(down(loss), rloss) <= TOL32
    assert rel_err(down(dl), rdl) <= TOL32
    # in place
    loss2, dl2 = dev.cross_entropy(ld, tgd, grad_scale=gs, dlogits=ld)
    assert torch.equal(dl2, dl) and torch.equal(loss2, loss)


def test_cross_entropy_reference_fixture_and_oor(dev, oracle, golden):
    torch = _torch()
    from ane_b200 import lib
    logits = gi.fixture_softmax_logits()                 # test_classifier.m:132-134
    tg = golden["ce_fixture_targets"].astype(np.int32)
    loss, dl = dev.cross_entropy(up(logits[None])[0], torch.from_numpy(tg[None]).cuda())
    assert abs(float(loss[0]) - float(golden["ce_fixture_stories_loss"])) <= TOL32 * float(golden["ce_fixture_stories_loss"])
    s = int(golden["ce_fixture_stories_dlogits_stride"])
    assert rel_err(down(dl).reshape(-1)[::s], golden["ce_fixture_stories_dlogits"]) <= TOL32
    # out-of-range target: plain softmax stays in the column (stories_cpu_ops.h:94-103)
    lg = gi.cfg4_logits(B=1, vocab=500, seq=8)
    tg = np.array([[1, 2, 600, 3, 4, 5, -6, 7]], np.int32)
    lib.poll_status(reset=True)
    loss, dl = dev.cross_entropy(up(lg)[0], torch.from_numpy(tg).cuda())
    rloss, rdl, oor = oracle.cross_entropy(lg, tg)
    assert rel_err(down(loss), rloss) <= TOL32 and rel_err(down(dl), rdl) <= TOL32
    assert lib.poll_status().oor_ids == oor == 2
    lib.poll_status(reset=True)


@pytest.mark.parametrize("dynamic,wd,b2", [(False, 0.0, 0.999), (True, 0.1, 0.95), (True, 0.0, 0.95)])
@pytest.mark.parametrize("n", [1 << 16, 1000003, 5])
def test_adam(dev, oracle, n, dynamic, wd, b2):
    torch = _torch()
    w, g, m, v = gi.adam_inputs(n=n)
    wd_, gd, md, vd = (torch.from_numpy(a.copy()).cuda() for a in (w, g, m, v))
    for t in (1, 2, 3):
        dev.adam(wd_, gd, md, vd, t, 3e-4, 0.9, b2, 1e-8, wd=wd, dynamic=dynamic)
        oracle.adam(w, g, m, v, t, 3e-4, 0.9, b2, 1e-8, wd=wd, variant=int(dynamic))
    for got, want in ((wd_, w), (md, m), (vd, v)):
        assert rel_err(down(got), want) <= TOL32


def test_adam_golden_and_grad_postprocessing(dev, oracle, golden):
    """Reference outputs (both Adam variants) and the scale / norm / clip chain of train.m:750-825."""
    torch = _torch()
    for name, wd, b2, dyn in (("stories", 0.0, 0.999, False), ("dynamic", 0.1, 0.95, True)):
        w, g, m, v = (torch.from_numpy(a).cuda() for a in gi.adam_inputs())
        for t in (1, 2, 3):
            dev.adam(w, g, m, v, t, 3e-4, 0.9, b2, 1e-8, wd=wd, dynamic=dyn)
        for arr, key in ((w, "w"), (m, "m"), (v, "v")):
            s = int(golden[f"adam_{name}_{key}_stride"])
            assert rel_err(down(arr).reshape(-1)[::s], golden[f"adam_{name}_{key}"]) <= TOL32
    n = 3000001
    w, g, m, v = gi.adam_inputs(n=n)
    g *= 300.0
    gsc = 1.0 / (10 * 256.0)
    gd = torch.from_numpy(g).cuda()
    nsq = dev.grad_norm_sq(gd, gsc)
    want = oracle.grad_norm_sq(g, gsc)
    assert abs(float(nsq[0]) - want) <= 1e-5 * want
    nsq2 = dev.grad_norm_sq(gd, gsc)
    assert torch.equal(nsq, nsq2)                              # fixed summation order
    clip = dev.clip_factor(nsq, 1.0)
    cf = oracle.clip_factor(np.float32(float(nsq[0])), 1.0)
    assert abs(float(clip[0]) - cf) <= 1e-6 * cf and cf < 1.0
    wd_, md, vd = (torch.from_numpy(a.copy()).cuda() for a in (w, m, v))
    dev.adam(wd_, gd, md, vd, 1, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, gscale=gsc, clip=clip)
    oracle.adam(w, g, m, v, 1, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, variant=1, gscale=gsc, clip=float(clip[0]))
    assert rel_err(down(wd_), w) <= TOL32 and rel_err(down(md), m) <= TOL32 and rel_err(down(vd), v) <= TOL32


# ------------------------------------------------------------------ host-pointer drop-ins
def test_host_dropins_match_oracle(dev, oracle):
    from ane_b200 import cpu_ops as ops
    x, w, dy = gi.cfg1()
    d, S = 768, 256
    out = np.empty((d, S), np.float32)
    ops.rmsnorm(out, x[0], w, d, S)
    assert rel_err(out, oracle.rmsnorm(x[0], w)) <= TOL32
    dx = np.zeros((d, S), np.float32)
    dw = np.full(d, 0.5, np.float32)
    ops.rmsnorm_bwd(dx, dw, dy[0], x[0], w, d, S)
    rdx, rdw = oracle.rmsnorm_bwd(dy[0], x[0], w, dw=np.full(d, 0.5, np.float32))
    assert rel_err(dx, rdx) <= TOL32 and rel_err(dw, rdw) <= TOL32

    wv, g, m, v = gi.adam_inputs(n=24 * 1024)
    st = ops.AdamState(wv.size)
    st.m[:], st.v[:] = m, v
    w2 = wv.copy()
    ops.adam_update(w2, g, st, 2, 3e-4, 0.9, 0.999, 1e-8)
    oracle.adam(wv, g, m, v, 2, 3e-4, 0.9, 0.999, 1e-8, variant=0)
    assert rel_err(w2, wv) <= TOL32 and rel_err(st.m, m) <= TOL32 and rel_err(st.v, v) <= TOL32
    ops.adam_update(w2, g, st, 3, 3e-4, 0.9, 0.95, 1e-8, wd=0.1)
    oracle.adam(wv, g, m, v, 3, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, variant=1)
    assert rel_err(w2, wv) <= TOL32

    V = 9200
    logits = gi.cfg4_logits(B=1, vocab=V, seq=S)[0]
    tg = gi.rng(2).integers(0, V, size=S).astype(np.uint16)
    dl = np.empty_like(logits)
    loss = ops.cross_entropy_loss(dl, logits, tg, V, S)
    rl, rdl, _ = oracle.cross_entropy(logits, tg.astype(np.int32))
    assert abs(loss - rl[0]) <= TOL32 * rl[0] and rel_err(dl, rdl) <= TOL32

    r = gi.rng(3)
    table = gi.normal(r, (32000, d), 0.02)
    tok = r.integers(0, 32000, size=S).astype(np.uint16)
    tok[5:9] = tok[4]
    xg = np.zeros((d, S), np.float32)
    ops.embed_lookup(xg, table, tok, d, S)
    assert np.array_equal(xg, oracle.embed_lookup(table, tok.astype(np.int32)[None])[0][0])
    dE = np.zeros((32000, d), np.float32)
    ops.embed_backward(dE, dy[0], tok, d, S)
    assert np.array_equal(dE, oracle.embed_backward(np.zeros((32000, d), np.float32), dy, tok.astype(np.int32)[None])[0])

    dq = gi.normal(r, (2048, S))
    want = oracle.rope(dq, 128, base=10000.0, inverse=True)
    ops.rope_backward_inplace(dq, S, 2048, 128)
    assert rel_err(dq, want) <= TOL32

    h1, h3, dd, xx, ff = (a[0] for a in gi.cfg2())
    o = np.empty_like(h1)
    ops.swiglu(o, h1, h3)
    assert rel_err(o, oracle.swiglu(h1, h3)) <= TOL32
    g1, g3 = np.empty_like(h1), np.empty_like(h1)
    ops.swiglu_bwd(g1, g3, h1, h3, dd)
    r1, r3 = oracle.swiglu_bwd(h1, h3, dd)
    assert rel_err(g1, r1) <= TOL32 and rel_err(g3, r3) <= TOL32
    o = np.empty_like(xx)
    ops.residual(o, xx, ff, 0.2041241452)
    assert np.array_equal(o, oracle.residual(xx, ff, np.float32(0.2041241452)))


@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_host_batched_forms(dev, oracle, dt, pinned):
    """The batched host-buffer entry points (several pipeline chunks, odd batch) give the same
    results as the device-resident operators they wrap."""
    torch = _torch()
    from ane_b200 import host_ops as hop
    tdt = getattr(torch, DT[dt])
    B, Cn, S, H, hd = 5, 1024, 2048, 3072, 128          # 4 or 8 MiB per sequence and tensor -> multi-chunk
    g = torch.Generator().manual_seed(3)

    def mk(*shape, dtype=tdt):
        t = torch.randn(*shape, generator=g).to(dtype)
        return t.pin_memory() if pinned else t

    def out_like(t):
        o = torch.empty_like(t)
        return o.pin_memory() if pinned else o

    x, f, dy, add = mk(B, Cn, S), mk(B, Cn, S), mk(B, Cn, S), mk(B, Cn, S)
    w = (1 + 0.02 * torch.randn(Cn, generator=g)).float()
    wd = w.cuda()
    o = out_like(x)
    hop.rmsnorm(o, x, w)
    assert torch.equal(o, dev.rmsnorm(x.cuda(), wd).cpu())
    x2, x2n = out_like(x), out_like(x)
    hop.residual_rmsnorm(x2, x2n, x, f, w, 0.25)
    d2, d2n = dev.residual_rmsnorm(x.cuda(), f.cuda(), wd, 0.25)
    assert torch.equal(x2, d2.cpu()) and torch.equal(x2n, d2n.cpu())
    dx, dw = out_like(x), torch.full((Cn,), 0.5)
    hop.rmsnorm_bwd(dx, dw, dy, x, w, add=add)
    ddw = torch.full((Cn,), 0.5, device="cuda")
    ddx = dev.rmsnorm_bwd(dy.cuda(), x.cuda(), wd, ddw, add=add.cuda())
    assert torch.equal(dx, ddx.cpu())
    assert rel_err(dw.numpy(), ddw.cpu().numpy()) <= 1e-5     # chunked accumulation order differs
    h1, h3, ds = mk(B, H, S), mk(B, H, S), mk(B, H, S)
    o = out_like(h1)
    hop.swiglu(o, h1, h3)
    assert torch.equal(o, dev.swiglu(h1.cuda(), h3.cuda()).cpu())
    g1, g3 = out_like(h1), out_like(h1)
    hop.swiglu_bwd(g1, g3, h1, h3, ds)
    e1, e3 = dev.swiglu_bwd(h1.cuda(), h3.cuda(), ds.cuda())
    assert torch.equal(g1, e1.cpu()) and torch.equal(g3, e3.cpu())
    o = out_like(x)
    hop.residual(o, x, f, 0.25)
    assert torch.equal(o, dev.residual(x.cuda(), f.cuda(), 0.25).cpu())
    q, dq = mk(B, 16 * hd, S), mk(B, 16 * hd, S)
    wq = (1 + 0.02 * torch.randn(hd, generator=g)).float()
    o = out_like(q)
    hop.qknorm_rope(o, q, wq, hd)
    assert torch.equal(o, dev.qknorm_rope(q.cuda(), wq.cuda(), hd).cpu())
    dxq, dwq = out_like(q), torch.zeros(hd)
    hop.rope_qknorm_bwd(dxq, dwq, dq, q, wq, hd)
    ddwq = torch.zeros(hd, device="cuda")
    ddxq = dev.rope_qknorm_bwd(dq.cuda(), q.cuda(), wq.cuda(), ddwq, hd)
    assert torch.equal(dxq, ddxq.cpu()) and rel_err(dwq.numpy(), ddwq.cpu().numpy()) <= 1e-5
    o = out_like(q)
    hop.rope(o, q, hd, base=1e6, inverse=True)
    assert torch.equal(o, dev.rope(q.cuda(), hd, base=1e6, inverse=True).cpu())


def test_buffers_and_errors(dev):
    from ane_b200 import lib
    L = lib.load()
    assert L.ane_cuda_version() == 100 and L.ane_cuda_device_count() >= 1
    buf = L.ane_cuda_alloc(1024)
    assert buf and L.ane_cuda_bufsize(buf) == 1024 and L.ane_cuda_devptr(buf)
    src = np.arange(256, dtype=np.float32)
    dst = np.zeros_like(src)
    assert L.ane_cuda_write(buf, 0, src.ctypes.data, 1024) == 0
    assert L.ane_cuda_read(buf, 0, dst.ctypes.data, 1024) == 0 and np.array_equal(src, dst)
    assert L.ane_cuda_write(buf, 512, src.ctypes.data, 1024) == lib.ERR_INVALID      # past the end
    assert b"outside buffer" in L.ane_cuda_last_error()
    L.ane_cuda_free(buf)
    p = L.ane_cuda_host_alloc(4096)
    assert p
    L.ane_cuda_host_free(p)
    # argument errors come back as codes, nothing is launched
    assert L.ane_cuda_rmsnorm_dev(None, lib.F32, 1, 0, 8, 1, 1, 1, C.c_float(1e-5)) == lib.ERR_INVALID
    assert L.ane_cuda_rmsnorm_dev(None, 7, 1, 8, 8, 1, 1, 1, C.c_float(1e-5)) == lib.ERR_INVALID
    assert L.ane_cuda_rmsnorm_dev(None, lib.F32, 1, 8, 8, None, None, None, C.c_float(1e-5)) == lib.ERR_INVALID
    assert L.ane_cuda_rope_dev(None, lib.F32, 1, 12, 8, 5, 1, 1, C.c_float(1e4), 0, 0) == lib.ERR_INVALID   # C % hd != 0
    assert L.ane_cuda_adam_dev(None, 8, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 1, None, 0) == lib.ERR_INVALID          # t = 0
    before = lib.launch_count()
    assert L.ane_cuda_init(0) == 0                                                      # idempotent
    assert lib.launch_count() == before


def test_another_host_thread_may_take_over_and_errors_stay_with_their_thread(dev, oracle):
    """The header's threading contract: one host thread at a time, any thread.  A worker thread that runs while the main
    thread waits gets the same bits as the main thread, and the text of an error made on the worker is the worker's:
    the main thread's last error is not overwritten (training/training_dynamic/train.m:727-749 -- the reference's
    operators are called from one thread at a time too)."""
    import threading
    from ane_b200 import lib
    L = lib.load()
    x = gi.normal(gi.rng(71), (3, 96, 40))
    w = (1.0 + 0.02 * gi.normal(gi.rng(72), (96,))).astype(np.float32)
    xt, _ = up(x)
    wt, _ = up(w)
    here = down(dev.rmsnorm(xt, wt))
    assert L.ane_cuda_rmsnorm_dev(None, 7, 1, 8, 8, 1, 1, 1, C.c_float(1e-5)) == lib.ERR_INVALID
    mine = L.ane_cuda_last_error()
    box = {}

    def worker():
        box["out"] = down(dev.rmsnorm(xt, wt))
        box["rc"] = L.ane_cuda_rope_dev(None, lib.F32, 1, 12, 8, 5, 1, 1, C.c_float(1e4), 0, 0)
        box["err"] = L.ane_cuda_last_error()

    th = threading.Thread(target=worker)
    th.start()
    th.join()
    assert np.array_equal(box["out"], here)
    assert box["rc"] == lib.ERR_INVALID and box["err"] and box["err"] != mine
    assert L.ane_cuda_last_error() == mine
    ref = np.stack([oracle.rmsnorm(x[b], w) for b in range(x.shape[0])])
    assert rel_err(here, ref) <= TOL32


# ------------------------------------------------------------------ benchmark sizes: size-independent properties
def test_full_size_properties(dev):
    """Qwen3 shapes at S = 2048 in bf16: RoPE forward then inverse returns the input (to bf16
    rounding), the gather is a permutation of table rows (checksum), dlogits columns sum to zero,
    and the fused kernels agree with the unfused sequence of operators."""
    torch = _torch()
    torch.manual_seed(0)
    B, S, hd = 4, 2048, 128
    q = torch.randn(B, 16 * hd, S, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.02 * torch.randn(hd, device="cuda")).float()
    y = dev.rope(q, hd, base=1e6)
    z = dev.rope(y, hd, base=1e6, inverse=True)
    assert float((z.float() - q.float()).abs().max()) <= 2 * 2 ** -8 * float(q.float().abs().max())
    fused = dev.qknorm_rope(q, w, hd)
    unfused = dev.rope(dev.qknorm(q, w, hd), hd, base=1e6)
    assert float((fused.float() - unfused.float()).abs().max()) <= 2 ** -7 * float(unfused.float().abs().max())

    V, D = 151936, 1024
    table = (0.02 * torch.randn(V, D, device="cuda")).to(torch.bfloat16)
    tok = torch.randint(0, V, (B, S), device="cuda", dtype=torch.int32)
    x = dev.embed_lookup(table, tok)
    assert torch.equal(x, table[tok.long()].permute(0, 2, 1).contiguous())

    dE = torch.zeros(V, D, device="cuda")
    dev.embed_backward(dE, x, tok)
    ref = torch.zeros(V, D, device="cuda", dtype=torch.float64)
    ref.index_add_(0, tok.long().reshape(-1), x.permute(0, 2, 1).reshape(-1, D).double())
    assert float((dE.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())

    Vs = 151936
    logits = torch.randn(1, Vs, 256, device="cuda")
    tg = torch.randint(0, Vs, (1, 256), device="cuda", dtype=torch.int32)
    loss, dl = dev.cross_entropy(logits, tg)
    assert float(dl.double().sum(dim=1).abs().max()) <= 1e-6          # sum_v (p - onehot) = 0 per token
    assert abs(float(loss[0]) - (np.log(Vs) + 0.5)) < 0.2              # E[loss] = log V + sigma^2/2 for N(0,1) logits


def test_layer_chain_matches_oracle_and_graph_replay(dev, oracle):
    """The whole operator chain of a micro-batch (ane_b200.layer_chain, the order of
    training_dynamic/train.m:405-728) on a tiny fp32 model: every product of the chain equals the
    same sequence of oracle operators, and replaying the captured CUDA graph gives the eager result
    bit for bit."""
    torch = _torch()
    from ane_b200.layer_chain import ChainConfig, FlatParams, LayerChain
    cfg = ChainConfig(layers=2, dim=64, hidden=96, heads=2, kv_heads=1, head_dim=64, seq=32, vocab=50,
                      dtype=torch.float32, alpha=0.5, rope_base=1e4)
    p = FlatParams(cfg, "cuda")
    p.init_random(seed=3)
    p.zero_produced_grads()
    ch = LayerChain(cfg, 2, p, "cuda", rotate=2, seed=5)
    ch.forward()
    ch.backward()
    torch.cuda.synchronize()

    def n(t):
        return t.detach().float().cpu().numpy().copy()

    # --- oracle replay of the same chain
    tok = n(ch.tokens).astype(np.int32)
    x, _ = oracle.embed_lookup(n(ch.table), tok)
    xs, x2s = [x], []
    for L in range(cfg.layers):
        assert rel_err(n(ch.layer_in[L]), xs[L]) <= TOL32
        x2 = oracle.residual(xs[L], n(ch.o_out[L]), cfg.alpha)
        x2s.append(x2)
        assert rel_err(n(ch.x2[L]), x2) <= TOL32
        xs.append(oracle.residual(x2, n(ch.ffn_out[L]), cfg.alpha))
    assert rel_err(n(ch.x_final), oracle.rmsnorm(xs[-1], n(p.norm_w("final")), cfg.eps)) <= TOL32
    r = (cfg.layers - 1) % ch.R
    assert rel_err(n(ch.q_r[r]), oracle.qknorm_rope(n(ch.q[cfg.layers - 1]), n(p.norm_w("q", cfg.layers - 1)), 64, cfg.qk_eps, cfg.rope_base)) <= TOL32
    assert rel_err(n(ch.gate[r]), oracle.swiglu(n(ch.h1[cfg.layers - 1]), n(ch.h3[cfg.layers - 1]))) <= TOL32
    dy, gfin = oracle.rmsnorm_bwd(n(ch.dy_cls), xs[-1], n(p.norm_w("final")), eps=cfg.eps)
    assert rel_err(n(p.norm_w("final", grad=True)), gfin) <= TOL32
    for L in range(cfg.layers - 1, -1, -1):
        r = L % ch.R
        d2, gffn = oracle.rmsnorm_bwd(n(ch.dx_ffn[r]), x2s[L], n(p.norm_w("ffn", L)), eps=cfg.eps)
        dx2 = oracle.add(d2, dy)
        d1, gatt = oracle.rmsnorm_bwd(n(ch.dx_attn[r]), xs[L], n(p.norm_w("att", L)), eps=cfg.eps)
        dy = oracle.add(d1, dx2)
        assert rel_err(n(p.norm_w("ffn", L, grad=True)), gffn) <= TOL32
        assert rel_err(n(p.norm_w("att", L, grad=True)), gatt) <= TOL32
        _, gq = oracle.rope_qknorm_bwd(n(ch.dq_in[r]), n(ch.q[L]), n(p.norm_w("q", L)), 64, eps=cfg.qk_eps, base=cfg.rope_base)
        assert rel_err(n(p.norm_w("q", L, grad=True)), gq) <= TOL32
    assert rel_err(n(ch.dy_out), dy) <= TOL32
    dE, _ = oracle.embed_backward(np.zeros((cfg.vocab, cfg.dim), np.float32), dy, tok)
    assert rel_err(n(p.embed(grad=True)), dE) <= TOL32

    # --- graph replay == eager
    eager = {k: n(v) for k, v in (("dy", ch.dy_out), ("xf", ch.x_final), ("g", p.g[p.n_matrix:p.n]))}
    p.zero_produced_grads()
    ch.capture()              # runs one eager pass, then records
    p.zero_produced_grads()
    ch.replay()
    torch.cuda.synchronize()
    assert np.array_equal(n(ch.dy_out), eager["dy"]) and np.array_equal(n(ch.x_final), eager["xf"])
    assert np.array_equal(n(p.g[p.n_matrix:p.n]), eager["g"])


@pytest.mark.gpu
def test_host_layer_chain_equals_device_chain(dev):
    """HostLayerChain.step() (contraction-side tensors in page-locked host memory, three streams) hands back
    bit for bit what the device-resident chain computes from the same inputs, over two consecutive steps
    (the second one reuses every buffer and event of the first)."""
    torch = _torch()
    from ane_b200.host_chain import HostLayerChain
    from ane_b200.layer_chain import ChainConfig, FlatParams, LayerChain
    cfg = ChainConfig(layers=5, dim=64, hidden=96, heads=2, kv_heads=1, head_dim=64, seq=32, vocab=50,
                      dtype=torch.bfloat16, alpha=0.5, rope_base=1e4)
    p = FlatParams(cfg, "cuda")
    p.init_random(seed=3)
    hc = HostLayerChain(cfg, 2, p, "cuda", rotate=2)
    for _ in range(2):
        p.zero_produced_grads()
        hc.step()
        hc.synchronize()
        torch.cuda.synchronize()
        g_host = p.g.clone()
        # the same inputs through a device-resident chain (every layer sees the same host bytes)
        p.zero_produced_grads()
        ref = LayerChain(cfg, 2, p, "cuda", rotate=2)
        ref.tokens.copy_(hc.h_tokens)
        ref.dy_cls.copy_(hc.h_dy_cls)
        for L in range(cfg.layers):
            for k, h in hc.h_in_f.items():
                getattr(ref, k)[L].copy_(h)
        ref.forward()
        torch.cuda.synchronize()
        r_last = (cfg.layers - 1) % ref.R
        for k, h in hc.h_out_f.items():                      # the shared host buffers hold the last layer's products
            assert torch.equal(h.cuda(), getattr(ref, k)[r_last]), k
        assert torch.equal(hc.h_x_final.cuda(), ref.x_final)
        for r in range(ref.R):
            for k, h in hc.h_in_b.items():
                getattr(ref, k)[r].copy_(h)
        ref.backward()
        torch.cuda.synchronize()
        for k, h in hc.h_out_b.items():                      # backward ends at layer 0
            assert torch.equal(h.cuda(), getattr(ref, k)[0]), k
        assert torch.equal(g_host, p.g)                      # norm-weight and embedding gradients
    assert hc.h2d_bytes_per_step == 2 * 32 * 2 * (5 * (128 + 64 + 64 + 192 + 64 + 96 + 64 + 128 + 64 + 64) + 64) + 2 * 32 * 4


def test_c_chain_object_equals_python_host_chain(dev):
    """ane_cuda_chain_step (the chain object a C caller uses, csrc/chain.cu) hands back the same bytes as
    HostLayerChain.step() from the same host buffers: every downloaded tensor and every accumulated gradient, over two
    consecutive steps; a null host table is an argument error."""
    torch = _torch()
    import ctypes as C
    from ane_b200 import lib
    from ane_b200.host_chain import CHostLayerChain, HostLayerChain
    from ane_b200.layer_chain import ChainConfig, FlatParams
    cfg = ChainConfig(layers=6, dim=64, hidden=96, heads=2, kv_heads=1, head_dim=64, seq=64, vocab=50,
                      dtype=torch.bfloat16, alpha=0.5, rope_base=1e4)
    p = FlatParams(cfg, "cuda")
    p.init_random(seed=3)
    hc = HostLayerChain(cfg, 3, p, "cuda", rotate=2)
    cc = CHostLayerChain(hc, p)
    outs = {**hc.h_out_f, **hc.h_out_b, "x_final": hc.h_x_final}
    assert cc.h2d_bytes_per_step == hc.h2d_bytes_per_step and cc.d2h_bytes_per_step == hc.d2h_bytes_per_step
    for _ in range(2):
        p.zero_produced_grads()
        hc.step()
        hc.synchronize()
        torch.cuda.synchronize()
        want = {k: v.clone() for k, v in outs.items()}
        want_g = p.g.clone()
        for v in outs.values():
            v.zero_()
        p.zero_produced_grads()
        torch.cuda.synchronize()
        cc.step()
        cc.synchronize()
        torch.cuda.synchronize()
        for k, v in outs.items():
            assert torch.equal(v, want[k]), k
        assert torch.equal(p.g, want_g)
    bad = type(cc.io).from_buffer_copy(cc.io)
    bad.gate = C.POINTER(C.c_void_p)()
    assert lib.load().ane_cuda_chain_step(cc.handle, C.byref(bad)) == lib.ERR_INVALID
    cc.close()


# Every operator picks one kernel by default; the others stay reachable through tuning knobs (library function
# ane_cuda_set_tuning).  Each alternate path must give the same results within the same tolerances.
ALT_KNOBS = [
    ("norm_fwd", 0), ("norm_fwd", 2), ("norm_fwd", 3), ("norm_fwd", 4), ("norm_fwd", 6),
    ("norm_bwd", 0), ("norm_bwd", 8), ("norm_bwd", 9), ("norm_bwd", 10), ("norm_bwd", 11), ("norm_bwd", 12),
    ("qk_fwd", 0), ("qk_fwd", 1), ("qk_fwd", 4), ("qk_bwd", 0), ("qk_bwd", 4), ("qk_fwd_pipe", 0), ("qk_bwd_pipe", 0), ("qk_bwd_pipe", 1),
    ("dep_launch", 31), ("swiglu_exact", 1), ("rope_lg", 8), ("rope_table", 0), ("embed_tiled", 0), ("embed_rows", 0), ("embed_sort", 1), ("xent_cluster", 1), ("xent_reverse", 0), ("xent_lg", 4), ("xent_lg", 8), ("xent_lg", 32), ("xent_split", 1), ("xent_split", 2), ("xent_split", 8),
]


@pytest.mark.parametrize("knob,value", ALT_KNOBS)
def test_alternate_kernels_match_the_oracle(dev, oracle, knob, value):
    torch = _torch()
    from ane_b200 import lib
    defaults = {"norm_fwd": None, "norm_bwd": None}
    lib.set_tuning(knob, value)
    try:
        dt = "bf16"
        if knob.startswith("norm") or knob == "dep_launch":
            B, Cn, S = 3, 1024, 128
            x, w, dy = gi.cfg1(seed=21, B=B, dim=Cn, seq=S)
            f = gi.normal(gi.rng(7), (B, Cn, S))
            xd, xr = up(x, dt)
            fd, fr = up(f, dt)
            dyd, dyr = up(dy, dt)
            wd, _ = up(w)
            assert close(down(dev.rmsnorm(xd, wd)), oracle.rmsnorm(xr, w), dt)
            x2, x2n = dev.residual_rmsnorm(xd, fd, wd, 0.25)
            rx2 = oracle.residual(xr, fr, 0.25)
            assert close(down(x2), rx2, dt)
            rx2_16 = down(up(rx2, dt)[0])                       # the norm reads the stored (rounded) sum
            assert close(down(x2n), oracle.rmsnorm(rx2_16, w), dt)
            dw = torch.zeros(Cn, device="cuda")
            dx = dev.rmsnorm_bwd(dyd, xd, wd, dw, add=fd)
            rdx, rdw = oracle.rmsnorm_bwd(dyr, xr, w)
            assert close(down(dx), oracle.add(rdx, fr), dt)
            assert rel_err(down(dw), rdw) <= 1e-4
        if knob.startswith("qk") or knob in ("rope_lg", "rope_table", "dep_launch"):
            B, heads, hd, S = 2, 4, 128, 256
            q = gi.normal(gi.rng(8), (B, heads * hd, S))
            dq = gi.normal(gi.rng(9), (B, heads * hd, S))
            wq = (1 + 0.1 * gi.normal(gi.rng(10), (hd,))).astype(np.float32)
            qd, qr = up(q, dt)
            dqd, dqr = up(dq, dt)
            wqd, _ = up(wq)
            assert close(down(dev.qknorm_rope(qd, wqd, hd, 1e-6, 1e6, 0)), oracle.qknorm_rope(qr, wq, hd, 1e-6, 1e6), dt)
            assert close(down(dev.rope(qd, hd, base=1e6)), oracle.rope(qr, hd, 1e6), dt)
            dwq = torch.zeros(hd, device="cuda")
            dx = dev.rope_qknorm_bwd(dqd, qd, wqd, dwq, hd, 1e-6, 1e6, 0)
            rdx, rdw = oracle.rope_qknorm_bwd(dqr, qr, wq, hd, eps=1e-6, base=1e6)
            assert close(down(dx), rdx, dt)
            assert rel_err(down(dwq), rdw) <= 1e-4
        if knob.startswith("swiglu"):
            arrs = [gi.normal(gi.rng(31 + i), (3 * 3072 * 64 + 5,)) for i in range(3)]
            for sdt in ("bf16", "f32"):
                (h1d, h1), (h3d, h3), (dd, d) = [up(a, sdt) for a in arrs]
                assert close(down(dev.swiglu(h1d, h3d)), oracle.swiglu(h1, h3), sdt)
                g1, g3 = dev.swiglu_bwd(h1d, h3d, dd)
                r1, r3 = oracle.swiglu_bwd(h1, h3, d)
                assert close(down(g1), r1, sdt) and close(down(g3), r3, sdt)
        if knob.startswith("embed"):
            V, D, B, S = 300, 256, 2, 64
            table = gi.normal(gi.rng(11), (V, D), 0.02)
            tok = gi.rng(12).integers(0, V, (B, S)).astype(np.int32)
            td, tr = up(table, dt)
            tokd = torch.from_numpy(tok).cuda()
            x = dev.embed_lookup(td, tokd)
            rx, _ = oracle.embed_lookup(tr, tok)
            assert np.array_equal(down(x), rx)                  # a copy: bit-exact
            dE = torch.zeros(V, D, device="cuda")
            dev.embed_backward(dE, x, tokd)
            rdE, _ = oracle.embed_backward(np.zeros((V, D), np.float32), rx, tok)
            assert np.array_equal(down(dE), rdE)                # same additions in the same order
        if knob.startswith("xent"):
            B, V, S = 2, 8192, 128
            logits = gi.normal(gi.rng(13), (B, V, S), 2.0)
            tg = gi.rng(14).integers(0, V, (B, S)).astype(np.int32)
            loss, dl = dev.cross_entropy(torch.from_numpy(logits).cuda(), torch.from_numpy(tg).cuda())
            rloss, rdl, _ = oracle.cross_entropy(logits, tg)
            assert rel_err(down(dl), rdl) <= TOL32
            assert np.allclose(down(loss), rloss, rtol=1e-5, atol=1e-6)
        assert lib.poll_status().wait_giveups == 0
    finally:
        lib.clear_tuning(knob)


class _DependentChain:
    """Operators that hand their results to each other in place, back to back on one stream: every launch reads what the
    launch before it wrote and overwrites what an earlier one read."""

    def __init__(self, torch, B=32, Cn=1024, S=2048, hd=128):
        self.torch, self.hd = torch, hd
        gen = torch.Generator(device="cuda").manual_seed(4242)
        self.x0 = torch.randn(B, Cn, S, device="cuda", generator=gen).bfloat16()
        self.f0 = torch.randn(B, Cn, S, device="cuda", generator=gen).bfloat16()
        self.w = (1.0 + 0.02 * torch.randn(Cn, device="cuda", generator=gen)).float()
        self.wq = (1.0 + 0.1 * torch.randn(hd, device="cuda", generator=gen)).float()
        self.x, self.f = self.x0.clone(), self.f0.clone()
        self.dw, self.dwq = torch.zeros(Cn, device="cuda"), torch.zeros(hd, device="cuda")
        self.x2, self.x2n, self.g, self.h, self.q, self.dq = (torch.empty_like(self.x0) for _ in range(6))

    def reset(self):
        self.x.copy_(self.x0)
        self.f.copy_(self.f0)
        self.dw.zero_()
        self.dwq.zero_()

    def run(self, dev, rounds):
        for _ in range(rounds):
            dev.residual_rmsnorm(self.x, self.f, self.w, 0.3, x2=self.x2, x2norm=self.x2n)
            dev.swiglu(self.x2n, self.x2, out=self.g)
            dev.qknorm_rope(self.g, self.wq, self.hd, 1e-6, 1e6, 0, out=self.q)
            dev.rope_qknorm_bwd(self.q, self.g, self.wq, self.dwq, self.hd, 1e-6, 1e6, 0, out=self.dq)
            dev.swiglu_bwd(self.x2n, self.x2, self.dq, dh1=self.h, dh3=self.f)   # f is overwritten: the next round's residual reads it
            dev.rmsnorm_bwd(self.h, self.x2, self.w, self.dw, add=self.q, out=self.x)   # x too
            dev.scale(self.x, 0.05, out=self.x)                                 # keeps the loop bounded

    def results(self):
        self.torch.cuda.synchronize()
        return [t.clone() for t in (self.x, self.f, self.x2, self.x2n, self.g, self.h, self.q, self.dq, self.dw, self.dwq)]


def test_dependent_launches_give_the_bits_of_plain_launches(dev):
    """Knob dep_launch starts the chain's kernels as programmatic dependent launches (the next kernel is placed while the
    running one drains, and stops before its first global access until that one is complete).  A kernel that touched global
    memory too early would read or overwrite data of the launch before it: the same in-place operator sequence must end with
    the same bits whether the launches are plain (default) or dependent (all kernel classes), eagerly and as a replayed graph."""
    torch = _torch()
    from ane_b200 import lib
    ch = _DependentChain(torch)
    ch.run(dev, 5)
    plain = ch.results()
    lib.set_tuning("dep_launch", 31)
    try:
        _dependent_launch_checks(dev, torch, lib, ch, plain)
    finally:
        lib.clear_tuning("dep_launch")


def _dependent_launch_checks(dev, torch, lib, ch, plain):
    assert all(bool(torch.isfinite(t.float()).all()) for t in plain)
    assert float(plain[0].float().abs().max()) > 0.0 and float(plain[8].abs().max()) > 0.0
    for _ in range(2):
        ch.reset()
        ch.run(dev, 5)
        for a, b in zip(ch.results(), plain):
            assert torch.equal(a, b)
    # the same launches as nodes of one graph (dependent edges between kernel nodes), replayed
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ch.run(dev, 5)
    for _ in range(2):
        ch.reset()
        graph.replay()
        for a, b in zip(ch.results(), plain):
            assert torch.equal(a, b)
    assert lib.poll_status().wait_giveups == 0


@pytest.mark.parametrize("nranks,n,lo", [(1, 1000, 0), (2, 4099, 8), (4, 1 << 16, 1 << 14), (8, 33, 3), (3, 70001, 4)])
def test_peer_memory_optimizer_kernels_with_emulated_ranks(dev, oracle, nranks, n, lo):
    """ane_cuda_p2p_reduce_dev / ane_cuda_p2p_adam_dev with the ranks' buffers all on this GPU: the reduce equals the
    rank-ordered fp32 sum, the update equals ane_cuda_adam_dev on the summed gradient bit for bit and reaches every
    rank's parameter buffer; elements outside the slice are untouched."""
    torch = _torch()
    total = lo + n + 5
    gen = torch.Generator(device="cuda").manual_seed(nranks * 1000 + n)
    gs = [torch.randn(total, device="cuda", generator=gen) * 0.01 for _ in range(nranks)]
    w0 = torch.randn(total, device="cuda", generator=gen) * 0.02
    ws = [w0.clone() for _ in range(nranks)]
    m = torch.randn(n, device="cuda", generator=gen) * 0.001
    v = (torch.randn(n, device="cuda", generator=gen) * 0.001).abs()
    gsl = torch.empty(n, device="cuda")
    nsq = dev.p2p_reduce([g.data_ptr() for g in gs], lo, n, gsl, gscale=0.5)
    want = gs[0][lo:lo + n].clone()
    for r in range(1, nranks):
        want = want + gs[r][lo:lo + n]                       # same order of fp32 additions
    assert torch.equal(gsl, want)
    ref_nsq = float(((want.double() * 0.5) ** 2).sum())
    assert abs(float(nsq.item()) - ref_nsq) <= 1e-5 * ref_nsq
    clip = torch.full((1,), 0.75, device="cuda")
    wr, mr, vr = w0[lo:lo + n].clone(), m.clone(), v.clone()
    dev.adam(wr, want, mr, vr, 3, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, gscale=0.5, clip=clip)
    dev.p2p_adam([w.data_ptr() for w in ws], nranks - 1, lo, n, gsl, m, v, 3, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, gscale=0.5, clip=clip)
    assert torch.equal(m, mr) and torch.equal(v, vr)
    for w in ws:
        assert torch.equal(w[lo:lo + n], wr)
        assert torch.equal(w[:lo], w0[:lo]) and torch.equal(w[lo + n:], w0[lo + n:])
