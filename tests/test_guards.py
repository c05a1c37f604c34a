"""Out-of-bounds writes: every output of every operator sits between two 256-byte guard zones filled with a
byte pattern, and the zones are checked after the call.  This stands in for a memory checker: a kernel
that stores one vector past the end of a ragged tile, or a bulk copy whose box overhangs its tensor, would
pass every value comparison and still corrupt a neighbour.

Shapes are chosen to end tiles everywhere: token counts that are not a multiple of any tile width (8, 16, 32,
64 tokens), channel counts that do not divide by the cluster sizes, vocabularies that do not divide by the
stripe splits, element counts one off a vector, plus the aligned shapes the vector and bulk-copy paths take.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GUARD = 256
PATTERN = 0xA5


class Guarded:
    """Allocates outputs inside guarded byte ranges and checks the guards afterwards."""

    def __init__(self, torch):
        self.torch = torch
        self.bufs = []

    def new(self, shape, dtype, fill=None, misalign=0):
        torch = self.torch
        n = int(np.prod(shape))
        esz = torch.empty((), dtype=dtype).element_size()
        lead = GUARD + misalign * esz
        raw = torch.full((lead + n * esz + GUARD,), PATTERN, dtype=torch.uint8, device="cuda")
        view = raw[lead:lead + n * esz].view(dtype).view(*shape)
        if fill is not None:
            view.copy_(fill)
        self.bufs.append((raw, lead, n * esz))
        return view

    def check(self, what=""):
        self.torch.cuda.synchronize()
        for i, (raw, lead, nbytes) in enumerate(self.bufs):
            head, tail = raw[:lead], raw[lead + nbytes:]
            assert bool((head == PATTERN).all()), f"{what}: output {i} written before its start"
            assert bool((tail == PATTERN).all()), f"{what}: output {i} written past its end"
        self.bufs = []


@pytest.fixture(scope="module")
def dev():
    import torch
    from ane_b200 import dev_ops, lib
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    lib.init(0)
    return dev_ops


def _dt(name):
    import torch
    return {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[name]


NORM_SHAPES = [(3, 7, 5), (2, 128, 257), (2, 129, 72), (1, 3000, 33), (5, 1024, 64), (3, 1024, 2048 + 24), (1, 257, 1), (2, 768, 256)]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", NORM_SHAPES)
def test_norm_operators_stay_inside_their_outputs(dev, shape, dt):
    import torch
    from ane_b200 import lib
    tdt = _dt(dt)
    B, C, S = shape
    g = torch.Generator(device="cuda").manual_seed(1)
    x, f, dy = (torch.randn(B, C, S, device="cuda", generator=g).to(tdt) for _ in range(3))
    w = 1 + 0.02 * torch.randn(C, device="cuda", generator=g)
    G = Guarded(torch)
    dev.rmsnorm(x, w, out=G.new(shape, tdt))
    G.check("rmsnorm")
    dev.residual_rmsnorm(x, f, w, 0.25, x2=G.new(shape, tdt), x2norm=G.new(shape, tdt))
    G.check("residual_rmsnorm")
    for knob in (None, 0, 8, 9, 10, 11, 12):
        if knob is not None:
            lib.set_tuning("norm_bwd", knob)
        try:
            for add in (None, f):
                dev.rmsnorm_bwd(dy, x, w, G.new((C,), torch.float32, fill=0.0), add=add, out=G.new(shape, tdt))
                G.check(f"rmsnorm_bwd knob {knob} add {add is not None}")
        finally:
            lib.clear_tuning("norm_bwd")
    for knob in (0, 2, 3, 4, 6):
        lib.set_tuning("norm_fwd", knob)
        try:
            dev.rmsnorm(x, w, out=G.new(shape, tdt))
            dev.residual_rmsnorm(x, f, w, 0.25, x2=G.new(shape, tdt), x2norm=G.new(shape, tdt))
            G.check(f"norm_fwd knob {knob}")
        finally:
            lib.clear_tuning("norm_fwd")
    # the allocation-free entry point writes the same outputs
    if C <= 2048:
        L = lib.load()
        dx, dw = G.new(shape, tdt), G.new((C,), torch.float32, fill=0.0)
        rc = L.ane_cuda_rmsnorm_bwd_static_dev(torch.cuda.current_stream().cuda_stream, lib.F32 if dt == "f32" else lib.BF16, B, C, S,
                                               dx.data_ptr(), dw.data_ptr(), dy.data_ptr(), x.data_ptr(), w.data_ptr(), None, 1e-5, 0)
        assert rc == lib.OK
        G.check("rmsnorm_bwd_static")


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("n,mis", [(1, 0), (1023, 0), (4099, 1), (2048 * 256, 0), (2048 * 256 + 7, 3)])
def test_flat_operators_stay_inside_their_outputs(dev, n, mis, dt):
    import torch
    tdt = _dt(dt)
    g = torch.Generator(device="cuda").manual_seed(2)
    a, b, c = (torch.randn(n, device="cuda", generator=g).to(tdt) for _ in range(3))
    G = Guarded(torch)
    dev.residual(a, b, 0.3, out=G.new((n,), tdt, misalign=mis))
    dev.scale(a, 0.3, out=G.new((n,), tdt, misalign=mis))
    dev.swiglu(a, b, out=G.new((n,), tdt, misalign=mis))
    dev.swiglu_bwd(a, b, c, dh1=G.new((n,), tdt, misalign=mis), dh3=G.new((n,), tdt, misalign=mis))
    dev.convert(a, torch.float32 if dt != "f32" else torch.bfloat16, out=G.new((n,), torch.float32 if dt != "f32" else torch.bfloat16))
    G.check("flat operators")
    if dt == "f32":
        w, m, v = G.new((n,), tdt, fill=a, misalign=mis), G.new((n,), tdt, fill=0.01 * b, misalign=mis), G.new((n,), tdt, fill=(0.01 * c).abs(), misalign=mis)
        nsq = dev.grad_norm_sq(b, 1.0, out=G.new((1,), torch.float32))
        clip = dev.clip_factor(nsq, 1.0, out=G.new((1,), torch.float32))
        dev.adam(w, b, m, v, 1, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, clip=clip)
        G.check("adam / grad norm")


QK_SHAPES = [(2, 3, 8, 37), (1, 2, 32, 5), (3, 16, 128, 40), (2, 4, 128, 64 * 3 + 8), (5, 16, 128, 2048 + 72), (1, 12, 64, 130)]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,heads,hd,S", QK_SHAPES)
def test_rope_and_qknorm_operators_stay_inside_their_outputs(dev, B, heads, hd, S, dt):
    import torch
    from ane_b200 import lib
    tdt = _dt(dt)
    g = torch.Generator(device="cuda").manual_seed(3)
    shape = (B, heads * hd, S)
    x, dy = (torch.randn(*shape, device="cuda", generator=g).to(tdt) for _ in range(2))
    w = 1 + 0.02 * torch.randn(hd, device="cuda", generator=g)
    G = Guarded(torch)
    lib.poll_status(reset=True)
    for knobs in ((), (("qk_fwd", 0), ("qk_bwd", 0)), (("qk_fwd", 4), ("qk_bwd", 4)), (("qk_fwd", 6), ("qk_bwd", 6))):
        for k, v in knobs:
            lib.set_tuning(k, v)
        try:
            dev.rope(x, hd, base=1e6, pos0=2, out=G.new(shape, tdt))
            dev.rope(x, hd, base=1e6, inverse=True, out=G.new(shape, tdt))
            dev.qknorm(x, w, hd, out=G.new(shape, tdt))
            dev.qknorm_rope(x, w, hd, out=G.new(shape, tdt))
            dev.qknorm_bwd(dy, x, w, G.new((hd,), torch.float32, fill=0.0), hd, out=G.new(shape, tdt))
            dev.rope_qknorm_bwd(dy, x, w, G.new((hd,), torch.float32, fill=0.0), hd, out=G.new(shape, tdt))
            G.check(f"qk operators, knobs {knobs}")
            if heads % 2 == 0:
                kv, ratio = heads // 2, 2
                xk = x[:, :kv * hd].contiguous()
                if hd in (64, 128) and (S * x.element_size()) % 16 == 0:      # the shapes the fused K-side forms cover
                    dev.qknorm_rope_tiled(xk, w, hd, ratio, out=G.new(shape, tdt))
                    dev.rope_qknorm_bwd_gqa(dy, xk, w, G.new((hd,), torch.float32, fill=0.0), hd, ratio, out=G.new((B, kv * hd, S), tdt))
                dev.gqa_tile(xk, kv, ratio, out=G.new(shape, tdt))
                dev.gqa_reduce(dy, kv, ratio, out=G.new((B, kv * hd, S), tdt))
                G.check(f"gqa operators, knobs {knobs}")
        finally:
            for k, _ in knobs:
                lib.clear_tuning(k)
    assert lib.poll_status().wait_giveups == 0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("B,D,S,V", [(3, 5, 7, 11), (1, 100, 33, 70000), (2, 1024, 72, 151936), (1, 768, 256, 32000), (2, 96, 130, 50)])
def test_embedding_operators_stay_inside_their_outputs(dev, B, D, S, V, dt):
    import torch
    from ane_b200 import lib
    tdt = _dt(dt)
    g = torch.Generator(device="cuda").manual_seed(4)
    table = (0.02 * torch.randn(V, D, device="cuda", generator=g)).to(tdt)
    tok = torch.randint(0, V, (B, S), device="cuda", dtype=torch.int32, generator=g)
    tok[0, : min(S, 9)] = tok[0, 0]                              # a run of one id
    G = Guarded(torch)
    for knobs in ((), (("embed_rows", 0),), (("embed_tiled", 0),)):
        for k, v in knobs:
            lib.set_tuning(k, v)
        try:
            x = dev.embed_lookup(table, tok, out=G.new((B, D, S), tdt))
            G.check(f"embed_lookup {knobs}")
            dev.embed_backward(G.new((V, D), torch.float32, fill=0.0), x.clone(), tok)
            G.check(f"embed_backward {knobs}")
        finally:
            for k, _ in knobs:
                lib.clear_tuning(k)


@pytest.mark.parametrize("B,V,S", [(3, 17, 4), (2, 1000, 37), (1, 9200, 256), (2, 32001, 72), (1, 151936, 40)])
def test_cross_entropy_stays_inside_its_outputs(dev, B, V, S):
    import torch
    from ane_b200 import lib
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(B, V, S, device="cuda", generator=g)
    tg = torch.randint(0, V, (B, S), device="cuda", dtype=torch.int32, generator=g)
    G = Guarded(torch)
    for knobs in ((), (("xent_cluster", 1),), (("xent_split", 8),), (("xent_lg", 4),), (("xent_lg", 32),)):
        for k, v in knobs:
            lib.set_tuning(k, v)
        try:
            dev.cross_entropy(logits, tg, dlogits=G.new((B, V, S), torch.float32))
            G.check(f"cross_entropy {knobs}")
        finally:
            for k, _ in knobs:
                lib.clear_tuning(k)
