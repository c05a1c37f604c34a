"""Generate tests/golden/golden.npz from the REFERENCE's own functions.

Run where the reference tree is present (it compiles the two reference operator headers into
oracle/_ref first):

    python tests/golden/make_golden.py

Inputs are the seeded sequences of ``gen_inputs.py`` (the reference tests' own drand48
fixtures plus PCG64 inputs with the benchmark shapes); outputs come from
``oracle.oracle.Reference`` -- i.e. from training/stories_cpu_ops.h and
training/training_dynamic/cpu_ops.h compiled unmodified.  To keep the fixture small each
large output is stored as a strided sample (``<name>`` with ``<name>_stride``) plus its
float64 sum and absolute sum; small outputs (dw, losses) are stored whole.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_oracle  # noqa: E402
from oracle.oracle import Reference, ReferenceInline  # noqa: E402
from tests.golden import gen_inputs as gi  # noqa: E402

OUT = os.path.join(HERE, "golden.npz")


def sample(store: dict, name: str, a: np.ndarray, stride: int) -> None:
    flat = np.ascontiguousarray(a).reshape(-1)
    store[name] = flat[::stride].copy()
    store[name + "_stride"] = np.int64(stride)
    store[name + "_sum"] = np.float64(flat.astype(np.float64).sum())
    store[name + "_abssum"] = np.float64(np.abs(flat.astype(np.float64)).sum())


def main() -> int:
    build_oracle.build_restatement()
    if not build_oracle.build_reference():
        print("reference tree not present; cannot regenerate golden vectors", file=sys.stderr)
        return 1
    ref = Reference()
    g: dict = {}

    # 1. training/test_rmsnorm_bwd.m fixture -> CPU rmsnorm_bwd (both header variants)
    x, dy, w = gi.fixture_rmsnorm_bwd()
    for variant in ("stories", "dynamic"):
        dx, dw = ref.rmsnorm_bwd(dy, x, w, variant=variant)
        sample(g, f"rmsbwd_fixture_{variant}_dx", dx, 53)
        g[f"rmsbwd_fixture_{variant}_dw"] = dw

    # 2. training/test_classifier.m test 1 fixture -> CPU rmsnorm
    x, w = gi.fixture_rmsnorm_fwd()
    for variant in ("stories", "dynamic"):
        sample(g, f"rms_fixture_{variant}_out", ref.rmsnorm(x, w, variant=variant), 53)

    # 3. training/test_classifier.m test 3 fixture (logits = 10u-5, V=32000, S=256):
    #    the reference CE on it, targets = (7919*t + 13) mod V.
    logits = gi.fixture_softmax_logits()
    V, S = logits.shape
    tg = ((7919 * np.arange(S) + 13) % V).astype(np.uint16)
    g["ce_fixture_targets"] = tg
    for variant in ("stories", "dynamic"):
        loss, dl = ref.cross_entropy_loss(logits, tg, variant=variant)
        g[f"ce_fixture_{variant}_loss"] = np.float32(loss)
        sample(g, f"ce_fixture_{variant}_dlogits", dl, 4099)
        # softmax of the first 4 positions (what test_classifier.m:173-185 looks at):
        # p = dlogits*S with the target's -1 undone
        p4 = dl[:, :4].astype(np.float64) * S
        for t in range(4):
            p4[tg[t], t] += 1.0
        g[f"ce_fixture_{variant}_psum4"] = p4.sum(axis=0)

    # 4. config-1 inputs (PCG64 1234) through the reference norm functions
    x, w, dy = gi.cfg1()
    sample(g, "cfg1_rms_out", ref.rmsnorm(x[0], w), 53)
    dx, dw = ref.rmsnorm_bwd(dy[0], x[0], w)
    sample(g, "cfg1_rmsbwd_dx", dx, 53)
    g["cfg1_rmsbwd_dw"] = dw

    # 5. Adam, both variants, three steps from the same state
    for name, wd in (("stories", None), ("dynamic", 0.1)):
        w0, g0, m0, v0 = gi.adam_inputs()
        b2 = 0.999 if wd is None else 0.95
        for t in (1, 2, 3):
            ref.adam_update(w0, g0, m0, v0, t, 3e-4, 0.9, b2, 1e-8, wd)
        sample(g, f"adam_{name}_w", w0, 17)
        sample(g, f"adam_{name}_m", m0, 17)
        sample(g, f"adam_{name}_v", v0, 17)

    # 6. embedding gather / scatter (dim 768, seq 256, vocab 32000; uint16 ids, some repeated)
    r = gi.rng(77)
    tok = r.integers(0, 32000, size=256).astype(np.uint16)
    tok[10:20] = tok[0]                      # repeated ids exercise the += order
    table = gi.normal(r, (32000, 768), 0.02)
    g["embed_tokens"] = tok
    xg = ref.embed_lookup(table, tok)
    sample(g, "embed_lookup_x", xg, 53)
    dxe = gi.normal(r, (768, 256))
    dE = ref.embed_backward(np.zeros((32000, 768), np.float32), dxe, tok)
    g["embed_backward_rows"] = dE[tok[:32].astype(np.int64)][:, ::7].copy()
    g["embed_backward_sum"] = np.float64(dE.astype(np.float64).sum())

    # 7. RoPE backward (dynamic header), Stories and Qwen3 head widths
    for name, (dim, hd) in (("hd64", (768, 64)), ("hd128", (2048, 128))):
        d = gi.normal(gi.rng(88), (dim, 256))
        sample(g, f"ropebwd_{name}", ref.rope_backward_inplace(d, hd), 53)

    # 8. vocab compaction
    data = gi.rng(99).integers(0, 32000, size=20000).astype(np.uint16)
    cv, f2c, c2f = ref.vocab_map_build(data, 32000)
    g["vocab_cv"] = np.int64(cv)
    g["vocab_c2f_head"] = c2f[:64].copy()
    g["vocab_f2c_sum"] = np.int64(f2c.astype(np.int64).sum())

    # 9. the inline operator blocks of training_dynamic/train.m and the helpers of training/forward.h
    rin = ReferenceInline()
    h1, h3, d, x, f = (a[0] for a in gi.cfg2())
    dh1, dh3 = rin.swiglu_bwd(h1, h3, d)                                   # train.m:538-554
    sample(g, "inline_swiglu_bwd_dh1", dh1, 53)
    sample(g, "inline_swiglu_bwd_dh3", dh3, 53)
    sample(g, "inline_swiglu", rin.swiglu(h1, h3), 53)                    # forward.h:101,149-151
    for name, alpha in (("a25", np.float32(24.0 ** -0.25)), ("a50", np.float32(1.0) / np.sqrt(np.float32(24.0)))):
        sample(g, f"inline_residual_{name}", rin.residual(x, f, alpha), 53)  # train.m:460 (alpha of train.m:188 is a50)
    q = gi.cfg3()[0][0]
    sample(g, "inline_rope_hd128", rin.rope_channel_first(q, 128), 53)    # forward.h:55-70
    sample(g, "inline_rope_hd64", rin.rope_channel_first(np.ascontiguousarray(q[:768]), 64), 53)
    layers, fin, emb = gi.grad_post_inputs()
    norm, nsq = rin.grad_scale_norm_clip(layers, fin, emb, gi.GRAD_POST_GSC, 1.0)   # train.m:754-767,770-788,809-825
    g["inline_grad_norm"] = np.float32(norm)
    g["inline_grad_norm_sq"] = np.float32(nsq)
    sample(g, "inline_grad_flat", gi.grad_post_flat(layers, fin, emb), 7)

    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT}: {os.path.getsize(OUT)/1024:.1f} KiB, {len(g)} arrays")
    return 0


if __name__ == "__main__":
    sys.exit(main())
