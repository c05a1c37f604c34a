"""Seeded inputs shared by the golden-vector generator and the tests.

Two families:

* ``drand48`` fixtures -- the exact input sequences of the reference's own tests
  (training/test_rmsnorm_bwd.m:26-33, training/test_classifier.m:25-27,132-134).  ``drand48``
  is the POSIX 48-bit linear congruential generator, restated here in numpy so the fixtures
  can be rebuilt on any box (``Drand48`` is checked against libc in the CPU tests).
* PCG64 inputs with the shapes and value distributions of the benchmark configurations
  (synthetic stand-ins: the reference's TinyStories token file and checkpoint are not
  available offline, and no item of that dataset is reproduced here).
"""
from __future__ import annotations

import numpy as np

_A = 0x5DEECE66D
_C = 0xB
_M48 = (1 << 48) - 1


def _mulmod48(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """(a*b) mod 2^48 for uint64 arrays holding 48-bit values (24-bit limb split)."""
    m24 = np.uint64((1 << 24) - 1)
    s24 = np.uint64(24)
    a_lo, a_hi = a & m24, a >> s24
    b_lo, b_hi = b & m24, b >> s24
    lo = a_lo * b_lo
    mid = (a_hi * b_lo + a_lo * b_hi) & m24
    return (lo + (mid << s24)) & np.uint64(_M48)


class Drand48:
    """POSIX srand48/drand48: X <- (0x5DEECE66D * X + 0xB) mod 2^48, value X / 2^48."""

    def __init__(self, seed: int):
        self.x = ((seed & 0xFFFFFFFF) << 16) | 0x330E

    def next(self, n: int) -> np.ndarray:
        """Next n drand48() values as float64."""
        blk = 4096
        first = min(n, blk)
        xs = np.empty(first, dtype=np.uint64)
        x = self.x
        for i in range(first):
            x = (_A * x + _C) & _M48
            xs[i] = x
        if n <= blk:
            self.x = int(xs[n - 1])
            return xs.astype(np.float64) / float(1 << 48)
        # jump-ahead by blk: X_{k+blk} = AK * X_k + CK
        ak, ck = 1, 0
        for _ in range(blk):
            ck = (_A * ck + _C) & _M48
            ak = (_A * ak) & _M48
        nblk = (n + blk - 1) // blk
        out = np.empty((nblk, blk), dtype=np.uint64)
        out[0] = xs
        AK = np.full(blk, ak, dtype=np.uint64)
        CK = np.uint64(ck)
        for b in range(1, nblk):
            out[b] = (_mulmod48(AK, out[b - 1]) + CK) & np.uint64(_M48)
        flat = out.reshape(-1)[:n]
        self.x = int(flat[-1])
        return flat.astype(np.float64) / float(1 << 48)


# ---------------------------------------------------------------- reference-test fixtures
def fixture_rmsnorm_bwd(dim: int = 768, seq: int = 256):
    """training/test_rmsnorm_bwd.m:26-33: srand48(42); x and dy drawn alternately per element,
    x = (2u-1)*0.5, dy = (2u-1)*0.1 (float casts as there); then w = 0.5u + 0.75."""
    g = Drand48(42)
    u = g.next(2 * dim * seq)
    x = ((u[0::2] * 2 - 1).astype(np.float32) * np.float32(0.5)).reshape(dim, seq)
    dy = ((u[1::2] * 2 - 1).astype(np.float32) * np.float32(0.1)).reshape(dim, seq)
    w = (g.next(dim) * 0.5 + 0.75).astype(np.float32)
    return np.ascontiguousarray(x), np.ascontiguousarray(dy), w


def fixture_rmsnorm_fwd(dim: int = 768, seq: int = 256):
    """training/test_classifier.m:25-27: srand48(42); x = 2u-1 ; w = 0.5u + 0.75."""
    g = Drand48(42)
    x = (g.next(dim * seq) * 2 - 1).astype(np.float32).reshape(dim, seq)
    w = (g.next(dim) * 0.5 + 0.75).astype(np.float32)
    return np.ascontiguousarray(x), w


def fixture_softmax_logits(vocab: int = 32000, seq: int = 256):
    """training/test_classifier.m:132-134: srand48(999); logits = 10u - 5, [VOCAB, SEQ]."""
    g = Drand48(999)
    return np.ascontiguousarray((g.next(vocab * seq) * 10 - 5).astype(np.float32).reshape(vocab, seq))


# ---------------------------------------------------------------- benchmark-shaped inputs
def rng(seed: int = 1234) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def normal(r: np.random.Generator, shape, std: float = 1.0, mean: float = 0.0) -> np.ndarray:
    return (r.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)


def cfg1(seed: int = 1234, B: int = 1, dim: int = 768, seq: int = 256):
    """RMSNorm fwd+bwd: x ~ N(0,1), w = 1 + 0.02 N(0,1), dy ~ N(0,1)."""
    r = rng(seed)
    x = normal(r, (B, dim, seq))
    w = normal(r, (dim,), 0.02, 1.0)
    dy = normal(r, (B, dim, seq))
    return x, w, dy


def cfg2(seed: int = 1234, B: int = 1, hidden: int = 2048, dim: int = 768, seq: int = 256):
    """SwiGLU fwd+bwd and the DeepNet residual: h1, h3, d ~ N(0,1); x, f ~ N(0,1)."""
    r = rng(seed + 1)
    h1 = normal(r, (B, hidden, seq))
    h3 = normal(r, (B, hidden, seq))
    d = normal(r, (B, hidden, seq))
    x = normal(r, (B, dim, seq))
    f = normal(r, (B, dim, seq))
    return h1, h3, d, x, f


def cfg3(seed: int = 1234, B: int = 1, heads: int = 16, kv_heads: int = 8, hd: int = 128, seq: int = 256):
    """QK-norm + RoPE: Q, K ~ N(0,1); weights 1 + 0.02 N(0,1); upstream grads ~ N(0,1)."""
    r = rng(seed + 2)
    q = normal(r, (B, heads * hd, seq))
    k = normal(r, (B, kv_heads * hd, seq))
    wq = normal(r, (hd,), 0.02, 1.0)
    wk = normal(r, (hd,), 0.02, 1.0)
    dq = normal(r, (B, heads * hd, seq))
    dk = normal(r, (B, kv_heads * hd, seq))
    return q, k, wq, wk, dq, dk


def cfg4_tokens(seed: int = 1234, B: int = 1, seq: int = 256, vocab: int = 151936):
    r = rng(seed + 3)
    return r.integers(0, vocab, size=(B, seq), dtype=np.int64).astype(np.int32)


def cfg4_table(seed: int = 1234, vocab: int = 151936, dim: int = 1024):
    return normal(rng(seed + 4), (vocab, dim), 0.02)


def cfg4_logits(seed: int = 1234, B: int = 1, vocab: int = 151936, seq: int = 256):
    return normal(rng(seed + 5), (B, vocab, seq))


def adam_inputs(seed: int = 1234, n: int = 1 << 16):
    """w ~ N(0, 0.02), g ~ N(0, 1e-2), m ~ N(0, 1e-3), v = (N(0, 1e-3))^2 (non-negative)."""
    r = rng(seed + 6)
    w = normal(r, (n,), 0.02)
    g = normal(r, (n,), 1e-2)
    m = normal(r, (n,), 1e-3)
    v = np.square(normal(r, (n,), 1e-3)).astype(np.float32)
    return w, g, m, v


# ---------------------------------------------------------------- bf16 helpers (numpy has no bf16)
GRAD_POST_GSC = float(np.float32(1.0) / np.float32(10 * 256.0))      # 1/(accum_steps*loss_scale), train.m:750
GRAD_POST_FIELDS = ("Wq", "Wk", "Wv", "Wo", "W1", "W2", "W3", "rms_att", "rms_ffn")


def grad_post_inputs(seed: int = 1234, n_layers: int = 3, dim: int = 48, q_dim: int = 64, kv_dim: int = 32, hidden: int = 80,
                     vocab: int = 96):
    """Unscaled gradients of a small model in the reference's per-tensor arrangement (LayerGrads of
    training_dynamic/config.h, grms_final, gembed): large enough that the clip at 1.0 triggers after the scale."""
    r = rng(seed + 5)
    sizes = {"Wq": q_dim * dim, "Wk": kv_dim * dim, "Wv": kv_dim * dim, "Wo": dim * q_dim, "W1": hidden * dim,
             "W2": dim * hidden, "W3": hidden * dim, "rms_att": dim, "rms_ffn": dim}
    layers = [{k: normal(r, (sizes[k],), 60.0) for k in GRAD_POST_FIELDS} for _ in range(n_layers)]
    return layers, normal(r, (dim,), 60.0), normal(r, (vocab * dim,), 60.0)


def grad_post_flat(layers, grms_final, gembed) -> np.ndarray:
    """All tensors of grad_post_inputs as one flat array, in the order the reference's norm loop visits them."""
    return np.concatenate([lay[k] for lay in layers for k in GRAD_POST_FIELDS] + [grms_final, gembed]).astype(np.float32)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern (uint16), round-to-nearest-even; NaN stays NaN."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(a)
    if nan.any():
        r = np.where(nan, np.uint16(0x7FC0), r)
    return r


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_bf16(a: np.ndarray) -> np.ndarray:
    return from_bf16_bits(to_bf16_bits(a))


def round_f16(a: np.ndarray) -> np.ndarray:
    return a.astype(np.float16).astype(np.float32)
