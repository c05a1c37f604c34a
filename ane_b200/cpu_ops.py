"""Host-side mirror of the reference's operator interface, backed by the GPU library.

The function names, argument order and overwrite / accumulate behaviour are those of
training/stories_cpu_ops.h and training/training_dynamic/cpu_ops.h (the module is named after
the latter); arguments are C-contiguous numpy arrays standing in for the reference's
``float *`` / ``uint16_t *``.  Every call goes through the host-pointer entry points of
libane_cuda (host -> device copy, kernel, device -> host copy); nothing is computed on the CPU.

The reference's functions trust their caller with the sizes; a numpy array that is smaller than
the (d, S) it is passed with would make the library read or write past it.  Every function here
therefore checks dtype, contiguity and element count of each array against its size arguments and
raises ValueError / TypeError before anything is handed to C.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _l

_fp = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)


def _f(a: np.ndarray, n=None, what="array"):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{what}: expected a C-contiguous float32 array")
    if n is not None and a.size != n:
        raise ValueError(f"{what}: {a.size} elements, the size arguments say {n}")
    return a.ctypes.data_as(_fp)


def _u(a: np.ndarray, n=None, what="array"):
    if not isinstance(a, np.ndarray) or a.dtype != np.uint16 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{what}: expected a C-contiguous uint16 array")
    if n is not None and a.size != n:
        raise ValueError(f"{what}: {a.size} elements, the size arguments say {n}")
    return a.ctypes.data_as(_u16p)


def _positive(**sizes):
    for k, v in sizes.items():
        if int(v) != v or v < 1:
            raise ValueError(f"{k} must be a positive integer (got {v!r})")


class AdamState:
    """``typedef struct { float *m, *v; size_t n; } AdamState`` (stories_config.h:56-59)."""

    def __init__(self, n: int):
        self.m = np.zeros(n, np.float32)
        self.v = np.zeros(n, np.float32)
        self.n = n

    def _c(self) -> _l.AdamState:
        return _l.AdamState(_f(self.m), _f(self.v), self.n)


def rmsnorm(out, x, w, d, S):
    """stories_cpu_ops.h:6 -- out[d,S] = x * rrms * w, eps = 1e-5."""
    _positive(d=d, S=S)
    _l.check(_l.load().ane_cuda_rmsnorm(_f(out, d * S, "out"), _f(x, d * S, "x"), _f(w, d, "w"), d, S))


def rmsnorm_bwd(dx, dw, dy, x, w, d, S):
    """stories_cpu_ops.h:23 -- dx overwritten, dw accumulated into."""
    _positive(d=d, S=S)
    _l.check(_l.load().ane_cuda_rmsnorm_bwd(_f(dx, d * S, "dx"), _f(dw, d, "dw"), _f(dy, d * S, "dy"), _f(x, d * S, "x"), _f(w, d, "w"), d, S))


def adam_update(w, g, s: AdamState, t, lr, b1, b2, eps, wd=None):
    """stories_cpu_ops.h:55 (wd is None) or training_dynamic/cpu_ops.h:56 (wd given)."""
    if s.m.size != s.n or s.v.size != s.n:
        raise ValueError("AdamState: m and v must hold n elements")
    if t < 1:
        raise ValueError("t counts optimizer steps from 1 (the bias correction divides by 1 - b^t)")
    cs = s._c()
    if wd is None:
        _l.check(_l.load().ane_cuda_adam_update(_f(w, s.n, "w"), _f(g, s.n, "g"), C.byref(cs), t, lr, b1, b2, eps))
    else:
        _l.check(_l.load().ane_cuda_adam_update_wd(_f(w, s.n, "w"), _f(g, s.n, "g"), C.byref(cs), t, lr, b1, b2, eps, wd))


def cross_entropy_loss(dlogits, logits, targets, V, S) -> float:
    """stories_cpu_ops.h:71 -- returns the mean loss, writes dlogits[V,S]."""
    _positive(V=V, S=S)
    loss = C.c_float(0.0)
    _l.check(_l.load().ane_cuda_cross_entropy_loss(C.byref(loss), _f(dlogits, V * S, "dlogits"), _f(logits, V * S, "logits"),
                                                   _u(targets, S, "targets"), V, S))
    return float(loss.value)


def embed_lookup(x, embed, tokens, dim, seq, vocab=None):
    """stories_cpu_ops.h:112 -- x[dim,seq] gathered from embed[vocab,dim]."""
    vocab = embed.shape[0] if vocab is None else vocab
    _positive(dim=dim, seq=seq, vocab=vocab)
    _l.check(_l.load().ane_cuda_embed_lookup(_f(x, dim * seq, "x"), _f(embed, vocab * dim, "embed"), _u(tokens, seq, "tokens"), dim, seq, vocab))


def embed_backward(d_embed, dx, tokens, dim, seq, vocab=None):
    """stories_cpu_ops.h:123 -- d_embed[tok] += dx[:,t]."""
    vocab = d_embed.shape[0] if vocab is None else vocab
    _positive(dim=dim, seq=seq, vocab=vocab)
    _l.check(_l.load().ane_cuda_embed_backward(_f(d_embed, vocab * dim, "d_embed"), _f(dx, dim * seq, "dx"), _u(tokens, seq, "tokens"), dim, seq, vocab))


def rope_backward_inplace(dx, seq, dim, hd):
    """training_dynamic/cpu_ops.h:168"""
    _positive(seq=seq, dim=dim, hd=hd)
    if dim % hd or hd % 2:
        raise ValueError(f"dim {dim} must be a multiple of the head width {hd}, which must be even (pairs of channels rotate together)")
    _l.check(_l.load().ane_cuda_rope_backward_inplace(_f(dx, dim * seq, "dx"), seq, dim, hd))


def residual(out, x, f, alpha):
    """training_dynamic/train.m:460 -- out = f*alpha + x"""
    _l.check(_l.load().ane_cuda_residual(_f(out, x.size, "out"), _f(x, None, "x"), _f(f, x.size, "f"), alpha, x.size))


def swiglu(out, h1, h3):
    """training/forward.h:101,149-151"""
    _l.check(_l.load().ane_cuda_swiglu(_f(out, h1.size, "out"), _f(h1, None, "h1"), _f(h3, h1.size, "h3"), h1.size))


def swiglu_bwd(dh1, dh3, h1, h3, dsilu):
    """training_dynamic/train.m:537-554"""
    n = h1.size
    _l.check(_l.load().ane_cuda_swiglu_bwd(_f(dh1, n, "dh1"), _f(dh3, n, "dh3"), _f(h1, None, "h1"), _f(h3, n, "h3"), _f(dsilu, n, "dsilu"), n))
