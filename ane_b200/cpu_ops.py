"""Host-side mirror of the reference's operator interface, backed by the GPU library.

The function names, argument order and overwrite / accumulate behaviour are those of
training/stories_cpu_ops.h and training/training_dynamic/cpu_ops.h (the module is named after
the latter); arguments are C-contiguous numpy arrays standing in for the reference's
``float *`` / ``uint16_t *``.  Every call goes through the host-pointer entry points of
libane_cuda (host -> device copy, kernel, device -> host copy); nothing is computed on the CPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _l

_fp = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)


def _f(a: np.ndarray):
    if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError("expected a C-contiguous float32 array")
    return a.ctypes.data_as(_fp)


def _u(a: np.ndarray):
    if a.dtype != np.uint16 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError("expected a C-contiguous uint16 array")
    return a.ctypes.data_as(_u16p)


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
    _l.check(_l.load().ane_cuda_rmsnorm(_f(out), _f(x), _f(w), d, S))


def rmsnorm_bwd(dx, dw, dy, x, w, d, S):
    """stories_cpu_ops.h:23 -- dx overwritten, dw accumulated into."""
    _l.check(_l.load().ane_cuda_rmsnorm_bwd(_f(dx), _f(dw), _f(dy), _f(x), _f(w), d, S))


def adam_update(w, g, s: AdamState, t, lr, b1, b2, eps, wd=None):
    """stories_cpu_ops.h:55 (wd is None) or training_dynamic/cpu_ops.h:56 (wd given)."""
    cs = s._c()
    if wd is None:
        _l.check(_l.load().ane_cuda_adam_update(_f(w), _f(g), C.byref(cs), t, lr, b1, b2, eps))
    else:
        _l.check(_l.load().ane_cuda_adam_update_wd(_f(w), _f(g), C.byref(cs), t, lr, b1, b2, eps, wd))


def cross_entropy_loss(dlogits, logits, targets, V, S) -> float:
    """stories_cpu_ops.h:71 -- returns the mean loss, writes dlogits[V,S]."""
    loss = C.c_float(0.0)
    _l.check(_l.load().ane_cuda_cross_entropy_loss(C.byref(loss), _f(dlogits), _f(logits), _u(targets), V, S))
    return float(loss.value)


def embed_lookup(x, embed, tokens, dim, seq, vocab=None):
    """stories_cpu_ops.h:112 -- x[dim,seq] gathered from embed[vocab,dim]."""
    vocab = embed.shape[0] if vocab is None else vocab
    _l.check(_l.load().ane_cuda_embed_lookup(_f(x), _f(embed), _u(tokens), dim, seq, vocab))


def embed_backward(d_embed, dx, tokens, dim, seq, vocab=None):
    """stories_cpu_ops.h:123 -- d_embed[tok] += dx[:,t]."""
    vocab = d_embed.shape[0] if vocab is None else vocab
    _l.check(_l.load().ane_cuda_embed_backward(_f(d_embed), _f(dx), _u(tokens), dim, seq, vocab))


def rope_backward_inplace(dx, seq, dim, hd):
    """training_dynamic/cpu_ops.h:168"""
    _l.check(_l.load().ane_cuda_rope_backward_inplace(_f(dx), seq, dim, hd))


def residual(out, x, f, alpha):
    """training_dynamic/train.m:460 -- out = f*alpha + x"""
    _l.check(_l.load().ane_cuda_residual(_f(out), _f(x), _f(f), alpha, x.size))


def swiglu(out, h1, h3):
    """training/forward.h:101,149-151"""
    _l.check(_l.load().ane_cuda_swiglu(_f(out), _f(h1), _f(h3), h1.size))


def swiglu_bwd(dh1, dh3, h1, h3, dsilu):
    """training_dynamic/train.m:537-554"""
    _l.check(_l.load().ane_cuda_swiglu_bwd(_f(dh1), _f(dh3), _f(h1), _f(h3), _f(dsilu), h1.size))
