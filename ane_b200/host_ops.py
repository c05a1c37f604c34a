"""Batched host-buffer operators (``ane_cuda_*_host``) on torch CPU tensors.

The tensors live in host memory (page-locked for full speed: ``tensor.pin_memory()`` or
``torch.empty(..., pin_memory=True)``); each call uploads its inputs, runs the CUDA kernels and
downloads the results through the library's three-stream pipeline, and returns when the results
are in host memory.  Activations are ``[B, C, S]`` of fp32 / bf16 / fp16; w and dw are fp32.
"""
from __future__ import annotations

import torch

from . import lib as _l

_DT = {torch.float32: _l.F32, torch.bfloat16: _l.BF16, torch.float16: _l.F16}


def _p(t, like=None, what="tensor"):
    """Host address of a contiguous CPU tensor; `like`: a tensor whose shape and dtype it must share, or an element count
    (for fp32 weight vectors) -- a buffer smaller than the shape arguments say would be read or written past its end."""
    if t is None:
        return None
    if t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{what}: expected a contiguous CPU tensor")
    if isinstance(like, int):
        if t.dtype != torch.float32 or t.numel() != like:
            raise ValueError(f"{what}: expected {like} float32 values, got {t.numel()} of {t.dtype}")
    elif like is not None and (t.shape != like.shape or t.dtype != like.dtype):
        raise ValueError(f"{what}: shape {tuple(t.shape)} / {t.dtype} does not match {tuple(like.shape)} / {like.dtype}")
    return t.data_ptr()


def _bcs(x):
    if x.dim() != 3:
        raise ValueError("activations are [B, C, S]")
    return x.shape


def rmsnorm(out, x, w, eps=1e-5):
    B, C, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rmsnorm_host(_DT[x.dtype], B, C, S, _p(out, x, "out"), _p(x), _p(w, C, "w"), eps))


def rmsnorm_bwd(dx, dw, dy, x, w, add=None, eps=1e-5, exact=False):
    B, C, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rmsnorm_bwd_host(_DT[x.dtype], B, C, S, _p(dx, x, "dx"), _p(dw, C, "dw"), _p(dy, x, "dy"), _p(x), _p(w, C, "w"), _p(add, x, "add"),
                                                eps, _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))


def residual(out, x, f, alpha):
    _l.check(_l.load().ane_cuda_residual_host(_DT[x.dtype], x.numel(), _p(out, x, "out"), _p(x), _p(f, x, "f"), alpha))


def residual_rmsnorm(x2, x2norm, x, f, w, alpha, eps=1e-5):
    B, C, S = _bcs(x)
    _l.check(_l.load().ane_cuda_residual_rmsnorm_host(_DT[x.dtype], B, C, S, _p(x2, x, "x2"), _p(x2norm, x, "x2norm"), _p(x), _p(f, x, "f"), _p(w, C, "w"),
                                                     alpha, eps))


def swiglu(out, h1, h3):
    _l.check(_l.load().ane_cuda_swiglu_host(_DT[h1.dtype], h1.numel(), _p(out, h1, "out"), _p(h1), _p(h3, h1, "h3")))


def swiglu_bwd(dh1, dh3, h1, h3, dsilu):
    _l.check(_l.load().ane_cuda_swiglu_bwd_host(_DT[h1.dtype], h1.numel(), _p(dh1, h1, "dh1"), _p(dh3, h1, "dh3"), _p(h1), _p(h3, h1, "h3"),
                                                _p(dsilu, h1, "dsilu")))


def rope(out, x, hd, base=10000.0, pos0=0, inverse=False):
    B, C, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rope_host(_DT[x.dtype], B, C, S, hd, _p(out, x, "out"), _p(x), base, pos0,
                                         _l.ROPE_INVERSE if inverse else _l.ROPE_FORWARD))


def qknorm_rope(out, x, w, hd, eps=1e-6, base=1e6, pos0=0):
    B, C, S = _bcs(x)
    if C % hd:
        raise ValueError(f"{C} channels are not a whole number of heads of {hd}")
    _l.check(_l.load().ane_cuda_qknorm_rope_host(_DT[x.dtype], B, C // hd, hd, S, _p(out, x, "out"), _p(x), _p(w, hd, "w"), eps, base, pos0))


def rope_qknorm_bwd(dx, dw, dy, x, w, hd, eps=1e-6, base=1e6, pos0=0, exact=False):
    B, C, S = _bcs(x)
    if C % hd:
        raise ValueError(f"{C} channels are not a whole number of heads of {hd}")
    _l.check(_l.load().ane_cuda_rope_qknorm_bwd_host(_DT[x.dtype], B, C // hd, hd, S, _p(dx, x, "dx"), _p(dw, hd, "dw"), _p(dy, x, "dy"), _p(x), _p(w, hd, "w"),
                                                    eps, base, pos0, _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))
