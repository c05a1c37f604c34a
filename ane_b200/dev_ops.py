"""Device-resident operators on torch CUDA tensors.

PyTorch is used for device memory and streams only: each function passes ``data_ptr()`` and the
current stream handle to the ``_dev`` entry points of libane_cuda.  Tensors are channel-first
``[B, C, S]`` (or flat), contiguous, on the device the library was initialised on.
"""
from __future__ import annotations

import torch

from . import lib as _l

_DT = {torch.float32: _l.F32, torch.bfloat16: _l.BF16, torch.float16: _l.F16}
_ID = {torch.int32: _l.ID_I32, torch.uint16: _l.ID_U16, torch.int16: _l.ID_U16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor")
    return t.data_ptr()


def _dt(t):
    return _DT[t.dtype]


def _bcs(t):
    if t.dim() == 2:
        return 1, t.shape[0], t.shape[1]
    if t.dim() == 3:
        return t.shape
    raise ValueError("expected [B, C, S] or [C, S]")


def rmsnorm(x, w, eps=1e-5, out=None):
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rmsnorm_dev(_stream(), _dt(x), B, Cn, S, _p(out), _p(x), _p(w), eps))
    return out


def rmsnorm_bwd(dy, x, w, dw, add=None, eps=1e-5, exact=False, out=None):
    """dx = rmsnorm_bwd(dy, x, w) (+ add); dw (fp32 [C]) is accumulated into."""
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rmsnorm_bwd_dev(_stream(), _dt(x), B, Cn, S, _p(out), _p(dw), _p(dy), _p(x), _p(w),
                                               _p(add), eps, _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))
    return out


def residual(x, f, alpha, out=None):
    out = torch.empty_like(x) if out is None else out
    _l.check(_l.load().ane_cuda_residual_dev(_stream(), _dt(x), x.numel(), _p(out), _p(x), _p(f), alpha))
    return out


def scale(x, alpha, out=None):
    out = torch.empty_like(x) if out is None else out
    _l.check(_l.load().ane_cuda_scale_dev(_stream(), _dt(x), x.numel(), _p(out), _p(x), alpha))
    return out


def residual_rmsnorm(x, f, w, alpha, eps=1e-5, x2=None, x2norm=None):
    x2 = torch.empty_like(x) if x2 is None else x2
    x2norm = torch.empty_like(x) if x2norm is None else x2norm
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_residual_rmsnorm_dev(_stream(), _dt(x), B, Cn, S, _p(x2), _p(x2norm), _p(x), _p(f),
                                                    _p(w), alpha, eps))
    return x2, x2norm


def swiglu(h1, h3, out=None):
    out = torch.empty_like(h1) if out is None else out
    _l.check(_l.load().ane_cuda_swiglu_dev(_stream(), _dt(h1), h1.numel(), _p(out), _p(h1), _p(h3)))
    return out


def swiglu_bwd(h1, h3, d, dh1=None, dh3=None):
    dh1 = torch.empty_like(h1) if dh1 is None else dh1
    dh3 = torch.empty_like(h1) if dh3 is None else dh3
    _l.check(_l.load().ane_cuda_swiglu_bwd_dev(_stream(), _dt(h1), h1.numel(), _p(dh1), _p(dh3), _p(h1), _p(h3),
                                              _p(d)))
    return dh1, dh3


def rope(x, hd, base=10000.0, pos0=0, inverse=False, out=None):
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rope_dev(_stream(), _dt(x), B, Cn, S, hd, _p(out), _p(x), base, pos0,
                                        _l.ROPE_INVERSE if inverse else _l.ROPE_FORWARD))
    return out


def qknorm(x, w, hd, eps=1e-6, out=None):
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_qknorm_dev(_stream(), _dt(x), B, Cn // hd, hd, S, _p(out), _p(x), _p(w), eps))
    return out


def qknorm_bwd(dy, x, w, dw, hd, eps=1e-6, exact=False, out=None):
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_qknorm_bwd_dev(_stream(), _dt(x), B, Cn // hd, hd, S, _p(out), _p(dw), _p(dy), _p(x),
                                              _p(w), eps, _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))
    return out


def qknorm_rope(x, w, hd, eps=1e-6, base=1e6, pos0=0, out=None):
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_qknorm_rope_dev(_stream(), _dt(x), B, Cn // hd, hd, S, _p(out), _p(x), _p(w), eps,
                                               base, pos0))
    return out


def rope_qknorm_bwd(dy, x, w, dw, hd, eps=1e-6, base=1e6, pos0=0, exact=False, out=None):
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rope_qknorm_bwd_dev(_stream(), _dt(x), B, Cn // hd, hd, S, _p(out), _p(dw), _p(dy),
                                                   _p(x), _p(w), eps, base, pos0,
                                                   _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))
    return out


def qknorm_rope_pair(q, k, wq, wk, hd, eps=1e-6, base=1e6, pos0=0, out_q=None, out_k=None):
    """qknorm_rope of Q and of K of one layer in one call (side by side on the GPU where the shapes allow it)."""
    out_q = torch.empty_like(q) if out_q is None else out_q
    out_k = torch.empty_like(k) if out_k is None else out_k
    B, Cq, S = _bcs(q)
    Bk, Ck, Sk = _bcs(k)
    if (Bk, Sk) != (B, S) or _dt(k) != _dt(q):
        raise ValueError("q and k must agree in batch, sequence length and dtype")
    _l.check(_l.load().ane_cuda_qknorm_rope_pair_dev(_stream(), _dt(q), B, Cq // hd, Ck // hd, hd, S, _p(out_q), _p(out_k),
                                                    _p(q), _p(k), _p(wq), _p(wk), eps, base, pos0))
    return out_q, out_k


def rope_qknorm_bwd_pair(dyq, dyk, q, k, wq, wk, dwq, dwk, hd, eps=1e-6, base=1e6, pos0=0, exact=False, out_q=None, out_k=None):
    """rope_qknorm_bwd of Q and of K of one layer in one call; dwq / dwk are accumulated into."""
    out_q = torch.empty_like(q) if out_q is None else out_q
    out_k = torch.empty_like(k) if out_k is None else out_k
    B, Cq, S = _bcs(q)
    Bk, Ck, Sk = _bcs(k)
    if (Bk, Sk) != (B, S) or _dt(k) != _dt(q):
        raise ValueError("q and k must agree in batch, sequence length and dtype")
    _l.check(_l.load().ane_cuda_rope_qknorm_bwd_pair_dev(_stream(), _dt(q), B, Cq // hd, Ck // hd, hd, S, _p(out_q), _p(out_k),
                                                        _p(dwq), _p(dwk), _p(dyq), _p(dyk), _p(q), _p(k), _p(wq), _p(wk),
                                                        eps, base, pos0,
                                                        _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))
    return out_q, out_k


def embed_lookup(table, tokens, out=None, zero_oor=False):
    """table [V, D], tokens [B, S] (int32 or uint16 bits) -> x [B, D, S] of table's dtype."""
    B, S = tokens.shape
    V, D = table.shape
    out = torch.empty((B, D, S), dtype=table.dtype, device=table.device) if out is None else out
    _l.check(_l.load().ane_cuda_embed_lookup_dev(_stream(), _dt(table), _ID[tokens.dtype], B, D, S, _p(out), _p(table),
                                                _p(tokens), V, _l.OOR_ZERO if zero_oor else _l.OOR_SKIP))
    return out


def embed_backward(d_embed, dx, tokens):
    """d_embed [V, D] fp32 accumulated into; dx [B, D, S]; tokens [B, S]."""
    B, D, S = dx.shape
    V = d_embed.shape[0]
    _l.check(_l.load().ane_cuda_embed_backward_dev(_stream(), _dt(dx), _ID[tokens.dtype], B, D, S, _p(d_embed), _p(dx),
                                                  _p(tokens), V))
    return d_embed


def cross_entropy(logits, targets, grad_scale=1.0, dlogits=None):
    """logits [B, V, S] fp32; returns (loss_seq [B], dlogits).  dlogits may be logits (in place)."""
    B, V, S = _bcs(logits)
    dlogits = torch.empty_like(logits) if dlogits is None else dlogits
    loss = torch.empty(B, dtype=torch.float32, device=logits.device)
    _l.check(_l.load().ane_cuda_cross_entropy_dev(_stream(), _ID[targets.dtype], B, V, S, _p(dlogits), _p(logits),
                                                 _p(targets), _p(loss), grad_scale))
    return loss, dlogits


def adam(w, g, m, v, t, lr, b1, b2, eps, wd=0.0, gscale=1.0, clip=None, dynamic=True):
    _l.check(_l.load().ane_cuda_adam_dev(_stream(), w.numel(), _p(w), _p(g), _p(m), _p(v), t, lr, b1, b2, eps, wd,
                                        gscale, _p(clip), _l.ADAM_DYNAMIC if dynamic else _l.ADAM_STORIES))


def grad_norm_sq(g, gscale=1.0, out=None):
    out = torch.empty(1, dtype=torch.float32, device=g.device) if out is None else out
    _l.check(_l.load().ane_cuda_grad_norm_sq_dev(_stream(), g.numel(), _p(g), gscale, _p(out)))
    return out


def clip_factor(normsq, clip, out=None):
    out = torch.empty(1, dtype=torch.float32, device=normsq.device) if out is None else out
    _l.check(_l.load().ane_cuda_clip_factor_dev(_stream(), _p(normsq), normsq.numel(), clip, _p(out)))
    return out


# ------------------------------------------------------------------ layout helpers
def gqa_tile(x, kv_heads, ratio, out=None):
    """[B][kv_heads*hd][S] -> [B][kv_heads*ratio*hd][S] (training_dynamic/io.h gqa_tile_kv)."""
    B, Cn, S = _bcs(x)
    hd = Cn // kv_heads
    out = torch.empty((B, Cn * ratio, S), dtype=x.dtype, device=x.device) if out is None else out
    _l.check(_l.load().ane_cuda_gqa_tile_dev(_stream(), _dt(x), B, kv_heads, ratio, hd, S, _p(out), _p(x)))
    return out


def gqa_reduce(x, kv_heads, ratio, out=None):
    """[B][kv_heads*ratio*hd][S] -> [B][kv_heads*hd][S], heads summed in order (io.h gqa_reduce_kv)."""
    B, Cn, S = _bcs(x)
    hd = Cn // (kv_heads * ratio)
    out = torch.empty((B, kv_heads * hd, S), dtype=x.dtype, device=x.device) if out is None else out
    _l.check(_l.load().ane_cuda_gqa_reduce_dev(_stream(), _dt(x), B, kv_heads, ratio, hd, S, _p(out), _p(x)))
    return out


def convert(x, dtype, out=None):
    """Element-wise cast between float32 / float16 / bfloat16 (stories_io.h cvt_f32_f16, cvt_f16_f32)."""
    out = torch.empty(x.shape, dtype=dtype, device=x.device) if out is None else out
    _l.check(_l.load().ane_cuda_convert_dev(_stream(), _dt(out), _dt(x), x.numel(), _p(out), _p(x)))
    return out


def pack_dyn(act, W, dtype=torch.float16, out=None):
    """act [ic][seq] fp32, W [ic][oc] fp32 -> [ic][seq+oc] 16-bit (io.h io_write_dyn)."""
    ic, seq = act.shape
    oc = W.shape[1]
    out = torch.empty((ic, seq + oc), dtype=dtype, device=act.device) if out is None else out
    _l.check(_l.load().ane_cuda_pack_dyn_dev(_stream(), _dt(out), ic, seq, oc, _p(out), _p(act), _p(W)))
    return out


def vocab_map_build(tokens, full_vocab):
    """-> (full_to_compact [V] int32, compact_to_full [V] int32 (first compact_vocab entries valid),
    compact_vocab [1] int32), all on the device (cpu_ops.h vocab_map_build)."""
    dev = tokens.device
    f2c = torch.empty(full_vocab, dtype=torch.int32, device=dev)
    c2f = torch.empty(full_vocab, dtype=torch.int32, device=dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    _l.check(_l.load().ane_cuda_vocab_map_build_dev(_stream(), _ID[tokens.dtype], tokens.numel(), _p(tokens), full_vocab,
                                                   _p(f2c), _p(c2f), _p(cnt)))
    return f2c, c2f, cnt


def vocab_compact_embed(full_embed, c2f, cnt, compact_max, out=None):
    V, dim = full_embed.shape
    out = torch.empty((compact_max, dim), dtype=torch.float32, device=full_embed.device) if out is None else out
    _l.check(_l.load().ane_cuda_vocab_compact_embed_dev(_stream(), _p(out), _p(full_embed), _p(c2f), _p(cnt), compact_max, dim, V))
    return out


def vocab_scatter_grads(full_gembed, compact_gembed, c2f, cnt, compact_max):
    V, dim = full_gembed.shape
    _l.check(_l.load().ane_cuda_vocab_scatter_grads_dev(_stream(), _p(full_gembed), _p(compact_gembed), _p(c2f), _p(cnt), compact_max, dim, V))
    return full_gembed


def vocab_update_full(full_embed, compact_embed, c2f, cnt, compact_max):
    V, dim = full_embed.shape
    _l.check(_l.load().ane_cuda_vocab_update_full_dev(_stream(), _p(full_embed), _p(compact_embed), _p(c2f), _p(cnt), compact_max, dim, V))
    return full_embed


# ------------------------------------------------------------------ optimizer step over peer memory
def _ptr_array(ptrs):
    import ctypes as C
    return (C.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def p2p_reduce(g_ptrs, lo, n, g_slice, gscale=1.0, normsq=None, scratch=None, max_blocks=0):
    """g_slice[:n] = sum over ranks (in rank order) of their gradient buffers at [lo, lo+n); normsq = sum (g*gscale)^2.
    g_ptrs: device addresses of every rank's flat gradient buffer (peer-mapped).  max_blocks > 0 limits the grid (a
    background reduce on a side stream)."""
    normsq = torch.zeros(1, dtype=torch.float32, device=g_slice.device) if normsq is None else normsq
    arr = _ptr_array(g_ptrs)
    if scratch is not None and scratch.numel() < 1184:
        raise ValueError("scratch must hold 1184 floats")
    _l.check(_l.load().ane_cuda_p2p_reduce_limited_dev(_stream(), len(g_ptrs), arr, lo, n, _p(g_slice), gscale, _p(normsq), _p(scratch),
                                                       int(max_blocks)))
    return normsq


def p2p_adam(w_ptrs, rank, lo, n, g_slice, m_slice, v_slice, t, lr, b1, b2, eps, wd=0.0, gscale=1.0, clip=None, dynamic=True):
    """Adam on [lo, lo+n) of the flat parameters; the new weights go to every rank's buffer (w_ptrs, peer-mapped)."""
    arr = _ptr_array(w_ptrs)
    _l.check(_l.load().ane_cuda_p2p_adam_dev(_stream(), len(w_ptrs), rank, arr, lo, n, _p(g_slice), _p(m_slice), _p(v_slice), t, lr, b1,
                                             b2, eps, wd, gscale, _p(clip), _l.ADAM_DYNAMIC if dynamic else _l.ADAM_STORIES))


def rope_qknorm_bwd_gqa(dy_tiled, x, w, dw, hd, ratio, eps=1e-6, base=1e6, pos0=0, exact=False, out=None):
    """RoPE^-1 + QK-norm backward of the K side; dy_tiled [B][kv_heads*ratio*hd][S] is summed over each KV head's
    `ratio` query heads inside the kernel (gqa_reduce folded in)."""
    out = torch.empty_like(x) if out is None else out
    B, Cn, S = _bcs(x)
    _l.check(_l.load().ane_cuda_rope_qknorm_bwd_gqa_dev(_stream(), _dt(x), B, Cn // hd, ratio, hd, S, _p(out), _p(dw), _p(dy_tiled),
                                                        _p(x), _p(w), eps, base, pos0,
                                                        _l.NORM_BWD_EXACT if exact else _l.NORM_BWD_REFERENCE))
    return out


def qknorm_rope_tiled(x, w, hd, ratio, eps=1e-6, base=1e6, pos0=0, out=None):
    """QK-norm + RoPE of K [B][kv_heads*hd][S] written into the tiled layout [B][kv_heads*ratio*hd][S]."""
    B, Cn, S = _bcs(x)
    out = torch.empty((B, Cn * ratio, S), dtype=x.dtype, device=x.device) if out is None else out
    _l.check(_l.load().ane_cuda_qknorm_rope_tiled_dev(_stream(), _dt(x), B, Cn // hd, ratio, hd, S, _p(out), _p(x), _p(w), eps, base, pos0))
    return out
