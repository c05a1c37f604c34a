"""ctypes front-end for the CPU checker (TEST INFRASTRUCTURE ONLY).

``Oracle`` wraps ``liboracle.so`` (the C restatement in ``oracle_ops.c``); ``Reference`` wraps
the reference's own operator headers compiled into ``oracle/_ref`` (see ``build_oracle.py``).
Only the tests, the smoke entry and the benchmark's CPU-baseline leg may import this module;
the shipped package never does.

All arrays are C-contiguous numpy arrays; fp32 data, int32 token ids (uint16 for the
reference wrappers, which keep the reference's token type).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_u16p = C.POINTER(C.c_uint16)


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_f32p)


def _ip(a: np.ndarray):
    assert a.dtype == np.int32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_i32p)


def _up(a: np.ndarray):
    assert a.dtype == np.uint16 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u16p)


def ensure_built() -> None:
    need = [os.path.join(HERE, "liboracle.so"), os.path.join(HERE, "liboracle_fast.so")]
    if not all(os.path.exists(p) for p in need):
        from . import build_oracle  # noqa: WPS433 (local import: builds on demand)

        build_oracle.build_restatement()


class Oracle:
    """The C restatement.  ``fast=True`` loads the -O3/-march=native/OpenMP build that the
    benchmark times; the default build keeps the arithmetic as written (-ffp-contract=off)."""

    def __init__(self, fast: bool = False):
        ensure_built()
        self.lib = C.CDLL(os.path.join(HERE, "liboracle_fast.so" if fast else "liboracle.so"))
        L = self.lib
        L.orc_rmsnorm_batched.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_rmsnorm_bwd_batched.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int,
                                              C.c_float, C.c_int]
        L.orc_residual.argtypes = [_f32p, _f32p, _f32p, C.c_float, C.c_size_t]
        L.orc_scale.argtypes = [_f32p, _f32p, C.c_float, C.c_size_t]
        L.orc_add.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.orc_swiglu.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.orc_swiglu_bwd.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_size_t]
        L.orc_rope_batched.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int]
        L.orc_qknorm_rope_batched.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                              C.c_float, C.c_float, C.c_int]
        L.orc_rope_qknorm_bwd_batched.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int,
                                                  C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]
        L.orc_qknorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_qknorm_bwd.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float,
                                     C.c_int]
        L.orc_embed_lookup.argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int]
        L.orc_embed_lookup.restype = C.c_int
        L.orc_embed_backward.argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int]
        L.orc_embed_backward.restype = C.c_int
        L.orc_cross_entropy.argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_float, C.POINTER(C.c_int)]
        L.orc_cross_entropy.restype = C.c_float
        L.orc_adam.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t, C.c_int, C.c_float, C.c_float, C.c_float,
                               C.c_float, C.c_float, C.c_int, C.c_float, C.c_float]
        L.orc_grad_norm_sq.argtypes = [_f32p, C.c_size_t, C.c_float]
        L.orc_grad_norm_sq.restype = C.c_double
        L.orc_clip_factor.argtypes = [C.c_float, C.c_float]
        L.orc_clip_factor.restype = C.c_float
        L.orc_vocab_map_build.argtypes = [_i32p, C.c_size_t, C.c_int, _i32p, _i32p]
        L.orc_vocab_map_build.restype = C.c_int
        for name in ("orc_vocab_compact_embed", "orc_vocab_scatter_grads", "orc_vocab_update_full"):
            getattr(L, name).argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int]
            getattr(L, name).restype = None
        for name in ("orc_gqa_tile_kv", "orc_gqa_reduce_kv"):
            getattr(L, name).argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int]
            getattr(L, name).restype = None
        L.orc_cvt_f32_f16.argtypes = [_u16p, _f32p, C.c_size_t]
        L.orc_cvt_f16_f32.argtypes = [_f32p, _u16p, C.c_size_t]
        L.orc_pack_dyn_f16.argtypes = [_u16p, _f32p, C.c_int, C.c_int, _f32p, C.c_int]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_set_chunk.argtypes = [C.c_int]

    # --- norms -----------------------------------------------------------------------
    def rmsnorm(self, x, w, eps=1e-5):
        """x [B,C,S] or [C,S] fp32 -> y same shape."""
        x3 = x.reshape((-1,) + x.shape[-2:])
        out = np.empty_like(x3)
        B, d, S = x3.shape
        self.lib.orc_rmsnorm_batched(_fp(out), _fp(x3), _fp(w), B, d, S, eps)
        return out.reshape(x.shape)

    def rmsnorm_bwd(self, dy, x, w, dw=None, eps=1e-5, exact=False):
        """Returns (dx, dw); dw is accumulated into a copy of the given array (zeros if None)."""
        x3 = x.reshape((-1,) + x.shape[-2:])
        dy3 = dy.reshape(x3.shape)
        B, d, S = x3.shape
        dx = np.zeros_like(x3)
        dwo = np.zeros(d, np.float32) if dw is None else dw.copy()
        self.lib.orc_rmsnorm_bwd_batched(_fp(dx), _fp(dwo), _fp(dy3), _fp(x3), _fp(w), B, d, S, eps, int(exact))
        return dx.reshape(x.shape), dwo

    # --- element-wise ------------------------------------------------------------------
    def residual(self, x, f, alpha):
        out = np.empty_like(x)
        self.lib.orc_residual(_fp(out), _fp(x), _fp(f), alpha, x.size)
        return out

    def scale(self, x, alpha):
        out = np.empty_like(x)
        self.lib.orc_scale(_fp(out), _fp(x), alpha, x.size)
        return out

    def add(self, a, b):
        out = np.empty_like(a)
        self.lib.orc_add(_fp(out), _fp(a), _fp(b), a.size)
        return out

    def swiglu(self, h1, h3):
        out = np.empty_like(h1)
        self.lib.orc_swiglu(_fp(out), _fp(h1), _fp(h3), h1.size)
        return out

    def swiglu_bwd(self, h1, h3, d):
        dh1 = np.empty_like(h1)
        dh3 = np.empty_like(h1)
        self.lib.orc_swiglu_bwd(_fp(dh1), _fp(dh3), _fp(h1), _fp(h3), _fp(d), h1.size)
        return dh1, dh3

    # --- rope / qk-norm ------------------------------------------------------------------
    def rope(self, x, hd, base=10000.0, pos0=0, inverse=False):
        x3 = np.ascontiguousarray(x.reshape((-1,) + x.shape[-2:])).copy()
        B, dim, S = x3.shape
        self.lib.orc_rope_batched(_fp(x3), B, S, dim, hd, base, pos0, int(inverse))
        return x3.reshape(x.shape)

    def qknorm(self, x, w, hd, eps=1e-6):
        x3 = x.reshape((-1,) + x.shape[-2:])
        B, dim, S = x3.shape
        out = np.empty_like(x3)
        for b in range(B):
            self.lib.orc_qknorm(_fp(out[b]), _fp(x3[b]), _fp(w), dim // hd, hd, S, eps)
        return out.reshape(x.shape)

    def qknorm_bwd(self, dy, x, w, hd, dw=None, eps=1e-6, exact=False):
        x3 = x.reshape((-1,) + x.shape[-2:])
        dy3 = dy.reshape(x3.shape)
        B, dim, S = x3.shape
        dx = np.zeros_like(x3)
        dwo = np.zeros(hd, np.float32) if dw is None else dw.copy()
        for b in range(B):
            self.lib.orc_qknorm_bwd(_fp(dx[b]), _fp(dwo), _fp(dy3[b]), _fp(x3[b]), _fp(w), dim // hd, hd, S, eps,
                                    int(exact))
        return dx.reshape(x.shape), dwo

    def qknorm_rope(self, x, w, hd, eps=1e-6, base=1e6, pos0=0):
        x3 = x.reshape((-1,) + x.shape[-2:])
        B, dim, S = x3.shape
        out = np.empty_like(x3)
        self.lib.orc_qknorm_rope_batched(_fp(out), _fp(x3), _fp(w), B, dim // hd, hd, S, eps, base, pos0)
        return out.reshape(x.shape)

    def rope_qknorm_bwd(self, dy, x, w, hd, dw=None, eps=1e-6, base=1e6, pos0=0, exact=False):
        x3 = x.reshape((-1,) + x.shape[-2:])
        dy3 = dy.reshape(x3.shape)
        B, dim, S = x3.shape
        dx = np.zeros_like(x3)
        dwo = np.zeros(hd, np.float32) if dw is None else dw.copy()
        self.lib.orc_rope_qknorm_bwd_batched(_fp(dx), _fp(dwo), _fp(dy3), _fp(x3), _fp(w), B, dim // hd, hd, S,
                                             eps, base, pos0, int(exact))
        return dx.reshape(x.shape), dwo

    # --- embedding -----------------------------------------------------------------------
    def embed_lookup(self, table, tokens, x_init=None):
        """table [V,D] fp32, tokens [B,S] int32 -> x [B,D,S]; returns (x, n_out_of_range)."""
        tok = np.ascontiguousarray(tokens.reshape(-1, tokens.shape[-1]).astype(np.int32))
        B, S = tok.shape
        V, D = table.shape
        x = np.zeros((B, D, S), np.float32) if x_init is None else x_init.reshape(B, D, S).copy()
        oor = 0
        for b in range(B):
            oor += self.lib.orc_embed_lookup(_fp(x[b]), _fp(table), _ip(tok[b]), D, S, V)
        return x, oor

    def embed_backward(self, d_embed, dx, tokens):
        """Accumulates into a copy of d_embed [V,D] in order b=0.., t=0..; returns (dE, n_oor)."""
        tok = np.ascontiguousarray(tokens.reshape(-1, tokens.shape[-1]).astype(np.int32))
        B, S = tok.shape
        V, D = d_embed.shape
        dx3 = dx.reshape(B, D, S)
        out = d_embed.copy()
        oor = 0
        for b in range(B):
            oor += self.lib.orc_embed_backward(_fp(out), _fp(dx3[b]), _ip(tok[b]), D, S, V)
        return out, oor

    # --- loss ------------------------------------------------------------------------------
    def cross_entropy(self, logits, targets, grad_scale=1.0):
        """logits [B,V,S] or [V,S]; returns (loss[B], dlogits, n_oor)."""
        l3 = logits.reshape((-1,) + logits.shape[-2:])
        B, V, S = l3.shape
        tg = np.ascontiguousarray(targets.reshape(B, S).astype(np.int32))
        dl = np.empty_like(l3)
        loss = np.zeros(B, np.float32)
        oor = 0
        for b in range(B):
            n = C.c_int(0)
            loss[b] = self.lib.orc_cross_entropy(_fp(dl[b]), _fp(l3[b]), _ip(tg[b]), V, S, grad_scale, C.byref(n))
            oor += n.value
        return loss, dl.reshape(logits.shape), oor

    # --- optimizer ---------------------------------------------------------------------------
    def adam(self, w, g, m, v, t, lr, b1, b2, eps, wd=0.0, variant=1, gscale=1.0, clip=1.0):
        """In place on w, m, v (flat fp32)."""
        self.lib.orc_adam(_fp(w), _fp(g), _fp(m), _fp(v), w.size, t, lr, b1, b2, eps, wd, variant, gscale, clip)

    def grad_norm_sq(self, g, gscale=1.0):
        return float(self.lib.orc_grad_norm_sq(_fp(g), g.size, gscale))

    def clip_factor(self, norm_sq, clip):
        return float(self.lib.orc_clip_factor(norm_sq, clip))

    # ---- layout helpers (training_dynamic/io.h, cpu_ops.h)
    def vocab_compact_embed(self, full_embed, c2f, cv):
        out = np.empty((cv, full_embed.shape[1]), np.float32)
        self.lib.orc_vocab_compact_embed(_fp(out), _fp(np.ascontiguousarray(full_embed, np.float32)), _ip(c2f), cv, full_embed.shape[1])
        return out

    def vocab_scatter_grads(self, full_g, compact_g, c2f, cv):
        out = np.ascontiguousarray(full_g, np.float32).copy()
        self.lib.orc_vocab_scatter_grads(_fp(out), _fp(np.ascontiguousarray(compact_g, np.float32)), _ip(c2f), cv, full_g.shape[1])
        return out

    def vocab_update_full(self, full_embed, compact_embed, c2f, cv):
        out = np.ascontiguousarray(full_embed, np.float32).copy()
        self.lib.orc_vocab_update_full(_fp(out), _fp(np.ascontiguousarray(compact_embed, np.float32)), _ip(c2f), cv, full_embed.shape[1])
        return out

    def gqa_tile(self, x, kv_heads, ratio):
        """x [B, kv_heads*hd, S] fp32 -> [B, kv_heads*ratio*hd, S]"""
        x = np.ascontiguousarray(x, np.float32)
        B, Cn, S = x.shape
        hd = Cn // kv_heads
        out = np.empty((B, Cn * ratio, S), np.float32)
        for b in range(B):
            self.lib.orc_gqa_tile_kv(_fp(out[b]), _fp(x[b]), kv_heads, ratio, hd, S)
        return out

    def gqa_reduce(self, x, kv_heads, ratio):
        x = np.ascontiguousarray(x, np.float32)
        B, Cn, S = x.shape
        hd = Cn // (kv_heads * ratio)
        out = np.empty((B, kv_heads * hd, S), np.float32)
        for b in range(B):
            self.lib.orc_gqa_reduce_kv(_fp(out[b]), _fp(x[b]), kv_heads, ratio, hd, S)
        return out

    def cvt_f32_f16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.lib.orc_cvt_f32_f16(_up(out), _fp(x), x.size)
        return out.view(np.float16)

    def cvt_f16_f32(self, h):
        h = np.ascontiguousarray(h, np.float16)
        out = np.empty(h.shape, np.float32)
        self.lib.orc_cvt_f16_f32(_fp(out), _up(h.view(np.uint16)), h.size)
        return out

    def pack_dyn(self, act, W):
        act, W = np.ascontiguousarray(act, np.float32), np.ascontiguousarray(W, np.float32)
        ic, seq = act.shape
        oc = W.shape[1]
        out = np.empty((ic, seq + oc), np.uint16)
        self.lib.orc_pack_dyn_f16(_up(out), _fp(act), ic, seq, _fp(W), oc)
        return out.view(np.float16)

    def vocab_map_build(self, data, full_vocab):
        d = np.ascontiguousarray(data.astype(np.int32).ravel())
        f2c = np.empty(full_vocab, np.int32)
        c2f = np.empty(full_vocab, np.int32)
        cv = self.lib.orc_vocab_map_build(_ip(d), d.size, full_vocab, _ip(f2c), _ip(c2f))
        return cv, f2c, c2f[:cv].copy()

    def num_threads(self):
        return int(self.lib.orc_num_threads())

    def set_num_threads(self, n):
        self.lib.orc_set_num_threads(int(n))

    def set_chunk(self, tokens):
        """Timed-baseline work splitting (0 = off, the parity setting); see oracle_ops.c."""
        self.lib.orc_set_chunk(int(tokens))


def reference_available() -> bool:
    return all(os.path.exists(os.path.join(HERE, "_ref", n)) for n in ("libref_stories.so", "libref_dynamic.so"))


def reference_inline_available() -> bool:
    return os.path.exists(os.path.join(HERE, "_ref", "libref_inline.so"))


class LayerGradPtrs(C.Structure):
    """Field order of the LayerGrads stand-in in ref_inline_exports.c.in."""
    _fields_ = [(n, _f32p) for n in ("Wq", "Wk", "Wv", "Wo", "W1", "W2", "W3", "rms_att", "rms_ffn")]


class ReferenceInline:
    """The reference's INLINE operator blocks (statements of training_dynamic/train.m's main()) and the plain-C
    helpers of training/forward.h, compiled by line range into oracle/_ref/libref_inline.so."""

    def __init__(self):
        if not reference_inline_available():
            raise FileNotFoundError("oracle/_ref/libref_inline.so is not built (run oracle/build_oracle.py where the reference is)")
        L = self.lib = C.CDLL(os.path.join(HERE, "_ref", "libref_inline.so"))
        L.ref_inline_residual.argtypes = [_f32p, _f32p, _f32p, C.c_float, C.c_int, C.c_int]
        L.ref_inline_swiglu_bwd.argtypes = [_f32p] * 7 + [C.c_int, C.c_int]
        L.ref_inline_grad_scale_norm_clip.argtypes = [C.POINTER(LayerGradPtrs), C.c_int, _f32p, _f32p] + [C.c_size_t] * 7 + \
            [C.c_int, C.c_int, C.c_float, C.c_float, _f32p]
        L.ref_inline_grad_scale_norm_clip.restype = C.c_float
        L.ref_inline_cpu_rope.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.ref_inline_silu.argtypes = [C.c_float]
        L.ref_inline_silu.restype = C.c_float
        L.ref_inline_swiglu.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]

    def residual(self, x, f, alpha):
        """train.m:460 on one [DIM, SEQ] pair (flat: the statement treats both as SEQ*DIM elements)."""
        out = np.empty_like(x)
        self.lib.ref_inline_residual(_fp(out), _fp(x), _fp(f), alpha, x.shape[-1], x.size // x.shape[-1])
        return out

    def swiglu_bwd(self, h1, h3, dsilu):
        """train.m:538-554 on [HIDDEN, SEQ] arrays -> (dh1, dh3)."""
        dh1, dh3, t1, t2 = (np.empty_like(h1) for _ in range(4))
        self.lib.ref_inline_swiglu_bwd(_fp(dh1), _fp(dh3), _fp(h1), _fp(h3), _fp(dsilu), _fp(t1), _fp(t2), h1.shape[0], h1.shape[1])
        return dh1, dh3

    def swiglu(self, h1, h3):
        """forward.h:149-151 (element-wise, so the row-major statement applies to any layout)."""
        out = np.empty_like(h1)
        self.lib.ref_inline_swiglu(_fp(out), _fp(h1), _fp(h3), 1, h1.size)
        return out

    def rope_channel_first(self, x, hd):
        """forward.h:55-70 (row-major [S][heads*hd], base 10000) applied to a channel-first [C, S] array."""
        Cn, S = x.shape
        q = np.ascontiguousarray(x.T).copy()
        k = q.copy()
        self.lib.ref_inline_cpu_rope(_fp(q), _fp(k), S, Cn // hd, hd)
        assert np.array_equal(q, k)
        return np.ascontiguousarray(q.T)

    def grad_scale_norm_clip(self, layers, grms_final, gembed, gsc, grad_clip):
        """train.m:754-767,770-788,809-825.  layers: list of dicts with the nine LayerGrads fields (Wq..W3 flat fp32 of
        equal per-field sizes across layers, rms_att / rms_ffn of DIM elements); every array is scaled / clipped in
        place.  Returns (grad_norm, grad_norm_sq)."""
        n = len(layers)
        arr = (LayerGradPtrs * n)()
        for i, lay in enumerate(layers):
            for name, _ in LayerGradPtrs._fields_:
                setattr(arr[i], name, _fp(lay[name]))
        sizes = [layers[0][k].size for k in ("Wq", "Wk", "Wv", "Wo", "W1", "W2", "W3")]
        dim = grms_final.size
        nsq = np.zeros(1, np.float32)
        norm = self.lib.ref_inline_grad_scale_norm_clip(arr, n, _fp(grms_final), _fp(gembed), *sizes, dim, gembed.size // dim,
                                                        gsc, grad_clip, _fp(nsq))
        return float(norm), float(nsq[0])


class Reference:
    """The reference's own functions (single sequence, uint16 ids, reference signatures)."""

    def __init__(self, fast: bool = False):
        if not reference_available():
            raise FileNotFoundError("oracle/_ref is not built (run oracle/build_oracle.py where the reference is)")
        suf = "_fast" if fast else ""
        self.st = C.CDLL(os.path.join(HERE, "_ref", f"libref_stories{suf}.so"))
        self.dy = C.CDLL(os.path.join(HERE, "_ref", f"libref_dynamic{suf}.so"))
        for lib, p in ((self.st, "ref_stories_"), (self.dy, "ref_dynamic_")):
            getattr(lib, p + "rmsnorm").argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
            getattr(lib, p + "rmsnorm_bwd").argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int]
            f = getattr(lib, p + "cross_entropy_loss")
            f.argtypes = [_f32p, _f32p, _u16p, C.c_int, C.c_int]
            f.restype = C.c_float
            getattr(lib, p + "embed_lookup").argtypes = [_f32p, _f32p, _u16p, C.c_int, C.c_int]
            getattr(lib, p + "embed_backward").argtypes = [_f32p, _f32p, _u16p, C.c_int, C.c_int]
        self.st.ref_stories_adam_update.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t, C.c_int, C.c_float,
                                                    C.c_float, C.c_float, C.c_float]
        self.dy.ref_dynamic_adam_update.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t, C.c_int, C.c_float,
                                                    C.c_float, C.c_float, C.c_float, C.c_float]
        self.dy.ref_dynamic_rope_backward_inplace.argtypes = [_f32p, C.c_int, C.c_int, C.c_int]
        self.dy.ref_dynamic_vocab_map_build.argtypes = [_u16p, C.c_size_t, C.c_int, _i32p, _i32p]
        self.dy.ref_dynamic_vocab_map_build.restype = C.c_int
        for name in ("ref_dynamic_vocab_compact_embed", "ref_dynamic_vocab_scatter_grads", "ref_dynamic_vocab_update_full"):
            getattr(self.dy, name).argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int]
            getattr(self.dy, name).restype = None
        self.st.ref_stories_set_vocab.argtypes = [C.c_int]

    def _lib(self, variant):
        return (self.st, "ref_stories_") if variant == "stories" else (self.dy, "ref_dynamic_")

    def rmsnorm(self, x, w, variant="stories"):
        lib, p = self._lib(variant)
        out = np.empty_like(x)
        getattr(lib, p + "rmsnorm")(_fp(out), _fp(x), _fp(w), x.shape[0], x.shape[1])
        return out

    def rmsnorm_bwd(self, dy, x, w, dw=None, variant="stories"):
        lib, p = self._lib(variant)
        dx = np.zeros_like(x)
        dwo = np.zeros(x.shape[0], np.float32) if dw is None else dw.copy()
        getattr(lib, p + "rmsnorm_bwd")(_fp(dx), _fp(dwo), _fp(dy), _fp(x), _fp(w), x.shape[0], x.shape[1])
        return dx, dwo

    def cross_entropy_loss(self, logits, targets_u16, variant="stories"):
        lib, p = self._lib(variant)
        dl = np.empty_like(logits)
        loss = getattr(lib, p + "cross_entropy_loss")(_fp(dl), _fp(logits), _up(targets_u16), logits.shape[0],
                                                      logits.shape[1])
        return float(loss), dl

    def embed_lookup(self, table, tokens_u16, variant="stories", x_init=None):
        lib, p = self._lib(variant)
        V, D = table.shape
        if variant == "stories":
            self.st.ref_stories_set_vocab(V)
        S = tokens_u16.size
        x = np.zeros((D, S), np.float32) if x_init is None else x_init.copy()
        getattr(lib, p + "embed_lookup")(_fp(x), _fp(table), _up(tokens_u16), D, S)
        return x

    def embed_backward(self, d_embed, dx, tokens_u16, variant="stories"):
        lib, p = self._lib(variant)
        V, D = d_embed.shape
        if variant == "stories":
            self.st.ref_stories_set_vocab(V)
        out = d_embed.copy()
        getattr(lib, p + "embed_backward")(_fp(out), _fp(dx), _up(tokens_u16), D, tokens_u16.size)
        return out

    def adam_update(self, w, g, m, v, t, lr, b1, b2, eps, wd=None):
        if wd is None:
            self.st.ref_stories_adam_update(_fp(w), _fp(g), _fp(m), _fp(v), w.size, t, lr, b1, b2, eps)
        else:
            self.dy.ref_dynamic_adam_update(_fp(w), _fp(g), _fp(m), _fp(v), w.size, t, lr, b1, b2, eps, wd)

    def rope_backward_inplace(self, dx, hd):
        out = dx.copy()
        self.dy.ref_dynamic_rope_backward_inplace(_fp(out), dx.shape[1], dx.shape[0], hd)
        return out

    def vocab_rows(self, which, a, b, c2f, cv):
        """which in compact_embed / scatter_grads / update_full; a is the destination (copied), b the source."""
        out = np.ascontiguousarray(a, np.float32).copy()
        getattr(self.dy, "ref_dynamic_vocab_" + which)(_fp(out), _fp(np.ascontiguousarray(b, np.float32)), _ip(c2f), cv, b.shape[1])
        return out

    def vocab_map_build(self, data_u16, full_vocab):
        f2c = np.empty(full_vocab, np.int32)
        c2f = np.empty(full_vocab, np.int32)
        cv = self.dy.ref_dynamic_vocab_map_build(_up(data_u16), data_u16.size, full_vocab, _ip(f2c), _ip(c2f))
        return cv, f2c, c2f[:cv].copy()
