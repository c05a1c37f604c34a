"""The layer chain with HOST buffers on the matmul side.

In the reference's training loop the contractions (QKV / output / FFN projections, SDPA, classifier) run on
another engine and hand their results over in host memory (training_dynamic/train.m:430-730); everything between
them is this library's operator set.  `HostLayerChain.step()` is that arrangement end to end: per layer it copies
the contraction outputs host -> device, runs the operators, and copies what the next contraction consumes
device -> host, on three streams so that the copies of one layer overlap the operators of its neighbours.
Tensors that only the operators themselves consume (the residual stream, x2, the running gradient) never leave
the device.

Bytes per token and layer (bf16): 38,912 host -> device (q, k, attention output, h1, h3, FFN output forward;
dsilu, dx_ffn, dq, dk, dx_attn backward), 34,816 device -> host (xnorm, q_rot, k_rot, x2norm, gate forward;
dh1, dh3, dq, dk backward).
"""
from __future__ import annotations

import torch

from .layer_chain import ChainConfig, FlatParams, LayerChain


class HostLayerChain:
    def __init__(self, cfg: ChainConfig, n_seqs: int, params: FlatParams, device, rotate: int = 4):
        self.cfg, self.B, self.device = cfg, n_seqs, device
        self.chain = LayerChain(cfg, n_seqs, params, device, rotate=rotate)
        c, ch = cfg, self.chain
        S = c.seq

        def pin(channels, fill):
            t = torch.empty((n_seqs, channels, S), dtype=c.dtype).pin_memory()
            if fill:
                t.normal_()
            return t

        # one page-locked buffer per tensor kind, shared by all layers (the host side only provides / receives bytes)
        self.h_in_f = {k: pin(n, True) for k, n in (("q", c.q_dim), ("k", c.kv_dim), ("o_out", c.dim), ("h1", c.hidden),
                                                    ("h3", c.hidden), ("ffn_out", c.dim))}
        self.h_out_f = {k: pin(n, False) for k, n in (("xnorm", c.dim), ("q_r", c.q_dim), ("k_r", c.kv_dim), ("x2norm", c.dim),
                                                      ("gate", c.hidden))}
        self.h_in_b = {k: pin(n, True) for k, n in (("dsilu", c.hidden), ("dx_ffn", c.dim), ("dq_in", c.q_dim), ("dk_in", c.kv_dim),
                                                    ("dx_attn", c.dim))}
        self.h_out_b = {k: pin(n, False) for k, n in (("dh1", c.hidden), ("dh3", c.hidden), ("dq", c.q_dim), ("dk", c.kv_dim))}
        self.h_dy_cls = pin(c.dim, True)
        self.h_x_final = pin(c.dim, False)
        self.h_tokens = torch.randint(0, c.vocab, (n_seqs, S), dtype=torch.int32).pin_memory()

        self.s_in, self.s_c, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        L = c.layers
        ev = lambda: torch.cuda.Event()
        self.e_in_f, self.e_c_f, self.e_out_f = [ev() for _ in range(L)], [ev() for _ in range(L)], [ev() for _ in range(L)]
        self.e_in_b, self.e_c_b, self.e_out_b = [ev() for _ in range(L)], [ev() for _ in range(L)], [ev() for _ in range(L)]
        self.e_misc_in, self.e_fwd_done, self.e_step_done = ev(), ev(), ev()
        self._first = True

        e = torch.empty((), dtype=c.dtype).element_size()
        T = n_seqs * S
        per_in = c.q_dim + c.kv_dim + c.dim + 2 * c.hidden + c.dim + c.hidden + c.dim + c.q_dim + c.kv_dim + c.dim
        per_out = c.dim + c.q_dim + c.kv_dim + c.dim + c.hidden + 2 * c.hidden + c.q_dim + c.kv_dim
        self.h2d_bytes_per_step = T * e * (L * per_in + c.dim) + T * 4
        self.d2h_bytes_per_step = T * e * (L * per_out + c.dim)

    def step(self):
        """One forward + backward pass of the chain with every contraction-side tensor crossing the host boundary."""
        c, ch, R = self.cfg, self.chain, self.chain.R
        L = c.layers
        s_in, s_c, s_out = self.s_in, self.s_c, self.s_out
        nb = dict(non_blocking=True)

        # ---- forward
        with torch.cuda.stream(s_in):
            if not self._first:
                s_in.wait_event(self.e_step_done)          # last step's operators still read the per-layer inputs
            ch.tokens.copy_(self.h_tokens, **nb)
            ch.dy_cls.copy_(self.h_dy_cls, **nb)
            self.e_misc_in.record(s_in)
            for l in range(L):
                for k, h in self.h_in_f.items():
                    getattr(ch, k)[l].copy_(h, **nb)
                self.e_in_f[l].record(s_in)
        with torch.cuda.stream(s_c):
            s_c.wait_event(self.e_misc_in)
            ch.fwd_begin()                                  # gather + the first layer's attention norm
            self.e_fwd_done.record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(self.e_fwd_done)
                self.h_out_f["xnorm"].copy_(ch.xnorm[0], **nb)
            for l in range(L):
                s_c.wait_event(self.e_in_f[l])
                if l >= R:
                    s_c.wait_event(self.e_out_f[l - R])    # the rotating outputs of layer l-R have left the device
                ch.fwd_layer(l)
                self.e_c_f[l].record(s_c)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(self.e_c_f[l])
                    r = l % R
                    for k, h in self.h_out_f.items():
                        if k != "xnorm":
                            h.copy_(getattr(ch, k)[r], **nb)
                        elif l + 1 < L:                     # layer l closes with the NEXT layer's attention norm
                            h.copy_(ch.xnorm[(l + 1) % R], **nb)
                    self.e_out_f[l].record(s_out)
            ch.fwd_end()
            self.e_fwd_done.record(s_c)
        with torch.cuda.stream(s_out):
            s_out.wait_event(self.e_fwd_done)
            self.h_x_final.copy_(ch.x_final, **nb)

        # ---- backward (layers in reverse).  One host loop over the layers: an event must have been recorded (host
        # call) before another stream is told to wait for it, or the wait would refer to the previous step's record.
        order = list(range(L - 1, -1, -1))
        with torch.cuda.stream(s_c):
            ch.bwd_begin()
        for i, l in enumerate(order):
            r = l % R
            with torch.cuda.stream(s_in):
                if i >= R:
                    s_in.wait_event(self.e_c_b[order[i - R]])      # the rotating inputs of that layer have been consumed
                for k, h in self.h_in_b.items():
                    getattr(ch, k)[r].copy_(h, **nb)
                self.e_in_b[l].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(self.e_in_b[l])
                if i >= R:
                    s_c.wait_event(self.e_out_b[order[i - R]])     # the rotating outputs of that layer have left the device
                ch.bwd_layer(l)
                self.e_c_b[l].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(self.e_c_b[l])
                for k, h in self.h_out_b.items():
                    h.copy_(getattr(ch, k)[r], **nb)
                self.e_out_b[l].record(s_out)
        with torch.cuda.stream(s_c):
            ch.bwd_end()
            self.e_step_done.record(s_c)
        self._first = False

    def synchronize(self):
        for s in (self.s_in, self.s_c, self.s_out):
            s.synchronize()


class CHostLayerChain:
    """The same step through the C ABI's chain object (ane_cuda_chain_create / _step / _sync, csrc/chain.cu): what a C
    caller of the library uses.  Host buffers, tokens and parameters are taken from a HostLayerChain `like` (same bytes
    in, so the same bytes must come out); only the device buffers, streams and the launch sequence are the library's."""

    def __init__(self, like: HostLayerChain, params: FlatParams):
        import ctypes as C

        from . import lib as _l

        self._l, self._C = _l, C
        c = like.cfg
        self.cfg, self.B, self.like = c, like.B, like
        L = c.layers

        class Config(C.Structure):
            _fields_ = [(n, C.c_int) for n in ("layers", "dim", "hidden", "heads", "kv_heads", "head_dim", "seq", "vocab", "dtype")] + \
                       [(n, C.c_float) for n in ("alpha", "eps", "qk_eps", "rope_base")] + [("norm_bwd_flags", C.c_uint), ("rotate", C.c_int)]

        class Params(C.Structure):
            _fields_ = [(n, C.c_void_p) for n in ("att_w", "ffn_w", "final_w", "q_w", "k_w", "att_g", "ffn_g", "final_g", "q_g", "k_g",
                                                  "table", "embed_g")]

        io_names = ("q", "k", "o_out", "h1", "h3", "ffn_out", "xnorm", "q_r", "k_r", "x2norm", "gate", "dsilu", "dx_ffn", "dq_in", "dk_in",
                    "dx_attn", "dh1", "dh3", "dq", "dk")

        class HostIO(C.Structure):
            _fields_ = [(n, C.POINTER(C.c_void_p)) for n in io_names] + [("dy_cls", C.c_void_p), ("x_final", C.c_void_p), ("tokens", C.c_void_p)]

        dt = {torch.float32: _l.F32, torch.bfloat16: _l.BF16, torch.float16: _l.F16}[c.dtype]
        cfg = Config(c.layers, c.dim, c.hidden, c.heads, c.kv_heads, c.head_dim, c.seq, c.vocab, dt, c.alpha, c.eps, c.qk_eps, c.rope_base,
                     _l.NORM_BWD_EXACT if c.exact_norm_bwd else _l.NORM_BWD_REFERENCE, like.chain.R)
        p = params
        ptr = lambda which, grad: p.norm_w(which, 0, grad=grad).data_ptr()
        par = Params(ptr("att", False), ptr("ffn", False), ptr("final", False), ptr("q", False), ptr("k", False),
                     ptr("att", True), ptr("ffn", True), ptr("final", True), ptr("q", True), ptr("k", True),
                     like.chain.table.data_ptr(), p.embed(grad=True).data_ptr())
        self._keep = (cfg, par)
        self.handle = _l.load().ane_cuda_chain_create(C.byref(cfg), like.B, C.byref(par))
        if not self.handle:
            raise _l.AneCudaError(-1, _l.load().ane_cuda_last_error().decode())
        hosts = {**like.h_in_f, **like.h_out_f, **like.h_in_b, **like.h_out_b}
        self._tables = {n: (C.c_void_p * L)(*([hosts[n].data_ptr()] * L)) for n in io_names}        # one host buffer per kind, all layers
        self.io = HostIO(*[C.cast(self._tables[n], C.POINTER(C.c_void_p)) for n in io_names], like.h_dy_cls.data_ptr(),
                         like.h_x_final.data_ptr(), like.h_tokens.data_ptr())
        self.h2d_bytes_per_step = int(_l.load().ane_cuda_chain_h2d_bytes(self.handle))
        self.d2h_bytes_per_step = int(_l.load().ane_cuda_chain_d2h_bytes(self.handle))

    def step(self):
        self._l.check(self._l.load().ane_cuda_chain_step(self.handle, self._C.byref(self.io)))

    def synchronize(self):
        self._l.check(self._l.load().ane_cuda_chain_sync(self.handle))

    def close(self):
        if self.handle:
            self._l.load().ane_cuda_chain_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
