"""The per-layer non-matmul operator chain of one training step, device-resident.

This is the caller's side of the hot path: the order in which
training/training_dynamic/train.m runs its CPU operators around the ANE matmul kernels
(forward :405-487, backward :513-728, optimizer :748-869), with the Qwen3 additions (per-head
QK-RMSNorm fused with RoPE).  The dense contractions themselves (QKV / Wo / FFN matmuls, SDPA,
classifier) are not part of this library: their outputs are buffers the caller owns, which the
benchmark and the tests pre-fill.

Per micro-batch of M sequences, layer L:

  forward   xnorm        = rmsnorm(layer_in[L], w_att[L])                      train.m:417
            q_r, k_r     = rope(qknorm(q[L])), rope(qknorm(k[L]))              mil_dynamic.h:131-168 (+ QK-norm)
            x2[L], x2n   = residual_rmsnorm(layer_in[L], o_out[L], w_ffn[L])   train.m:460-461
            gate         = swiglu(h1[L], h3[L])                                mil_dynamic.h:264-266
            layer_in[L+1]= residual(x2[L], ffn_out[L])                         mil_dynamic.h:279-283
  backward  dh1, dh3     = swiglu_bwd(h1[L], h3[L], dsilu)                     train.m:537-554
            dx2          = rmsnorm_bwd(dx_ffn, x2[L], w_ffn[L]) + dy           train.m:588-590
            dq, dk       = qknorm_bwd(rope^-1(dq'), q[L]), ... (dk', k[L])     train.m:659-660 (+ QK-norm)
            dy           = rmsnorm_bwd(dx_attn, layer_in[L], w_att[L]) + dx2   train.m:719-721

plus the embedding gather in front (train.m:405), the final RMSNorm forward / backward
(train.m:487,513) and the embedding scatter-add behind (train.m:728).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import dev_ops as ops


@dataclass
class ChainConfig:
    layers: int = 28
    dim: int = 1024
    hidden: int = 3072
    heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    seq: int = 2048
    vocab: int = 151936
    dtype: torch.dtype = torch.bfloat16
    eps: float = 1e-5          # block norms (stories_cpu_ops.h:13)
    qk_eps: float = 1e-6
    rope_base: float = 1e6
    alpha: float = (2.0 * 28) ** -0.5      # train.m:188, 1/sqrt(2*NLAYERS)
    exact_norm_bwd: bool = False
    fuse_layer_boundary: bool = True   # closing residual of a layer fused with the norm that reads it next

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def matrix_params_per_layer(self) -> int:
        d, h = self.dim, self.hidden
        return 2 * self.q_dim * d + 2 * self.kv_dim * d + 3 * h * d

    def bytes_per_token_layer(self) -> int:
        """Algorithmic HBM bytes per token and layer of the chain above (every tensor crosses
        HBM once per operator): forward 2(Qd+KVd) + 4D + 3H + 4D elements (two fused residual + norm
        operators; the first layer's attention norm is counted with the ends), backward
        5H + 4D + 3(Qd+KVd) + 4D elements."""
        e = torch.empty((), dtype=self.dtype).element_size()
        d, h, qk = self.dim, self.hidden, self.q_dim + self.kv_dim
        fwd = 2 * qk + 4 * d + 3 * h + (4 * d if self.fuse_layer_boundary else 5 * d)
        bwd = 5 * h + 4 * d + 3 * qk + 4 * d
        return (fwd + bwd) * e

    def bytes_per_token_ends(self) -> int:
        """Gather (ids + table row + x), the first layer's attention norm fwd (2D), final norm bwd (3D), scatter-add staging
        (read dx once; the d_embed rows are counted per distinct id by the caller)."""
        e = torch.empty((), dtype=self.dtype).element_size()
        return 4 + 2 * self.dim * e + 2 * self.dim * e + 3 * self.dim * e + self.dim * e


class FlatParams:
    """All trainable parameters, their gradients and Adam moments as four flat fp32 buffers.

    Layout: [ per-layer matrices | embedding table | norm weights ].  The first two blocks get
    weight decay, the norm weights do not (train.m:837-869), so the optimizer is two range
    updates.  Gradient views into the flat buffer are handed to the operators that produce
    them (dw of the norms, d_embed of the scatter-add)."""

    @staticmethod
    def padded_count(cfg: ChainConfig, pad_to: int = 1) -> int:
        """Length of each flat buffer for this configuration."""
        n = (cfg.layers * cfg.matrix_params_per_layer() + cfg.vocab * cfg.dim + cfg.layers * 2 * cfg.dim + cfg.dim
             + cfg.layers * 2 * cfg.head_dim)
        return (n + pad_to - 1) // pad_to * pad_to

    def __init__(self, cfg: ChainConfig, device, pad_to: int = 1, wg_buffers=None):
        """wg_buffers: optional pre-allocated (w, g) flat fp32 tensors of the padded length, e.g. peer-addressable
        ones from ane_b200.sharded.symmetric_buffers."""
        c = cfg
        self.cfg = cfg
        self.n_matrix = c.layers * c.matrix_params_per_layer()
        self.n_embed = c.vocab * c.dim
        self.n_decay = self.n_matrix + self.n_embed
        self.n_norm = c.layers * 2 * c.dim + c.dim + c.layers * 2 * c.head_dim
        self.n = self.n_decay + self.n_norm
        self.n_padded = (self.n + pad_to - 1) // pad_to * pad_to
        self.padded_length = self.n_padded
        if wg_buffers is not None:
            self.w, self.g = wg_buffers
            if self.w.numel() != self.n_padded or self.g.numel() != self.n_padded:
                raise ValueError("wg_buffers must hold padded_length elements each")
        else:
            self.w = torch.empty(self.n_padded, dtype=torch.float32, device=device)
            self.g = torch.empty(self.n_padded, dtype=torch.float32, device=device)
        self.m = torch.zeros(self.n_padded, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.n_padded, dtype=torch.float32, device=device)
        o = self.n_decay
        self.off_att = o
        self.off_ffn = o + c.layers * c.dim
        self.off_final = o + 2 * c.layers * c.dim
        self.off_wq = self.off_final + c.dim
        self.off_wk = self.off_wq + c.layers * c.head_dim

    def init_random(self, seed: int = 1234, grad_std: float = 1e-2):
        gen = torch.Generator(device=self.w.device).manual_seed(seed)
        self.w.normal_(0.0, 0.02, generator=gen)
        self.w[self.n_decay:self.n] = 1.0 + 0.02 * torch.randn(self.n_norm, device=self.w.device, generator=gen)
        self.g.normal_(0.0, grad_std, generator=gen)
        if self.n_padded > self.n:
            self.w[self.n:].zero_()
            self.g[self.n:].zero_()

    def _view(self, buf, off, n):
        return buf[off:off + n]

    def norm_w(self, which: str, layer: int = 0, grad: bool = False):
        c = self.cfg
        buf = self.g if grad else self.w
        if which == "att":
            return self._view(buf, self.off_att + layer * c.dim, c.dim)
        if which == "ffn":
            return self._view(buf, self.off_ffn + layer * c.dim, c.dim)
        if which == "final":
            return self._view(buf, self.off_final, c.dim)
        if which == "q":
            return self._view(buf, self.off_wq + layer * c.head_dim, c.head_dim)
        if which == "k":
            return self._view(buf, self.off_wk + layer * c.head_dim, c.head_dim)
        raise KeyError(which)

    def embed(self, grad: bool = False):
        c = self.cfg
        buf = self.g if grad else self.w
        return self._view(buf, self.n_matrix, self.n_embed).view(c.vocab, c.dim)

    def zero_produced_grads(self):
        """Clear the gradients this library's operators accumulate into (train.m:874-877)."""
        from . import lib as _l
        part = self.g[self.n_matrix:self.n]
        _l.check(_l.load().ane_cuda_zero_dev(torch.cuda.current_stream().cuda_stream, part.data_ptr(), part.numel() * 4))


class LayerChain:
    """Buffers and launch order for one micro-batch of M sequences on one GPU."""

    def __init__(self, cfg: ChainConfig, micro_batch: int, params: FlatParams, device, rotate: int = 3, seed: int = 1):
        self.cfg, self.M, self.p, self.device = cfg, micro_batch, params, device
        c, M = cfg, micro_batch
        gen = torch.Generator(device=device).manual_seed(seed)

        def rnd(ch, std=1.0):
            t = torch.empty((M, ch, c.seq), dtype=c.dtype, device=device)
            t.normal_(0.0, std, generator=gen)
            return t

        def emp(ch):
            return torch.empty((M, ch, c.seq), dtype=c.dtype, device=device)

        L = c.layers
        # the embedding table in activation dtype (the reference gathers from the fp32 master; the
        # bf16 copy is what a mixed-precision loop keeps resident)
        self.table = torch.empty((c.vocab, c.dim), dtype=c.dtype, device=device).normal_(0.0, 0.02, generator=gen)
        self.tokens = torch.randint(0, c.vocab, (M, c.seq), device=device, dtype=torch.int32, generator=gen)
        # saved per layer: produced by this chain
        self.layer_in = [emp(c.dim) for _ in range(L + 1)]
        self.x2 = [emp(c.dim) for _ in range(L)]
        # per layer, stand-ins for matmul / SDPA outputs of the forward pass
        self.q = [rnd(c.q_dim) for _ in range(L)]
        self.k = [rnd(c.kv_dim) for _ in range(L)]
        self.o_out = [rnd(c.dim) for _ in range(L)]
        self.h1 = [rnd(c.hidden) for _ in range(L)]
        self.h3 = [rnd(c.hidden) for _ in range(L)]
        self.ffn_out = [rnd(c.dim) for _ in range(L)]
        # rotating sets: operator outputs that feed matmuls, and matmul outputs of the backward pass
        self.R = rotate
        self.xnorm = [emp(c.dim) for _ in range(rotate)]
        self.q_r = [emp(c.q_dim) for _ in range(rotate)]
        self.k_r = [emp(c.kv_dim) for _ in range(rotate)]
        self.x2norm = [emp(c.dim) for _ in range(rotate)]
        self.gate = [emp(c.hidden) for _ in range(rotate)]
        self.dsilu = [rnd(c.hidden) for _ in range(rotate)]
        self.dx_ffn = [rnd(c.dim) for _ in range(rotate)]
        self.dq_in = [rnd(c.q_dim) for _ in range(rotate)]
        self.dk_in = [rnd(c.kv_dim) for _ in range(rotate)]
        self.dx_attn = [rnd(c.dim) for _ in range(rotate)]
        self.dh1 = [emp(c.hidden) for _ in range(rotate)]
        self.dh3 = [emp(c.hidden) for _ in range(rotate)]
        self.dq = [emp(c.q_dim) for _ in range(rotate)]
        self.dk = [emp(c.kv_dim) for _ in range(rotate)]
        self.x_final = emp(c.dim)
        self.dy_cls = rnd(c.dim)          # classifier backward output (train.m:501)
        self.dy = [emp(c.dim), emp(c.dim)]
        self.dx2 = emp(c.dim)
        self.timed_op = None              # (name, list of (start, end) events) filled when tracing one operator

    def tokens_per_microbatch(self) -> int:
        return self.M * self.cfg.seq

    def _maybe_time(self, name, fn):
        if self.timed_op is not None and self.timed_op[0] == name:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn()
            e.record()
            self.timed_op[1].append((s, e))
            return r
        return fn()

    def fwd_layer(self, L):
        """Operators of layer L.  xnorm of this layer was produced by the previous layer's closing fused
        residual + RMSNorm (by fwd_begin for layer 0): the residual stream crosses HBM once between layers."""
        c, p = self.cfg, self.p
        r = L % self.R
        x = self.layer_in[L]
        # Q and K in one call: the two launches share the GPU instead of following each other
        ops.qknorm_rope_pair(self.q[L], self.k[L], p.norm_w("q", L), p.norm_w("k", L), c.head_dim, c.qk_eps, c.rope_base, 0,
                             out_q=self.q_r[r], out_k=self.k_r[r])
        ops.residual_rmsnorm(x, self.o_out[L], p.norm_w("ffn", L), c.alpha, c.eps, x2=self.x2[L], x2norm=self.x2norm[r])
        ops.swiglu(self.h1[L], self.h3[L], out=self.gate[r])
        # x_next = x2 + alpha*ffn (train.m:497) fused with the norm that reads it next: the next layer's attention
        # norm, or the final norm after the last layer
        w_next = p.norm_w("att", L + 1) if L + 1 < c.layers else p.norm_w("final")
        n_next = self.xnorm[(L + 1) % self.R] if L + 1 < c.layers else self.x_final
        if c.fuse_layer_boundary:
            ops.residual_rmsnorm(self.x2[L], self.ffn_out[L], w_next, c.alpha, c.eps, x2=self.layer_in[L + 1], x2norm=n_next)
        else:
            ops.residual(self.x2[L], self.ffn_out[L], c.alpha, out=self.layer_in[L + 1])
            ops.rmsnorm(self.layer_in[L + 1], w_next, c.eps, out=n_next)

    def fwd_begin(self):
        c, p = self.cfg, self.p
        ops.embed_lookup(self.table, self.tokens, out=self.layer_in[0])
        ops.rmsnorm(self.layer_in[0], p.norm_w("att", 0), c.eps, out=self.xnorm[0])

    def fwd_end(self):
        pass

    def forward(self):
        self.fwd_begin()
        for L in range(self.cfg.layers):
            self.fwd_layer(L)
        self.fwd_end()

    def bwd_begin(self):
        c, p = self.cfg, self.p
        self._cur = 0
        self._dy = self.dy[0]
        ops.rmsnorm_bwd(self.dy_cls, self.layer_in[c.layers], p.norm_w("final"), p.norm_w("final", grad=True), eps=c.eps,
                        exact=c.exact_norm_bwd, out=self._dy)

    def bwd_layer(self, L):
        c, p = self.cfg, self.p
        ex = c.exact_norm_bwd
        r = L % self.R
        dy = self._dy
        self._maybe_time("swiglu_bwd", lambda: ops.swiglu_bwd(self.h1[L], self.h3[L], self.dsilu[r], dh1=self.dh1[r], dh3=self.dh3[r]))
        ops.rmsnorm_bwd(self.dx_ffn[r], self.x2[L], p.norm_w("ffn", L), p.norm_w("ffn", L, grad=True), add=dy, eps=c.eps,
                        exact=ex, out=self.dx2)
        ops.rope_qknorm_bwd_pair(self.dq_in[r], self.dk_in[r], self.q[L], self.k[L], p.norm_w("q", L), p.norm_w("k", L),
                                 p.norm_w("q", L, grad=True), p.norm_w("k", L, grad=True), c.head_dim, c.qk_eps, c.rope_base, 0,
                                 exact=ex, out_q=self.dq[r], out_k=self.dk[r])
        nxt = self.dy[1 - self._cur]
        ops.rmsnorm_bwd(self.dx_attn[r], self.layer_in[L], p.norm_w("att", L), p.norm_w("att", L, grad=True), add=self.dx2,
                        eps=c.eps, exact=ex, out=nxt)
        self._dy, self._cur = nxt, 1 - self._cur

    def bwd_end(self):
        ops.embed_backward(self.p.embed(grad=True), self._dy, self.tokens)
        self.dy_out = self._dy

    def backward(self):
        self.bwd_begin()
        for L in range(self.cfg.layers - 1, -1, -1):
            self.bwd_layer(L)
        self.bwd_end()

    # ------------------------------------------------------------------ CUDA graph replay
    def capture(self):
        """Record forward() + backward() of one micro-batch into a CUDA graph.  The operator
        chain is a fixed sequence of a few hundred short kernels, so replaying it as a graph removes
        the per-launch host cost and most of the gap between kernels.  One eager pass runs first so
        that the library's scratch range has reached its final size (no allocation may happen while
        a stream is being captured)."""
        from . import lib as _lib
        before = _lib.launch_count()
        self.forward()
        self.backward()
        self.launches_measured = _lib.launch_count() - before
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward()
            self.backward()
        self.graph = g
        return g

    def replay(self):
        self.graph.replay()

    def launches_per_microbatch(self) -> int:
        """Kernels of this library launched by forward() + backward() (counted during capture())."""
        return getattr(self, "launches_measured", 0)

    # ------------------------------------------------------------------ backward in segments (gradient exchange beside it)
    def layer_groups(self, n_groups: int):
        """The layers split into n_groups contiguous groups, in the order the backward pass finishes them:
        [(hi, lo), ...] with hi >= lo, first the top layers."""
        L = self.cfg.layers
        n_groups = max(1, min(n_groups, L))
        edges = [round(i * L / n_groups) for i in range(n_groups + 1)]
        return [(edges[i + 1] - 1, edges[i]) for i in range(n_groups - 1, -1, -1)]

    def run_segment(self, groups, i):
        """Segment i of a micro-batch launched from the host: segment 0 is the forward pass, the final norm's backward and
        the backward of the first (top) group of layers; the last segment ends with the embedding scatter-add."""
        if i == 0:
            self.forward()
            self.bwd_begin()
        hi, lo = groups[i]
        for L in range(hi, lo - 1, -1):
            self.bwd_layer(L)
        if i == len(groups) - 1:
            self.bwd_end()

    def capture_segments(self, n_groups: int):
        """The same micro-batch as capture(), recorded as one CUDA graph per group of layers of the backward pass, so that
        the caller can start exchanging a group's weight gradients (on another stream) as soon as the group is done --
        what a data-parallel loop does while the rest of the backward pass runs.  capture() must have run before (it sizes the
        library's scratch)."""
        groups = self.layer_groups(n_groups)
        torch.cuda.synchronize()
        graphs = []
        for i in range(len(groups)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.run_segment(groups, i)
            graphs.append(g)
        self.segment_groups, self.segment_graphs = groups, graphs
        return groups
