"""Token sharding and the collectives around the operator chain (one process per GPU).

Every operator of the chain is independent per token (per sequence for RoPE positions), so the
sequences of a step are split contiguously over the ranks and no collective runs inside the
layer loop.  The exchanges are the ones a data-parallel step needs:

* gradients: one reduce-scatter (sum) over the flat fp32 gradient buffer -- it carries the
  embedding gradient and the norm-weight gradients produced by this library together with the
  matmul gradients the caller produced;
* the squared gradient norm: one scalar all-reduce, so that every rank clips with the same factor
  (train.m:770-825);
* parameters: Adam runs on the rank's 1/N slice of (w, m, v) and the updated slices are
  all-gathered.

``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) is the transport.  The reduction
order inside NCCL is fixed for a given world size, so results are reproducible run to run; they
agree with the single-GPU result to fp32 rounding, not bit for bit.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_items: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of range(n_items): the first n_items % world ranks get one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def padded_length(n: int, world: int, align: int = 256) -> int:
    """Length of a flat buffer that splits into `world` equal slices of a multiple of `align`."""
    q = world * align
    return (n + q - 1) // q * q


class ShardedAdam:
    """ZeRO-1 style optimizer step over FlatParams-like flat buffers.

    ``kernels`` supplies grad_norm_sq(g, gscale) -> 1-element tensor, clip_factor(normsq, clip)
    -> 1-element tensor and adam(w, g, m, v, t, lr, b1, b2, eps, wd=, gscale=, clip=); the default
    is this library's device operators.  The CPU tests pass stand-ins to exercise the collective
    choreography without a GPU."""

    def __init__(self, w, g, m, v, n_decay: int, n_params: int, world: int = 1, rank: int = 0, group=None,
                 lr: float = 3e-4, b1: float = 0.9, b2: float = 0.95, eps: float = 1e-8, wd: float = 0.1,
                 clip: float = 1.0, kernels=None, peer_ptrs=None, n_early: int = 0):
        """peer_ptrs = (w_ptrs, g_ptrs): device addresses of every rank's flat parameter and gradient buffer, mapped
        into this process (see symmetric_buffers).  With them the reduce-scatter and the all-gather are not separate
        collectives: the reduce kernel reads the peers' gradients and the Adam kernel writes the peers' parameters.
        n_early: gradients [0, n_early) are complete when begin_step() is called (the caller's matmul gradients, as
        opposed to the embedding and norm-weight gradients the operator chain produces during the step); in peer mode
        their part of the reduce then runs on a side stream beside the chain.  Off by default: measured on 2 and 8
        B200s it shortens the optimizer phase but lengthens the whole step, because the operator chain it runs beside is
        HBM-bound and pays for the bytes the side stream reads."""
        if w.numel() % world:
            raise ValueError("flat buffers must be padded to a multiple of the world size (see padded_length)")
        self.w, self.g, self.m, self.v = w, g, m, v
        self.n_decay, self.n_params = n_decay, n_params
        self.world, self.rank, self.group = world, rank, group
        self.lr, self.b1, self.b2, self.eps, self.wd, self.clip = lr, b1, b2, eps, wd, clip
        self.slice_len = w.numel() // world
        self.lo = rank * self.slice_len
        self.hi = self.lo + self.slice_len
        if kernels is None:
            from . import dev_ops as kernels  # noqa: WPS433
        self.k = kernels
        self.g_slice = torch.empty(self.slice_len, dtype=g.dtype, device=g.device) if world > 1 else None
        self.normsq = None
        self.peer_ptrs = peer_ptrs if world > 1 else None
        self._token = torch.zeros(1, dtype=torch.float32, device=g.device) if self.peer_ptrs else None
        self.n_early = n_early if self.peer_ptrs else 0
        self._early = None            # (event, end of the range already reduced) of the step in flight
        if self.peer_ptrs:
            self._side = torch.cuda.Stream(device=g.device)
            self._normsq2 = torch.zeros(2, dtype=torch.float32, device=g.device)
            self._token2 = torch.zeros(1, dtype=torch.float32, device=g.device)
            self._scratch = torch.zeros(1184, dtype=torch.float32, device=g.device)   # block partials of the side-stream reduce
        self.phase_events = None      # set to [] to collect (name, start, end) CUDA events of the next steps

    def _reduce_scatter(self):
        if self.world == 1:
            return self.g[self.lo:self.hi]
        if dist.get_backend(self.group) == "gloo":      # gloo has no reduce-scatter
            dist.all_reduce(self.g, op=dist.ReduceOp.SUM, group=self.group)
            self.g_slice.copy_(self.g[self.lo:self.hi])
        else:
            dist.reduce_scatter_tensor(self.g_slice, self.g, op=dist.ReduceOp.SUM, group=self.group)
        return self.g_slice

    def _mark(self, name, fn):
        if self.phase_events is None or not self.g.is_cuda:
            return fn()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        r = fn()
        e.record()
        self.phase_events.append((name, s, e))
        return r

    def step(self, t: int, gscale: float = 1.0):
        if self.peer_ptrs:
            return self._mark("peer_memory_step", lambda: self._step_peer(t, gscale))
        gs = self._mark("reduce_scatter", self._reduce_scatter)
        return self._mark("norm_clip_adam_gather", lambda: self._update(gs, t, gscale))

    def _rank_sync(self):
        """Stream-ordered meeting point of all ranks: a one-element all-reduce completes on a rank only after every
        rank has reached it on its stream, i.e. after everything each of them enqueued before it."""
        dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.group)

    def begin_step(self, gscale: float = 1.0):
        """Peer mode with n_early > 0: start reducing the part of this rank's slice whose gradients are already complete,
        on a side stream, so that it overlaps the operator chain.  Every rank must call it (it contains a collective)."""
        if not self.peer_ptrs or self.n_early <= 0:
            return
        w_ptrs, g_ptrs = self.peer_ptrs
        a, b = self.lo, min(self.hi, self.n_early)
        cur = torch.cuda.current_stream()
        self._side.wait_stream(cur)
        with torch.cuda.stream(self._side):
            dist.all_reduce(self._token2, op=dist.ReduceOp.SUM, group=self.group)      # all ranks' early gradients are in place
            self._normsq2.zero_()
            if a < b:
                self.k.p2p_reduce(g_ptrs, a, b - a, self.g_slice[:b - a], gscale, normsq=self._normsq2[0:1], scratch=self._scratch)
            ev = torch.cuda.Event()
            ev.record(self._side)
        self._early = (ev, max(a, b), gscale)

    def _step_peer(self, t: int, gscale: float):
        w_ptrs, g_ptrs = self.peer_ptrs
        start = self.lo
        if self._early is not None:
            ev, start, gs0 = self._early
            if gs0 != gscale:
                raise ValueError("begin_step and step must use the same gscale")
            torch.cuda.current_stream().wait_event(ev)
            self._early = None
        else:
            self._normsq2.zero_()
        self._mark("peer.sync_gradients_complete", self._rank_sync)     # every rank's gradients are complete
        if start < self.hi:
            self._mark("peer.reduce", lambda: self.k.p2p_reduce(g_ptrs, start, self.hi - start, self.g_slice[start - self.lo:], gscale,
                                                                  normsq=self._normsq2[1:2]))
        # the squared norm; also: every rank has finished reading gradients
        self._mark("peer.allreduce_norm", lambda: dist.all_reduce(self._normsq2, op=dist.ReduceOp.SUM, group=self.group))
        normsq = self._normsq2.sum().reshape(1)
        self.normsq = normsq
        factor = self.k.clip_factor(self._normsq2, self.clip)

        def update():
            for lo, hi, wd in ((0, self.n_decay, self.wd), (self.n_decay, self.n_params, 0.0)):
                a, b = max(lo, self.lo), min(hi, self.hi)
                if a < b:
                    sl = slice(a, b)
                    gl = slice(a - self.lo, b - self.lo)
                    self.k.p2p_adam(w_ptrs, self.rank, a, b - a, self.g_slice[gl], self.m[sl], self.v[sl], t, self.lr, self.b1, self.b2,
                                    self.eps, wd=wd, gscale=gscale, clip=factor)

        self._mark("peer.adam_store_all", update)
        self._mark("peer.sync_parameters_landed", self._rank_sync)      # every rank's parameter stores have landed
        return factor

    def _update(self, gs, t: int, gscale: float):
        normsq = self.k.grad_norm_sq(gs, gscale)
        if self.world > 1:
            dist.all_reduce(normsq, op=dist.ReduceOp.SUM, group=self.group)
        self.normsq = normsq
        factor = self.k.clip_factor(normsq, self.clip)
        # slice ∩ [0, n_decay): weight decay; slice ∩ [n_decay, n_params): none (train.m:837-869)
        for lo, hi, wd in ((0, self.n_decay, self.wd), (self.n_decay, self.n_params, 0.0)):
            a, b = max(lo, self.lo), min(hi, self.hi)
            if a < b:
                sl = slice(a, b)
                gl = slice(a - self.lo, b - self.lo)
                self.k.adam(self.w[sl], gs[gl], self.m[sl], self.v[sl], t, self.lr, self.b1, self.b2, self.eps,
                            wd=wd, gscale=gscale, clip=factor)
        if self.world > 1:
            self._mark("all_gather", lambda: dist.all_gather_into_tensor(
                self.w, self.w[self.lo:self.hi].clone() if dist.get_backend(self.group) == "gloo" else self.w[self.lo:self.hi],
                group=self.group))
        return factor


def allreduce_scalar_sum(x: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Sum of a small tensor over the ranks (the loss all-reduce of a data-parallel step)."""
    if world > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x


def symmetric_buffers(n: int, device, group=None):
    """Two flat fp32 buffers of n elements (parameters, gradients) that every rank of the group can address directly,
    and the device addresses of all ranks' copies: (w, g, (w_ptrs, g_ptrs)).  Uses torch's symmetric memory (CUDA
    IPC over NVLink on one node).  Raises if the ranks cannot map each other's memory; callers fall back to plain
    buffers and NCCL collectives."""
    import torch.distributed._symmetric_memory as symm

    group = group if group is not None else dist.group.WORLD
    out, ptrs = [], []
    for _ in range(2):
        t = symm.empty(n, dtype=torch.float32, device=device)
        try:
            h = symm.rendezvous(t, group=group)
        except TypeError:
            h = symm.rendezvous(t, group.group_name)
        out.append(t)
        ptrs.append([int(p) for p in h.buffer_ptrs])
    return out[0], out[1], (ptrs[0], ptrs[1])
