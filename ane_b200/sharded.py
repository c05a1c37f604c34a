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

    def flush(self):
        """Nothing is deferred in this form."""

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


class RegionShardedAdam:
    """The peer-memory optimizer step with the gradient exchange spread over the backward pass.

    The flat parameter space is cut into REGIONS at `boundaries` (for the layer chain: groups of layers in the order the
    backward pass finishes them, then the embedding and norm weights), and every rank owns the same fraction of EVERY
    region instead of one contiguous slice.  As soon as a rank's backward pass has finished a group of layers, the rank
    PUSHES its gradients of that region to their owners: one copy per peer into the owner's staging buffer, issued on a
    side stream and carried out by the copy engines over NVLink -- no SM is taken from the operator chain (whose
    persistent kernels assume they have the GPU to themselves: a reduce KERNEL resident beside them, even on 32 blocks,
    was measured to slow the chain by more than it saved), and no rank waits for another during the chain.  At the end of
    the step one rank sync says that every push has landed; the owner then adds the staged copies and its own gradients
    in rank order from LOCAL memory (HBM speed instead of NVLink speed), pulls only the regions that were never pushed
    (the last layer group, embedding, norm weights) through the peer-reading reduce kernel, and goes on as ShardedAdam's
    peer form does: norm, clip factor, Adam with the stores to every rank.  Per element the arithmetic is the same as
    there; the squared norm is summed region by region, so the clip factor can differ in the last bit."""

    def __init__(self, w, g, m, v, n_decay: int, n_params: int, world: int, rank: int, peer_ptrs, boundaries, group=None,
                 lr: float = 3e-4, b1: float = 0.9, b2: float = 0.95, eps: float = 1e-8, wd: float = 0.1, clip: float = 1.0,
                 kernels=None, staging=None, deferred_broadcast: bool = False):
        """staging = (tensor, ptrs): a peer-addressable fp32 buffer of staging_floats(...) elements on every rank and the
        device addresses of all ranks' copies (symmetric_buffer); None: nothing can be pushed, every region is pulled.
        deferred_broadcast: Adam writes the new weights of the owned parts to LOCAL memory only and the copy engines carry
        them to the peers afterwards: the range without weight decay (the norm weights, which the operator chain reads from
        its first kernel on) at once, confirmed by the closing rank sync; everything else (matrices, embedding table: read by
        the contractions, layer by layer, not by this library) on the side stream, beside the next step's operator chain,
        confirmed by the NEXT step's first rank sync -- or by flush().  A full training loop would issue these copies in
        layer order and let each layer's contraction wait for its own event; here nothing consumes them before the next
        optimizer step."""
        if world < 2 or peer_ptrs is None:
            raise ValueError("RegionShardedAdam needs two or more ranks with peer-mapped buffers")
        b = list(boundaries)
        if b[0] != 0 or b[-1] != w.numel() or any(y <= x for x, y in zip(b, b[1:])):
            raise ValueError("boundaries must rise from 0 to the length of the flat buffers")
        if any((y - x) % (world * 4) for x, y in zip(b, b[1:])):
            raise ValueError("every region must split into `world` parts of a multiple of four floats")
        self.w, self.g, self.m, self.v = w, g, m, v
        self.n_decay, self.n_params = n_decay, n_params
        self.world, self.rank, self.group = world, rank, group
        self.lr, self.b1, self.b2, self.eps, self.wd, self.clip = lr, b1, b2, eps, wd, clip
        self.peer_ptrs = peer_ptrs
        self.bounds = b
        self.part_len = [(y - x) // world for x, y in zip(b, b[1:])]
        self.parts = self.partition(b, world, rank)
        self.offsets = [0]
        for n in self.part_len:
            self.offsets.append(self.offsets[-1] + n)
        if kernels is None:
            from . import dev_ops as kernels  # noqa: WPS433
        self.k = kernels
        dev = g.device
        self.g_slice = torch.empty(self.offsets[-1], dtype=g.dtype, device=dev)
        self._normsq = torch.zeros(len(self.parts), dtype=torch.float32, device=dev)
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        self._side = torch.cuda.Stream(device=dev)
        self._events, self._pushed = [], set()
        self.deferred_broadcast = deferred_broadcast
        self._bcast_done = None
        self.staging = staging
        if staging is not None and staging[0].numel() < self.staging_floats(b, world):
            raise ValueError("the staging buffer is too small for these regions")
        self.normsq = None
        self.phase_events = None
        self.lo, self.hi = self.parts[0]          # for callers that only report a range

    _mark = ShardedAdam._mark

    @staticmethod
    def partition(boundaries, world: int, rank: int):
        """The ranges rank `rank` owns: part `rank` of `world` equal parts of every region."""
        return [(x + rank * ((y - x) // world), x + (rank + 1) * ((y - x) // world)) for x, y in zip(boundaries, boundaries[1:])]

    @staticmethod
    def staging_floats(boundaries, world: int) -> int:
        """Floats of staging every rank needs: one slot per peer, each holding this rank's part of every region."""
        return (world - 1) * sum((y - x) // world for x, y in zip(boundaries, boundaries[1:]))

    def owned_ranges(self):
        return list(self.parts)

    def begin_step(self, gscale: float = 1.0):
        self._events, self._pushed = [], set()

    def _slot(self, src: int, owner: int) -> int:
        """Slot of rank `src` in rank `owner`'s staging buffer."""
        return src if src < owner else src - 1

    def push_region(self, i: int, after: "torch.cuda.Event"):
        """This rank's gradients of region i are complete on its compute stream (`after` = an event recorded there): copy
        each peer's part of the region into that peer's staging buffer, on the side stream."""
        if self.staging is None:
            raise ValueError("no staging buffer was given")
        from . import lib as _l
        L = _l.load()
        _, st_ptrs = self.staging
        x, n = self.bounds[i], self.part_len[i]
        g_base = self.g.data_ptr()
        with torch.cuda.stream(self._side):
            self._side.wait_event(after)
            sid = self._side.cuda_stream
            for owner in range(self.world):
                if owner == self.rank:
                    continue
                dst = st_ptrs[owner] + 4 * (self._slot(self.rank, owner) * self.offsets[-1] + self.offsets[i])
                _l.check(L.ane_cuda_copy_dev(sid, dst, g_base + 4 * (x + owner * n), 4 * n))
            ev = torch.cuda.Event()
            ev.record(self._side)
        self._events.append(ev)
        self._pushed.add(i)

    reduce_region = push_region

    def step(self, t: int, gscale: float = 1.0):
        return self._mark("peer_memory_step", lambda: self._step(t, gscale))

    def _step(self, t: int, gscale: float):
        w_ptrs, g_ptrs = self.peer_ptrs
        cur = torch.cuda.current_stream()
        for ev in self._events:
            cur.wait_event(ev)
        if self._bcast_done is not None:        # this rank's weight copies of the last step: landed before the sync below says so
            cur.wait_event(self._bcast_done)
            self._bcast_done = None
        # every rank's gradients are complete and every push has landed
        self._mark("peer.sync_gradients_complete", lambda: dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.group))

        def reduce_all():
            for i, (a, e) in enumerate(self.parts):
                gs = self.g_slice[self.offsets[i]:self.offsets[i + 1]]
                if i in self._pushed:      # the peers' copies are in this rank's staging buffer: a local sum, in rank order
                    mine = self.staging[0].data_ptr()
                    ptrs = [self.g.data_ptr() if r == self.rank
                            else mine + 4 * (self._slot(r, self.rank) * self.offsets[-1] + self.offsets[i] - a) for r in range(self.world)]
                    self.k.p2p_reduce(ptrs, a, e - a, gs, gscale, normsq=self._normsq[i:i + 1])
                else:
                    self.k.p2p_reduce(g_ptrs, a, e - a, gs, gscale, normsq=self._normsq[i:i + 1])

        self._mark("peer.reduce", reduce_all)
        self._mark("peer.allreduce_norm", lambda: dist.all_reduce(self._normsq, op=dist.ReduceOp.SUM, group=self.group))
        self.normsq = self._normsq.sum().reshape(1)
        factor = self.k.clip_factor(self._normsq, self.clip)

        deferred = self.deferred_broadcast
        later = []                               # (a, b) ranges whose copies to the peers run beside the next step

        def update():
            targets, me = ([self.w.data_ptr()], 0) if deferred else (w_ptrs, self.rank)
            for i, (pa, pe) in enumerate(self.parts):
                for lo, hi, wd in ((0, self.n_decay, self.wd), (self.n_decay, self.n_params, 0.0)):
                    a, b = max(lo, pa), min(hi, pe)
                    if a < b:
                        off = self.offsets[i] + (a - pa)
                        self.k.p2p_adam(targets, me, a, b - a, self.g_slice[off:off + (b - a)], self.m[a:b], self.v[a:b], t, self.lr,
                                        self.b1, self.b2, self.eps, wd=wd, gscale=gscale, clip=factor)
                        if deferred:
                            if wd == 0.0:
                                self._copy_to_peers(cur, a, b)       # norm weights: needed by the next step's first operator
                            else:
                                later.append((a, b))

        self._mark("peer.adam_store_all" if not deferred else "peer.adam_local_and_norm_weights", update)
        if later:
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self._side):
                self._side.wait_event(done)
                for a, b in later:
                    self._copy_to_peers(self._side, a, b)
                self._bcast_done = torch.cuda.Event()
                self._bcast_done.record(self._side)
        self._mark("peer.sync_parameters_landed", lambda: dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.group))
        self._events, self._pushed = [], set()
        return factor

    def _copy_to_peers(self, stream, a: int, b: int):
        from . import lib as _l
        L = _l.load()
        w_ptrs, _ = self.peer_ptrs
        src = self.w.data_ptr() + 4 * a
        for r in range(self.world):
            if r != self.rank:
                _l.check(L.ane_cuda_copy_dev(stream.cuda_stream, w_ptrs[r] + 4 * a, src, 4 * (b - a)))

    def flush(self):
        """Ends with every rank's deferred weight copies landed everywhere (a rank sync on the current stream)."""
        if self._bcast_done is not None:
            torch.cuda.current_stream().wait_event(self._bcast_done)
            self._bcast_done = None
            dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.group)


def allreduce_scalar_sum(x: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Sum of a small tensor over the ranks (the loss all-reduce of a data-parallel step)."""
    if world > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x


def symmetric_buffer(n: int, device, group=None):
    """One flat fp32 buffer of n elements that every rank of the group can address, and the device addresses of all
    ranks' copies: (tensor, ptrs)."""
    import torch.distributed._symmetric_memory as symm

    group = group if group is not None else dist.group.WORLD
    t = symm.empty(n, dtype=torch.float32, device=device)
    try:
        h = symm.rendezvous(t, group=group)
    except TypeError:
        h = symm.rendezvous(t, group.group_name)
    return t, [int(p) for p in h.buffer_ptrs]


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
