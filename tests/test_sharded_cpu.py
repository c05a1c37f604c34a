"""CPU tests of the multi-GPU host logic: sequence sharding and the sharded optimizer step,
run as two gloo ranks.  The Adam / norm kernels are replaced by the CPU oracle here (this file
has no GPU), so what is under test is the collective choreography of ane_b200.sharded: the
reduce-scatter of gradients, the scalar all-reduce of the squared norm, the per-slice update
with and without weight decay, and the all-gather of parameters."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ane_b200.sharded import ShardedAdam, padded_length, shard_range
from tests.golden import gen_inputs as gi


def test_shard_range_partitions_exactly():
    for n in (256, 257, 7, 1, 0, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)
    assert padded_length(1000, 8) == 2048 and padded_length(2048, 8) == 2048


class OracleKernels:
    """Stand-ins with the signatures of ane_b200.dev_ops, computed by the CPU oracle."""

    def __init__(self):
        from oracle.oracle import Oracle
        self.o = Oracle()

    def grad_norm_sq(self, g, gscale=1.0):
        return torch.tensor([self.o.grad_norm_sq(g.numpy(), gscale)], dtype=torch.float32)

    def clip_factor(self, normsq, clip):
        return torch.tensor([self.o.clip_factor(float(normsq[0]), clip)], dtype=torch.float32)

    def adam(self, w, g, m, v, t, lr, b1, b2, eps, wd=0.0, gscale=1.0, clip=None, dynamic=True):
        wn, gn, mn, vn = (np.ascontiguousarray(x.numpy()) for x in (w, g, m, v))
        self.o.adam(wn, gn, mn, vn, t, lr, b1, b2, eps, wd=wd, variant=1, gscale=gscale, clip=float(clip[0]))
        w.copy_(torch.from_numpy(wn)); m.copy_(torch.from_numpy(mn)); v.copy_(torch.from_numpy(vn))


N, N_DECAY = 5000, 4200


def _inputs(world):
    w, _, m, v = gi.adam_inputs(n=N)
    grads = [gi.normal(gi.rng(100 + r), (N,), 2.0) for r in range(world)]
    return w, grads, m, v


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w, grads, m, v = _inputs(world)
        L = padded_length(N, world, 16)

        def padded(a):
            t = torch.zeros(L)
            t[:N] = torch.from_numpy(a)
            return t

        opt = ShardedAdam(padded(w), padded(grads[rank]), padded(m), padded(v), N_DECAY, N, world, rank,
                          lr=3e-4, b2=0.95, wd=0.1, clip=1.0, kernels=OracleKernels())
        f1 = opt.step(1, gscale=1.0 / 64)
        out[rank] = (opt.w[:N].numpy().copy(), float(f1[0]), float(opt.normsq[0]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2])
def test_sharded_adam_matches_single_process(world):
    from oracle.oracle import Oracle
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), out), nprocs=world, join=True)
    # single process: summed gradient, one update over the two decay classes
    o = Oracle()
    w, grads, m, v = _inputs(world)
    g = np.sum(grads, axis=0, dtype=np.float32)
    nsq = o.grad_norm_sq(g, 1.0 / 64)
    factor = o.clip_factor(np.float32(nsq), 1.0)
    assert factor < 1.0
    for lo, hi, wd in ((0, N_DECAY, 0.1), (N_DECAY, N, 0.0)):
        ws, gs, ms, vs = (np.ascontiguousarray(a[lo:hi]) for a in (w, g, m, v))
        o.adam(ws, gs, ms, vs, 1, 3e-4, 0.9, 0.95, 1e-8, wd=wd, variant=1, gscale=1.0 / 64, clip=factor)
        w[lo:hi] = ws
    for r in range(world):
        wr, fr, nr = out[r]
        assert abs(nr - nsq) <= 1e-5 * nsq
        assert abs(fr - factor) <= 1e-6
        assert np.max(np.abs(wr - w)) <= 1e-6 * np.max(np.abs(w))
    assert np.array_equal(out[0][0], out[1][0])          # every rank ends with the same parameters


def test_region_ownership_covers_the_flat_space_exactly_once():
    """RegionShardedAdam's ownership: the parts of all ranks tile every region without gap or overlap, every rank owns the
    same number of elements, and the staging buffer holds one slot per peer."""
    from ane_b200.sharded import RegionShardedAdam
    bounds = [0, 4096, 4096 + 8 * 1000, 20000 + 8 * 13, 65536]
    for world in (2, 4, 8):
        seen = [0] * bounds[-1]
        sizes = []
        for rank in range(world):
            parts = RegionShardedAdam.partition(bounds, world, rank)
            assert len(parts) == len(bounds) - 1
            sizes.append(sum(e - a for a, e in parts))
            for (a, e), lo, hi in zip(parts, bounds, bounds[1:]):
                assert lo <= a < e <= hi
                for i in range(a, e):
                    seen[i] += 1
        assert all(c == 1 for c in seen) and len(set(sizes)) == 1
        assert RegionShardedAdam.staging_floats(bounds, world) == (world - 1) * sizes[0]


def _rank_that_leaves(rank, world, port, out):
    """Rank 1 leaves the job between two steps (nothing of it is in flight); rank 0 learns of it when its next collective
    fails within the process group's short timeout, and reports instead of hanging."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    w, grads, m, v = _inputs(world)
    L = padded_length(N, world, 16)

    def padded(a):
        t = torch.zeros(L)
        t[:N] = torch.from_numpy(a)
        return t

    opt = ShardedAdam(padded(w), padded(grads[rank]), padded(m), padded(v), N_DECAY, N, world, rank,
                      lr=3e-4, b2=0.95, wd=0.1, clip=1.0, kernels=OracleKernels())
    opt.step(1, gscale=1.0 / 64)
    w_after_1 = opt.w[:N].numpy().copy()
    dist.barrier()
    if rank == 1:
        out[1] = "left after step 1"
        os._exit(0)                      # the rank is gone: no destroy_process_group, no goodbye
    t0 = time.time()
    try:
        opt.step(2, gscale=1.0 / 64)
        out[0] = "no error"
    except Exception as exc:             # gloo reports the closed connection or the timeout
        out[0] = ("detected", time.time() - t0, type(exc).__name__, bool(np.array_equal(opt.w[:N].numpy()[opt.lo:min(opt.hi, N)],
                                                                                   w_after_1[opt.lo:min(opt.hi, N)])))
    os._exit(0)                          # the group is broken; leave without the collective shutdown


def test_a_rank_that_leaves_between_steps_is_detected_not_waited_for():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_rank_that_leaves, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert not p.is_alive(), "a rank hung"
    assert out[1] == "left after step 1"
    assert out[0][0] == "detected", out[0]
    assert out[0][1] < 60.0               # within the group's timeout, not forever
    assert out[0][3]                      # the failed step did not half-update this rank's own slice


def test_layer_groups_cover_the_layers_in_backward_order():
    """LayerChain.layer_groups: the groups tile the layers exactly, top layers first, for any group count; together with
    RegionShardedAdam.partition this fixes which gradients a rank pushes after which part of the backward pass."""
    from ane_b200.layer_chain import ChainConfig, LayerChain
    for layers in (1, 5, 28):
        ch = LayerChain.__new__(LayerChain)
        ch.cfg = ChainConfig(layers=layers)
        for n in (1, 2, 7, 28, 40):
            groups = ch.layer_groups(n)
            assert len(groups) == min(n, layers)
            assert groups[0][0] == layers - 1 and groups[-1][1] == 0
            assert all(hi >= lo for hi, lo in groups)
            assert all(groups[i][1] == groups[i + 1][0] + 1 for i in range(len(groups) - 1))
