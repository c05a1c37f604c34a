"""Two ranks on two GPUs: the sharded optimizer step over peer memory (reduce kernel reading the other rank's
gradients, Adam kernel storing the new weights to both ranks) gives the same parameters and moments as the same
step through NCCL reduce-scatter / all-gather.  Skipped on a machine with fewer than two GPUs; the kernels
themselves are covered on one GPU with emulated ranks (test_gpu_parity.py)."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def m2_full(m_local, opt, dist, dev, n):
    """The first moments of all ranks' slices of a one-slice optimizer, gathered (each rank only updates its own slice)."""
    import torch
    out = torch.empty(n, device=dev)
    dist.all_gather_into_tensor(out, m_local[opt.lo:opt.hi].contiguous())
    return out


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from ane_b200 import lib
    from ane_b200.sharded import RegionShardedAdam, ShardedAdam, padded_length, symmetric_buffer, symmetric_buffers

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    lib.init(rank)
    n_params, n_decay = 100_003, 90_000
    n = padded_length(n_params, world)
    w, g, ptrs = symmetric_buffers(n, dev)
    gen = torch.Generator(device=dev).manual_seed(7)                   # same parameters on every rank
    w.copy_(torch.randn(n, device=dev, generator=gen) * 0.02)
    gen_r = torch.Generator(device=dev).manual_seed(100 + rank)        # each rank its own gradients
    g.copy_(torch.randn(n, device=dev, generator=gen_r) * 0.01)
    g[n_params:] = 0
    w2, g2 = w.clone(), g.clone()
    w3, g3, ptrs3 = symmetric_buffers(n, dev)
    w3.copy_(w)
    g3.copy_(g)
    w4, g4, ptrs4 = symmetric_buffers(n, dev)
    w4.copy_(w)
    g4.copy_(g)
    m4, v4 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    bounds = [0, 40_000, 80_000, n]
    regions = RegionShardedAdam(w4, g4, m4, v4, n_decay, n_params, world, rank, ptrs4, bounds,
                                staging=symmetric_buffer(RegionShardedAdam.staging_floats(bounds, world), dev))
    w5, g5, ptrs5 = symmetric_buffers(n, dev)
    w5.copy_(w)
    g5.copy_(g)
    m5, v5 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    deferred = RegionShardedAdam(w5, g5, m5, v5, n_decay, n_params, world, rank, ptrs5, bounds, deferred_broadcast=True,
                                 staging=symmetric_buffer(RegionShardedAdam.staging_floats(bounds, world), dev))
    m, v, m2, v2, m3, v3 = (torch.zeros(n, device=dev) for _ in range(6))
    peer = ShardedAdam(w, g, m, v, n_decay, n_params, world, rank, peer_ptrs=ptrs)
    nccl = ShardedAdam(w2, g2, m2, v2, n_decay, n_params, world, rank)
    early = ShardedAdam(w3, g3, m3, v3, n_decay, n_params, world, rank, peer_ptrs=ptrs3, n_early=70_001)   # part of the reduce ahead of time
    for t in (1, 2):
        early.begin_step(0.5)
        peer.step(t, 0.5)
        nccl.step(t, 0.5)
        early.step(t, 0.5)
        # every rank owns a part of every region; two of the three regions are pushed to their owners "during the step"
        regions.begin_step(0.5)
        for i in (1, 0):
            ev = torch.cuda.Event()
            ev.record()
            regions.reduce_region(i, ev)
        regions.step(t, 0.5)
        # the same with the weights leaving through the copy engines after a local Adam; the norm weights (no decay) must be
        # everywhere when step() is over, the rest after the next step's first sync or flush()
        deferred.begin_step(0.5)
        ev = torch.cuda.Event()
        ev.record()
        deferred.push_region(0, ev)
        deferred.step(t, 0.5)
        torch.cuda.synchronize()
        dist.barrier()
        norms_there = bool(torch.equal(w5[n_decay:n_params], w4[n_decay:n_params]))
    deferred.flush()
    torch.cuda.synchronize()
    dist.barrier()
    own = torch.zeros(n, dtype=torch.bool, device=dev)
    for a, e in regions.owned_ranges():
        own[a:e] = True
    ok_regions = bool(torch.allclose(regions.normsq, nccl.normsq, rtol=1e-6)) and bool(torch.allclose(w4, w2, rtol=1e-5, atol=1e-8)) \
        and bool(torch.allclose(m4[own], m2_full(m2, nccl, dist, dev, n)[own], rtol=1e-5, atol=1e-10)) and int(own.sum()) == n // world \
        and norms_there and bool(torch.equal(w5, w4))
    ok = bool(torch.equal(w, w2)) and bool(torch.equal(m[peer.lo:peer.hi], m2[peer.lo:peer.hi])) \
        and bool(torch.equal(v[peer.lo:peer.hi], v2[peer.lo:peer.hi])) and bool(torch.equal(peer.normsq, nccl.normsq)) \
        and bool(torch.allclose(early.normsq, nccl.normsq, rtol=1e-6)) \
        and bool(torch.allclose(w3, w2, rtol=1e-5, atol=1e-8)) \
        and bool(torch.allclose(m3[peer.lo:peer.hi], m2[peer.lo:peer.hi], rtol=1e-5, atol=1e-10))
    # (the early form adds the squared norm as two partial sums, so its clip factor, and with it the update, may differ
    # from the one-pass forms in the last bit)
    changed = bool((w != torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) * 0.02)[:n_params].any())
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok and changed and ok_regions else f"mismatch ok={ok} changed={changed} regions={ok_regions}")
    dist.barrier()
    dist.destroy_process_group()


def test_peer_memory_step_equals_nccl_step(tmp_path):
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"
