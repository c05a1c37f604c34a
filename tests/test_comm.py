"""The multi-GPU group of the C ABI (ane_cuda_comm_*, ane_cuda_allreduce_f32, ane_cuda_sharded_adam_step).

Without a GPU: the argument and state errors, and that a plain C caller compiles and links.  On one GPU: a group of
one rank computes the same step as the device operators, and a rank that waits for a peer which never joins gets
ANE_CUDA_ERR_TIMEOUT from the host-side deadline (no GPU work is involved in that wait).  On two GPUs: two processes of
tests/c_driver/sharded_step_driver.c end with the bits that two ranks of ane_b200.sharded.ShardedAdam end with,
through NCCL and through peer memory.
"""
import ctypes as C
import os
import shutil
import socket
import subprocess

import numpy as np
import pytest

from ane_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c_driver", "sharded_step_driver.c")
N_PARAMS, N_DECAY = 100003, 90000


def _build(tmp_path):
    lib.load()
    exe = str(tmp_path / "sharded_step_driver")
    cmd = ["gcc", "-O1", "-Wall", "-Werror", SRC, "-I", os.path.join(ROOT, "include"), "-L", os.path.join(ROOT, "ane_b200", "lib"),
           "-lane_cuda", "-Wl,-rpath," + os.path.join(ROOT, "ane_b200", "lib"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def hashed(n, seed, scale):
    """tests/c_driver/sharded_step_driver.c hashed(), vectorised: the same bits"""
    m = np.uint64(0xFFFFFFFF)
    x = (np.arange(n, dtype=np.uint64) * np.uint64(2654435761) + np.uint64(seed * 40503 + 12345)) & m
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(2246822519)) & m
    x ^= x >> np.uint64(13)
    x = (x * np.uint64(3266489917)) & m
    x ^= x >> np.uint64(16)
    return ((x >> np.uint64(8)).astype(np.float32) * np.float32(1.0 / 16777216.0) - np.float32(0.5)) * np.float32(scale)


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_caller_of_the_group_compiles_and_links(tmp_path):
    assert os.path.getsize(_build(tmp_path)) > 0


def test_group_calls_before_init_return_codes():
    L = lib.load()
    buf = (C.c_ubyte * 128)()
    if L.ane_cuda_version() and not _gpu():
        assert L.ane_cuda_comm_init(1, 0, buf, 1.0) == lib.ERR_NOT_INIT
        assert L.ane_cuda_allreduce_f32(None, None, 4) == lib.ERR_NOT_INIT
        assert L.ane_cuda_sharded_adam_step(None, None, None, None, None, 8, 4, 8, 1, 0, 0, 0, 0, 0, 0, 0, 1, None) == lib.ERR_NOT_INIT
        assert L.ane_cuda_comm_map_peers(None, None, 8) == lib.ERR_NOT_INIT
    assert L.ane_cuda_comm_unique_id(None) == lib.ERR_INVALID
    assert L.ane_cuda_comm_size() == 0 and L.ane_cuda_comm_rank() == -1
    assert L.ane_cuda_comm_destroy() == lib.OK                       # nothing to destroy: still fine


def _gpu():
    import torch
    return torch.cuda.is_available()


@pytest.mark.gpu
def test_group_of_one_rank_equals_the_device_operators():
    import torch
    from ane_b200 import dev_ops as ops
    assert torch.cuda.is_available()
    lib.init(0)
    L = lib.load()
    ident = (C.c_ubyte * 128)()
    lib.check(L.ane_cuda_comm_unique_id(ident))
    assert L.ane_cuda_comm_init(0, 0, ident, 5.0) == lib.ERR_INVALID
    assert L.ane_cuda_comm_init(2, 2, ident, 5.0) == lib.ERR_INVALID
    lib.check(L.ane_cuda_comm_init(1, 0, ident, 20.0))
    try:
        assert L.ane_cuda_comm_size() == 1 and L.ane_cuda_comm_rank() == 0
        assert L.ane_cuda_comm_init(1, 0, ident, 5.0) == lib.ERR_INVALID      # only one group at a time
        n = 4096 * 3
        w = torch.from_numpy(hashed(n, 1, 0.08)).cuda()
        g = torch.from_numpy(hashed(n, 2, 40.0)).cuda()                       # large: the clip triggers
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        w2, m2, v2 = w.clone(), m.clone(), v.clone()
        nsq = torch.zeros(1, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        assert L.ane_cuda_sharded_adam_step(st, w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n, 0, n + 1, 1, 3e-4, 0.9, 0.95,
                                            1e-8, 0.1, 0.5, 1.0, lib.ADAM_DYNAMIC, None) == lib.ERR_INVALID
        n_decay = 9000
        for t in (1, 2):
            lib.check(L.ane_cuda_sharded_adam_step(st, w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n, n_decay, n - 5, t, 3e-4, 0.9,
                                                   0.95, 1e-8, 0.1, 0.5, 1.0, lib.ADAM_DYNAMIC, nsq.data_ptr()))
            lib.check(L.ane_cuda_comm_wait(st, 20.0))
            want_nsq = ops.grad_norm_sq(g, 0.5)
            clip = ops.clip_factor(want_nsq, 1.0)
            assert float(clip[0]) < 1.0
            ops.adam(w2[:n_decay], g[:n_decay], m2[:n_decay], v2[:n_decay], t, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, gscale=0.5, clip=clip)
            ops.adam(w2[n_decay:n - 5], g[n_decay:n - 5], m2[n_decay:n - 5], v2[n_decay:n - 5], t, 3e-4, 0.9, 0.95, 1e-8, wd=0.0, gscale=0.5, clip=clip)
            assert torch.equal(nsq, want_nsq)
        assert torch.equal(w, w2) and torch.equal(m, m2) and torch.equal(v, v2)
        x = torch.arange(5, device="cuda", dtype=torch.float32)
        lib.check(L.ane_cuda_allreduce_f32(st, x.data_ptr(), 5))
        lib.check(L.ane_cuda_comm_wait(st, -1.0))
        assert torch.equal(x.cpu(), torch.arange(5, dtype=torch.float32))
    finally:
        lib.check(L.ane_cuda_comm_destroy())
    assert L.ane_cuda_allreduce_f32(None, None, 1) == lib.ERR_NOT_INIT


@pytest.mark.gpu
def test_a_rank_that_never_joins_ends_in_a_timeout_code():
    """Host-made failure: this process is rank 0 of a group of two whose rank 1 does not exist.  The join runs into the
    host-side deadline, the half-made communicator is aborted, and the library keeps working afterwards."""
    import time
    import torch
    lib.init(0)
    L = lib.load()
    ident = (C.c_ubyte * 128)()
    lib.check(L.ane_cuda_comm_unique_id(ident))
    t0 = time.time()
    rc = L.ane_cuda_comm_init(2, 0, ident, 1.0)
    assert rc == lib.ERR_TIMEOUT, L.ane_cuda_last_error()
    assert b"aborted" in L.ane_cuda_last_error()
    assert time.time() - t0 < 30.0
    assert L.ane_cuda_comm_size() == 0
    lib.check(L.ane_cuda_comm_unique_id(ident))                     # a new group can be made
    lib.check(L.ane_cuda_comm_init(1, 0, ident, 20.0))
    lib.check(L.ane_cuda_comm_destroy())
    from ane_b200 import dev_ops as ops
    x = torch.randn(2, 64, 32, device="cuda")
    assert bool(torch.isfinite(ops.rmsnorm(x, torch.ones(64, device="cuda"))).all())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _python_ranks(rank, world, port, out_dir, steps):
    import torch
    import torch.distributed as dist
    from ane_b200.sharded import ShardedAdam, padded_length
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    lib.init(rank)
    n = padded_length(N_PARAMS, world)
    w, g = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    w[:N_PARAMS] = torch.from_numpy(hashed(N_PARAMS, 7, 0.08)).to(dev)
    g[:N_PARAMS] = torch.from_numpy(hashed(N_PARAMS, 100 + rank, 0.04)).to(dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    opt = ShardedAdam(w, g, m, v, N_DECAY, N_PARAMS, world, rank, lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=1.0)
    for t in range(1, steps + 1):
        opt.step(t, 0.5)
    torch.cuda.synchronize()
    out = np.concatenate([w.cpu().numpy(), m[opt.lo:opt.hi].cpu().numpy(), v[opt.lo:opt.hi].cpu().numpy(), opt.normsq.cpu().numpy()])
    out.astype(np.float32).tofile(os.path.join(out_dir, f"py_rank{rank}.bin"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_two_c_processes_equal_two_python_ranks(tmp_path):
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, steps = 2, 2
    exe = _build(tmp_path)
    mp.spawn(_python_ranks, args=(world, _free_port(), str(tmp_path), steps), nprocs=world, join=True)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for form in ("nccl", "peer"):
        idf = str(tmp_path / f"id_{form}")
        procs = [subprocess.Popen([exe, str(world), str(r), idf, str(tmp_path / f"c_{form}_rank{r}.bin"), form, str(steps)],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
        outs = [p.communicate(timeout=240)[0] for p in procs]
        for r, p in enumerate(procs):
            assert p.returncode == 0, outs[r]
        for r in range(world):
            got = np.fromfile(tmp_path / f"c_{form}_rank{r}.bin", np.float32)
            want = np.fromfile(tmp_path / f"py_rank{r}.bin", np.float32)
            assert got.size == want.size
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (form, r, float(np.abs(got - want).max()))
    moved = np.fromfile(tmp_path / "py_rank0.bin", np.float32)[:N_PARAMS]
    assert np.abs(moved - hashed(N_PARAMS, 7, 0.08)).max() > 1e-5            # the steps did change the parameters
