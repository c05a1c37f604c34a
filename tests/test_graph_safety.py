"""Library-owned device memory against captured CUDA graphs, and host-injected allocation failures.

The operators keep a scratch range and cached RoPE cos/sin tables between calls.  A CUDA graph bakes their
addresses in, so the library never frees, moves or refills an address it has handed out: these tests capture a
graph, then make the library grow its scratch and fill more tables than the old four-slot cache held, replay the
graph and compare with the eager result.  Failure paths are driven from the host (a refused allocation through the
"fail_alloc" hook, a frozen library); nothing here faults or hangs the GPU.
"""
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch
    from ane_b200 import dev_ops, lib
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    lib.init(0)
    return dev_ops


def _inputs(torch, B, heads, hd, S, C):
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(B, heads * hd, S, device="cuda", generator=g).to(torch.bfloat16)
    dq = torch.randn(B, heads * hd, S, device="cuda", generator=g).to(torch.bfloat16)
    wq = 1 + 0.02 * torch.randn(hd, device="cuda", generator=g)
    x = torch.randn(B, C, S, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(B, C, S, device="cuda", generator=g).to(torch.bfloat16)
    w = 1 + 0.02 * torch.randn(C, device="cuda", generator=g)
    return q, dq, wq, x, dy, w


def test_replay_after_cache_growth_matches_eager(dev):
    import torch
    from ane_b200 import lib
    B, heads, hd, S, C = 2, 4, 128, 256, 512
    q, dq, wq, x, dy, w = _inputs(torch, B, heads, hd, S, C)
    out = {k: torch.empty_like(q) for k in ("qr", "dqo", "r")}
    dx = torch.empty_like(x)
    dwq, dw = torch.zeros(hd, device="cuda"), torch.zeros(C, device="cuda")

    def chain():
        dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0, out=out["qr"])
        dev.rope(q, hd, base=1e6, pos0=0, out=out["r"])
        dev.rope_qknorm_bwd(dq, q, wq, dwq, hd, 1e-6, 1e6, 0, out=out["dqo"])
        dev.rmsnorm_bwd(dy, x, w, dw, out=dx)

    chain()                                               # everything a capture needs exists before it
    torch.cuda.synchronize()
    want = {k: v.clone() for k, v in out.items()}
    want_dx, want_dw, want_dwq = dx.clone(), dw.clone(), dwq.clone()
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            chain()
    ws_before = lib.load().ane_cuda_workspace_bytes()

    # later eager calls: six more table keys (the graph's table must survive) and a scratch need far above the present one
    for pos0 in range(1, 7):
        dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, pos0)
    big = torch.randn(300, 2048, 64, device="cuda").to(torch.bfloat16)
    dev.rmsnorm_bwd(big, big, torch.ones(2048, device="cuda"), torch.zeros(2048, device="cuda"))
    lib.check(lib.load().ane_cuda_reserve_workspace(ws_before * 4 + (64 << 20)))
    assert lib.load().ane_cuda_workspace_bytes() > ws_before
    torch.cuda.synchronize()

    for t in out.values():
        t.zero_()
    dx.zero_()
    dw.zero_()
    dwq.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for k in out:
        assert torch.equal(out[k], want[k]), k
    assert torch.equal(dx, want_dx)
    # a capture does not execute: one replay onto zeroed accumulators equals the one eager run
    assert torch.equal(dw, want_dw) and torch.equal(dwq, want_dwq)
    assert lib.poll_status().wait_giveups == 0


def test_missing_table_inside_a_capture_is_refused_not_baked_in(dev):
    import torch
    from ane_b200 import lib
    B, heads, hd, S, C = 1, 2, 128, 128, 256
    q, dq, wq, x, dy, w = _inputs(torch, B, heads, hd, S, C)
    dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0)
    want_rope = dev.rope(q, hd, base=1e6, pos0=977)       # eager: fills the table for first position 977
    lib.check(lib.load().ane_cuda_release_caches())       # and drop it again
    want_fused = None
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    got_rope = torch.empty_like(q)
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            with pytest.raises(lib.AneCudaError) as err:
                dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 977)            # no table for this key yet
            assert err.value.code == lib.ERR_UNSUPPORTED
            dev.rope(q, hd, base=1e6, pos0=977, out=got_rope)        # the stand-alone RoPE evaluates cos/sin in the kernel instead
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(got_rope, want_rope)                          # the same bits as with the table
    want_fused = dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 977)          # outside the capture the table is made
    assert bool(torch.isfinite(want_fused.float()).all())


def test_frozen_library_refuses_to_grow(dev):
    import torch
    from ane_b200 import lib
    L = lib.load()
    B, heads, hd, S, C = 1, 2, 128, 64, 256
    q, dq, wq, x, dy, w = _inputs(torch, B, heads, hd, S, C)
    dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0)
    lib.check(L.ane_cuda_freeze(1))
    try:
        dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0)                               # known key: fine
        with pytest.raises(lib.AneCudaError) as err:
            dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 12345)                       # new key
        assert err.value.code == lib.ERR_UNSUPPORTED and "frozen" in str(err.value)
        assert L.ane_cuda_reserve_workspace(L.ane_cuda_workspace_bytes() + (32 << 20)) == lib.ERR_UNSUPPORTED
        ws = L.ane_cuda_workspace_bytes()
        Sx = 1024
        Bx = (ws // 4 + (1 << 20)) // Sx + 1                                   # more per-token losses than the scratch holds
        logits = torch.zeros(Bx, 2, Sx, device="cuda")
        tg = torch.zeros(Bx, Sx, device="cuda", dtype=torch.int32)
        with pytest.raises(lib.AneCudaError) as err:
            dev.cross_entropy(logits, tg)
        assert err.value.code == lib.ERR_NOMEM
        assert L.ane_cuda_workspace_bytes() == ws
    finally:
        lib.check(L.ane_cuda_freeze(0))
    dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 12345)                               # allowed again
    loss, _ = dev.cross_entropy(logits, tg)                                    # and the scratch grows
    assert L.ane_cuda_workspace_bytes() > ws
    assert abs(float(loss[0]) - 0.6931472) < 1e-5                              # log 2 per token


def test_refused_allocations_come_back_as_error_codes(dev, oracle):
    """The allocation hook makes the next device allocations fail as if the GPU were out of memory: every entry point
    that allocates returns ANE_CUDA_ERR_NOMEM, nothing is launched on a null pointer, and the same call works afterwards."""
    import numpy as np
    import torch
    from ane_b200 import lib
    from tests.conftest import rel_err
    L = lib.load()
    lib.set_tuning("fail_alloc", 1)
    assert not L.ane_cuda_alloc(1 << 20)
    assert b"cudaMalloc" in L.ane_cuda_last_error()
    buf = L.ane_cuda_alloc(1 << 20)
    assert buf
    L.ane_cuda_free(buf)
    # a cos/sin table that cannot be allocated
    B, heads, hd, S, C = 1, 2, 128, 64, 256
    q, dq, wq, x, dy, w = _inputs(torch, B, heads, hd, S, C)
    lib.set_tuning("fail_alloc", 1)
    with pytest.raises(lib.AneCudaError) as err:
        dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 4242)
    assert err.value.code == lib.ERR_NOMEM
    got = dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 4242)
    want = oracle.qknorm_rope(q.float().cpu().numpy(), wq.cpu().numpy(), hd, 1e-6, 1e6, 4242)
    assert rel_err(got.float().cpu().numpy(), want) <= 2.0 ** -8
    # scratch growth that fails twice (the larger and the exact request)
    ws = L.ane_cuda_workspace_bytes()
    lib.set_tuning("fail_alloc", 2)
    assert L.ane_cuda_reserve_workspace(ws + (16 << 20)) == lib.ERR_NOMEM
    assert L.ane_cuda_workspace_bytes() == ws
    assert L.ane_cuda_reserve_workspace(ws + (16 << 20)) == lib.OK
    # a host-pointer drop-in whose device staging cannot be allocated (a fresh library state: nothing staged yet)
    from ane_b200 import cpu_ops
    torch.cuda.synchronize()
    L.ane_cuda_shutdown()
    lib.init(0)
    xs = np.random.default_rng(0).standard_normal((1024, 256)).astype(np.float32)
    out = np.empty_like(xs)
    lib.set_tuning("fail_alloc", 1)
    try:
        with pytest.raises(lib.AneCudaError) as err:
            cpu_ops.rmsnorm(out, xs, np.ones(1024, np.float32), 1024, 256)
        assert err.value.code == lib.ERR_NOMEM
    finally:
        lib.clear_tuning("fail_alloc")
    cpu_ops.rmsnorm(out, xs, np.ones(1024, np.float32), 1024, 256)
    assert rel_err(out, oracle.rmsnorm(xs, np.ones(1024, np.float32))) <= 1e-5


@pytest.mark.parametrize("which", ["fwd", "bwd"])
def test_ring_kernel_gives_up_cleanly_when_a_copy_never_arrives(dev, oracle, which):
    """The bounded waits of the TMA ring kernels, made to run out on purpose and harmlessly: a test hook lets the
    producer arm the barrier of one work item without starting its copy, with a short wait limit.  The call returns,
    the give-up is counted in the status words, nothing faults, and the next ordinary call is correct."""
    import numpy as np
    import torch
    from ane_b200 import lib
    from tests.conftest import rel_err
    B, heads, hd, S = 2, 4, 128, 256
    q, dq, wq, *_ = _inputs(torch, B, heads, hd, S, 256)
    dw = torch.zeros(hd, device="cuda")
    dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0)                     # table exists, scratch sized
    dev.rope_qknorm_bwd(dq, q, wq, dw, hd, 1e-6, 1e6, 0)
    torch.cuda.synchronize()
    lib.poll_status(reset=True)
    lib.set_tuning("qk_test_skip_item", 1)
    lib.set_tuning("qk_wait_limit", 64)
    try:
        if which == "fwd":
            dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0)
        else:
            dev.rope_qknorm_bwd(dq, q, wq, torch.zeros(hd, device="cuda"), hd, 1e-6, 1e6, 0)
        torch.cuda.synchronize()
    finally:
        lib.clear_tuning("qk_test_skip_item")
        lib.clear_tuning("qk_wait_limit")
    assert lib.poll_status(reset=True).wait_giveups > 0
    qn, wn = q.float().cpu().numpy(), wq.cpu().numpy()
    got = dev.qknorm_rope(q, wq, hd, 1e-6, 1e6, 0)
    assert rel_err(got.float().cpu().numpy(), oracle.qknorm_rope(qn, wn, hd, 1e-6, 1e6, 0)) <= 2.0 ** -8
    dw = torch.zeros(hd, device="cuda")
    dx = dev.rope_qknorm_bwd(dq, q, wq, dw, hd, 1e-6, 1e6, 0)
    rdx, rdw = oracle.rope_qknorm_bwd(dq.float().cpu().numpy(), qn, wn, hd, eps=1e-6, base=1e6, pos0=0)
    assert rel_err(dx.float().cpu().numpy(), rdx) <= 2.0 ** -8 and rel_err(dw.cpu().numpy(), rdw) <= 1e-4
    assert lib.poll_status().wait_giveups == 0


def test_extent_checking_mode_catches_buffers_that_are_too_small(dev):
    """With the debug knob check_extents = 1 every device range an operator will touch is checked against the allocation
    that holds the pointer, before anything is launched: an output (or input) one element short is an argument error
    that names the argument, and the guard bytes behind it stay untouched."""
    import ctypes as C
    import torch
    from ane_b200 import lib
    L = lib.load()
    B, Cn, S = 2, 64, 40
    nbytes = B * Cn * S * 4
    bufs = {k: L.ane_cuda_alloc(nbytes) for k in ("x", "out", "f")}
    short = L.ane_cuda_alloc(nbytes - 4)
    w = L.ane_cuda_alloc(Cn * 4)
    assert all(bufs.values()) and short and w
    ptr = lambda b: L.ane_cuda_devptr(b)
    st = None
    lib.set_tuning("check_extents", 1)
    try:
        assert L.ane_cuda_rmsnorm_dev(st, lib.F32, B, Cn, S, ptr(bufs["out"]), ptr(bufs["x"]), ptr(w), C.c_float(1e-5)) == lib.OK
        assert L.ane_cuda_rmsnorm_dev(st, lib.F32, B, Cn, S, ptr(short), ptr(bufs["x"]), ptr(w), C.c_float(1e-5)) == lib.ERR_INVALID
        assert b"out" in L.ane_cuda_last_error() and b"bytes" in L.ane_cuda_last_error()
        assert L.ane_cuda_rmsnorm_dev(st, lib.F32, B, Cn, S, ptr(bufs["out"]), ptr(short), ptr(w), C.c_float(1e-5)) == lib.ERR_INVALID
        assert L.ane_cuda_rmsnorm_dev(st, lib.F32, B, Cn + 1, S, ptr(bufs["out"]), ptr(bufs["x"]), ptr(w), C.c_float(1e-5)) == lib.ERR_INVALID   # w too small too
        n = B * Cn * S
        assert L.ane_cuda_residual_dev(st, lib.F32, n, ptr(bufs["out"]), ptr(bufs["x"]), ptr(bufs["f"]), C.c_float(0.5)) == lib.OK
        assert L.ane_cuda_residual_dev(st, lib.F32, n, ptr(bufs["out"]), ptr(bufs["x"]), ptr(short), C.c_float(0.5)) == lib.ERR_INVALID
        assert L.ane_cuda_swiglu_dev(st, lib.F32, n + 1, ptr(bufs["out"]), ptr(bufs["x"]), ptr(bufs["f"])) == lib.ERR_INVALID
        assert L.ane_cuda_qknorm_rope_dev(st, lib.F32, B, 1, Cn, S, ptr(short), ptr(bufs["x"]), ptr(w), C.c_float(1e-6), C.c_float(1e4), 0) == lib.ERR_INVALID
        host = (C.c_float * 4)()
        assert L.ane_cuda_residual_dev(st, lib.F32, 4, ptr(bufs["out"]), C.cast(host, C.c_void_p), ptr(bufs["f"]), C.c_float(0.5)) == lib.ERR_INVALID   # not device memory
        # a torch tensor inside the caching allocator's segment: the check sees the segment, so an in-range view passes
        t = torch.zeros(B, Cn, S, device="cuda")
        assert L.ane_cuda_rmsnorm_dev(torch.cuda.current_stream().cuda_stream, lib.F32, B, Cn, S, t.data_ptr(), t.data_ptr(), ptr(w), C.c_float(1e-5)) == lib.OK
    finally:
        lib.clear_tuning("check_extents")
    # off again: the same short buffer is not looked at (and the call below stays inside it)
    assert L.ane_cuda_residual_dev(st, lib.F32, n - 1, ptr(short), ptr(bufs["x"]), ptr(bufs["f"]), C.c_float(0.5)) == lib.OK
    torch.cuda.synchronize()
    for b in list(bufs.values()) + [short, w]:
        L.ane_cuda_free(b)
