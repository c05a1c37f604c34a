"""GPU test of ane_cuda_rmsnorm_bwd_static_dev, the RMSNorm backward that never allocates.

Who needs it: a caller that shares the GPU with a framework which grabbed all device memory for
its own pool at start-up (any cudaMalloc from a side library then fails or fragments that pool),
or a latency-critical loop that cannot afford the device-wide synchronisation a cudaMalloc may
bring.  The regular entry point keeps its dw partials in a scratch range that grows with
cudaMalloc; this variant keeps them in a fixed 2.3 MiB array built into the library, which is
why it is limited to C <= 2048 and why calls that overlap on the GPU would race on that array.

The file sorts last on purpose, so that a run that stops at the first failure has already run
every other test.  It passes on its own in a fresh process (the new entry point is called before
ane_cuda_init, which it does not need) and after the other tests.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(L, fn, dt, B, C, S, dx, dw, dy, x, w, add, flags=0):
    import torch
    return fn(torch.cuda.current_stream().cuda_stream, dt, B, C, S, dx.data_ptr(), dw.data_ptr(), dy.data_ptr(), x.data_ptr(),
              w.data_ptr(), add.data_ptr() if add is not None else None, 1e-5, flags)


@pytest.mark.parametrize("dtype,with_add", [("float32", False), ("bfloat16", True)])
def test_static_scratch_matches_regular_entry_point(dtype, with_add):
    import torch
    from ane_b200 import lib
    assert torch.cuda.is_available(), "needs a CUDA device"
    torch.cuda.set_device(0)
    L = lib.load()
    tdt = getattr(torch, dtype)
    dt = {"float32": lib.F32, "bfloat16": lib.BF16}[dtype]
    g = torch.Generator(device="cuda").manual_seed(5)
    B, C, S = 6, 1024, 512
    x = torch.randn(B, C, S, device="cuda", generator=g).to(tdt)
    dy = torch.randn(B, C, S, device="cuda", generator=g).to(tdt)
    add = torch.randn(B, C, S, device="cuda", generator=g).to(tdt) if with_add else None
    w = 1 + 0.02 * torch.randn(C, device="cuda", generator=g)

    # the allocation-free entry point first, twice in a row (it must not depend on ane_cuda_init
    # nor on what an earlier call left in the shared array)
    outs = []
    for _ in range(2):
        dx = torch.empty_like(x)
        dw = torch.full((C,), 0.25, device="cuda")
        rc = _call(L, L.ane_cuda_rmsnorm_bwd_static_dev, dt, B, C, S, dx, dw, dy, x, w, add)
        assert rc == lib.OK, L.ane_cuda_last_error()
        torch.cuda.synchronize()
        outs.append((dx, dw))

    lib.init(0)
    dx_ref = torch.empty_like(x)
    dw_ref = torch.full((C,), 0.25, device="cuda")
    assert _call(L, L.ane_cuda_rmsnorm_bwd_dev, dt, B, C, S, dx_ref, dw_ref, dy, x, w, add) == lib.OK
    torch.cuda.synchronize()

    def same_dx(a, b):
        # the two entry points may sum the per-token statistics in different orders: fp32 within 1e-5,
        # 16-bit within one rounding step and 2e-3 in the L2 norm (the tolerances of test_gpu_parity)
        a, b = a.float(), b.float()
        scale = float(b.abs().max())
        if dtype == "float32":
            return float((a - b).abs().max()) <= 1e-5 * scale
        return float((a - b).abs().max()) <= 2.0 ** -8 * scale and float((a - b).norm()) <= 2e-3 * float(b.norm())

    for dx, dw in outs:
        assert same_dx(dx, dx_ref)
        err = float((dw - dw_ref).abs().max()) / float(dw_ref.abs().max())
        assert err <= (1e-5 if dtype == "float32" else 1e-4)                  # the tolerances of test_gpu_parity
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])

    # a smaller problem afterwards: rows of the shared array beyond its grid keep old values and
    # must not leak into the result
    Bs, Ss = 1, 64
    dxs, dws = torch.empty_like(x[:Bs, :, :Ss].contiguous()), torch.zeros(C, device="cuda")
    xs, dys = x[:Bs, :, :Ss].contiguous(), dy[:Bs, :, :Ss].contiguous()
    assert _call(L, L.ane_cuda_rmsnorm_bwd_static_dev, dt, Bs, C, Ss, dxs, dws, dys, xs, w, None) == lib.OK
    dxr, dwr = torch.empty_like(dxs), torch.zeros(C, device="cuda")
    assert _call(L, L.ane_cuda_rmsnorm_bwd_dev, dt, Bs, C, Ss, dxr, dwr, dys, xs, w, None) == lib.OK
    torch.cuda.synchronize()
    assert same_dx(dxs, dxr)
    assert float((dws - dwr).abs().max()) <= 1e-4 * float(dwr.abs().max())


# (B, C, S, dtype, fused add): 320 and 1280 token tiles against at most 296 blocks (every block walks several
# tiles and the shared array is used row by row up to its cap), a ragged fp32 shape that takes the scalar
# path (S not a multiple of the vector width), odd channel counts, and the largest channel count the array holds.
ORACLE_CASES = [(40, 1024, 512, "bfloat16", True), (40, 1024, 512, "float32", False), (3, 100, 33, "float32", False),
                (2, 333, 40, "bfloat16", True), (5, 2047, 96, "float32", True), (2, 2048, 72, "bfloat16", False)]


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("B,C,S,dtype,with_add", ORACLE_CASES)
def test_static_scratch_matches_the_cpu_oracle_and_allocates_nothing(oracle, B, C, S, dtype, with_add, exact):
    """dx and dw of the allocation-free entry point against the CPU oracle (the tolerances of test_gpu_parity),
    and the property the entry point exists for: across the call, neither the free device memory nor the
    library's cudaMalloc-grown scratch range changes."""
    import torch
    from ane_b200 import lib
    from tests.test_gpu_parity import close
    assert torch.cuda.is_available(), "needs a CUDA device"
    torch.cuda.set_device(0)
    L = lib.load()
    tdt = getattr(torch, dtype)
    dt, short = {"float32": (lib.F32, "f32"), "bfloat16": (lib.BF16, "bf16")}[dtype]
    rng = np.random.default_rng(C * 7 + S)
    mk = lambda *sh: torch.from_numpy(rng.standard_normal(sh).astype(np.float32)).cuda().to(tdt)
    x, dy = mk(B, C, S), mk(B, C, S)
    add = mk(B, C, S) if with_add else None
    w_np = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
    dw0 = (0.1 * rng.standard_normal(C)).astype(np.float32)
    w = torch.from_numpy(w_np).cuda()
    flags = lib.NORM_BWD_EXACT if exact else lib.NORM_BWD_REFERENCE

    def run():
        dx = torch.empty_like(x)
        dw = torch.from_numpy(dw0).cuda()
        torch.cuda.synchronize()
        free0, ws0 = torch.cuda.mem_get_info()[0], L.ane_cuda_workspace_bytes()
        rc = _call(L, L.ane_cuda_rmsnorm_bwd_static_dev, dt, B, C, S, dx, dw, dy, x, w, add, flags)
        assert rc == lib.OK, L.ane_cuda_last_error()
        torch.cuda.synchronize()
        return dx, dw, free0 - torch.cuda.mem_get_info()[0], L.ane_cuda_workspace_bytes() - ws0

    run()                                   # the first call on a device resolves the array's address
    dx, dw, free_delta, ws_delta = run()
    assert free_delta == 0 and ws_delta == 0
    rdx, rdw = oracle.rmsnorm_bwd(dy.float().cpu().numpy(), x.float().cpu().numpy(), w_np, dw=dw0, eps=1e-5, exact=exact)
    if with_add:
        rdx = oracle.add(rdx, add.float().cpu().numpy())
    assert close(dx.float().cpu().numpy(), rdx, short)
    err = float(np.abs(dw.cpu().numpy() - rdw).max()) / float(np.abs(rdw).max())
    assert err <= (1e-5 if dtype == "float32" else 1e-4)


def test_static_scratch_rejects_sizes_beyond_its_array():
    import torch
    from ane_b200 import lib
    L = lib.load()
    t = torch.zeros(16, device="cuda")
    rc = L.ane_cuda_rmsnorm_bwd_static_dev(None, lib.F32, 1, 2049, 4, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                           t.data_ptr(), None, 1e-5, 0)
    assert rc == lib.ERR_UNSUPPORTED
    assert b"2048" in L.ane_cuda_last_error()
    assert L.ane_cuda_rmsnorm_bwd_static_dev(None, lib.F32, 1, 8, 4, None, None, None, None, None, None, 1e-5, 0) == lib.ERR_INVALID
