"""Benchmark of the hot path: the Qwen3-0.6B non-matmul layer chain plus the Adam step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the operator chain (ane_b200.layer_chain: embedding gather, 28 layers of
forward and backward operators, final norm, embedding scatter-add) over 256 sequences x 2048
tokens in bf16, followed by gradient-norm / clip / Adam over 596 M fp32 parameters.  The 256
sequences are split over the N ranks (total work fixed: strong scaling) and run in micro-batches;
matmul and attention outputs are pre-filled synthetic buffers (not executed, not timed).

Rank 0 prints ONE JSON line:
  value      tokens/s, inputs resident in HBM, device-timed (CUDA events, max over ranks)
  roofline   the dominant kernel (SwiGLU backward): algorithmic bytes / measured launch time
             against the measured HBM copy bandwidth of MEASURED_PEAKS.json
  ops        per-operator achieved GB/s on benchmark-sized tensors (each launch rotates over
             buffer sets larger than L2)
  e2e        the same chain through the host-buffer entry points (ane_cuda_*_host) with
             page-locked host tensors: every operator's inputs are uploaded and its outputs
             downloaded inside the timed region
  cpu_baseline  the CPU oracle (a port of the reference's operators) on the host cores, bounded sample
`--impl reference` times that CPU path alone, on the same configuration and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOTAL_SEQS = 256
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
SWIGLU_BWD_DRAM_BYTES_PER_ALGORITHMIC_BYTE = 0.953


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro-batch", type=int, default=64, help="sequences per micro-batch and GPU")
    ap.add_argument("--seqs", type=int, default=TOTAL_SEQS, help="sequences per step over all GPUs")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--no-ops", action="store_true", help="skip the per-operator table")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--no-p2p", action="store_true", help="N > 1: use NCCL reduce-scatter / all-gather instead of the peer-memory optimizer kernels")
    ap.add_argument("--early-reduce", action="store_true", help="N > 1, peer memory: reduce the matmul gradients on a side stream beside the chain instead of at the end of the step (measured slower: the chain is HBM-bound)")
    ap.add_argument("--no-boundary-fusion", action="store_true", help="run the closing residual and the next norm as two operators")
    ap.add_argument("--overlap-groups", type=int, default=7, help="N > 1, peer memory: the backward pass of a step's last micro-batch runs as this many groups of layers, and each group's gradients are reduced on a side stream while the next groups run (0 or 1: reduce everything at the end of the step)")
    ap.add_argument("--no-deferred-broadcast", action="store_true", help="N > 1 with --overlap-groups: the Adam kernel stores the new weights to every rank itself instead of leaving matrices and embedding to the copy engines beside the next step")
    ap.add_argument("--cpu-seqs", type=int, default=2, help="sequences in the CPU sample")
    ap.add_argument("--e2e-seqs", type=int, default=8, help="sequences per rank and step of the host-buffer (e2e) measurement")
    return ap.parse_args()


def measured_peak():
    from ane_b200.peaks import hbm_peak_gbs
    return hbm_peak_gbs()


# ------------------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "power_w_max": max(self.power) if self.power else None, "samples": len(self.samples)}


# ------------------------------------------------------------------------------------- CPU path
def cpu_chain(cfg_kw, n_seqs: int, steps: int, warmup: int, threads=None):
    """The same operator chain on the host cores with the CPU oracle (fp32, as the reference's CPU
    operators are), on `n_seqs` sequences, all host threads; Adam on 1/32 of the parameters.
    Returns tokens/s extrapolated to the full step: t_step = t_chain * (seqs / n_seqs) + t_adam * 32.
    Output buffers are allocated once, outside the timed region."""
    import numpy as np

    from oracle.oracle import Oracle, _fp, _ip

    orc = Oracle(fast=True)
    if not threads:      # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1)
        try:
            threads = len(os.sched_getaffinity(0))
        except AttributeError:
            threads = os.cpu_count() or 1
    orc.set_num_threads(threads)
    nthreads = orc.num_threads()
    orc.set_chunk(128)      # spread (sequence, 128-token block) pairs over the threads
    C = orc.lib
    L, D, H = cfg_kw["layers"], 1024, 3072
    Qd, KVd, hd, S, V = 2048, 1024, 128, 2048, 151936
    alpha = float(np.float32((2.0 * L) ** -0.5))
    rng = np.random.Generator(np.random.PCG64(1234))

    def rnd(*shape, std=1.0):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)

    def emp(ch):
        return np.zeros((n_seqs, ch, S), np.float32)

    B = n_seqs
    sets = 2
    bufs = [dict(q=rnd(B, Qd, S), k=rnd(B, KVd, S), o=rnd(B, D, S), h1=rnd(B, H, S), h3=rnd(B, H, S), f=rnd(B, D, S),
                 dsilu=rnd(B, H, S), dxf=rnd(B, D, S), dq=rnd(B, Qd, S), dk=rnd(B, KVd, S), dxa=rnd(B, D, S)) for _ in range(sets)]
    table = rnd(V, D, std=0.02)
    tok = rng.integers(0, V, size=(B, S)).astype(np.int32)
    w = (1 + rnd(D, std=0.02)).astype(np.float32)
    wq = (1 + rnd(hd, std=0.02)).astype(np.float32)
    dw, dwq = np.zeros(D, np.float32), np.zeros(hd, np.float32)
    dE = np.zeros((V, D), np.float32)
    xs = [emp(D) for _ in range(L + 1)]
    x2s = [emp(D) for _ in range(L)]
    xn, qr, kr, gate, dh1, dh3, dqo, dko = emp(D), emp(Qd), emp(KVd), emp(H), emp(H), emp(H), emp(Qd), emp(KVd)
    dy, dy2, dx2, tmp = emp(D), emp(D), emp(D), emp(D)
    dy_cls = rnd(B, D, S)
    n_adam = 596_042_752 // 32
    aw, ag, am, av = rnd(n_adam, std=0.02), rnd(n_adam, std=1e-2), np.zeros(n_adam, np.float32), np.zeros(n_adam, np.float32)
    nD, nH = B * D * S, B * H * S

    def chain():
        for b in range(B):
            C.orc_embed_lookup(_fp(xs[0][b]), _fp(table), _ip(tok[b]), D, S, V)
        for l in range(L):
            u = bufs[l % sets]
            C.orc_rmsnorm_batched(_fp(xn), _fp(xs[l]), _fp(w), B, D, S, 1e-5)
            C.orc_qknorm_rope_batched(_fp(qr), _fp(u["q"]), _fp(wq), B, Qd // hd, hd, S, 1e-6, 1e6, 0)
            C.orc_qknorm_rope_batched(_fp(kr), _fp(u["k"]), _fp(wq), B, KVd // hd, hd, S, 1e-6, 1e6, 0)
            C.orc_residual(_fp(x2s[l]), _fp(xs[l]), _fp(u["o"]), alpha, nD)          # train.m:460
            C.orc_rmsnorm_batched(_fp(xn), _fp(x2s[l]), _fp(w), B, D, S, 1e-5)        # train.m:461
            C.orc_swiglu(_fp(gate), _fp(u["h1"]), _fp(u["h3"]), nH)
            C.orc_residual(_fp(xs[l + 1]), _fp(x2s[l]), _fp(u["f"]), alpha, nD)
        C.orc_rmsnorm_batched(_fp(xn), _fp(xs[L]), _fp(w), B, D, S, 1e-5)
        C.orc_rmsnorm_bwd_batched(_fp(dy), _fp(dw), _fp(dy_cls), _fp(xs[L]), _fp(w), B, D, S, 1e-5, 0)
        cur, nxt = dy, dy2
        for l in range(L - 1, -1, -1):
            u = bufs[l % sets]
            C.orc_swiglu_bwd(_fp(dh1), _fp(dh3), _fp(u["h1"]), _fp(u["h3"]), _fp(u["dsilu"]), nH)
            C.orc_rmsnorm_bwd_batched(_fp(tmp), _fp(dw), _fp(u["dxf"]), _fp(x2s[l]), _fp(w), B, D, S, 1e-5, 0)
            C.orc_add(_fp(dx2), _fp(tmp), _fp(cur), nD)                                # train.m:590
            C.orc_rope_qknorm_bwd_batched(_fp(dqo), _fp(dwq), _fp(u["dq"]), _fp(u["q"]), _fp(wq), B, Qd // hd, hd, S, 1e-6, 1e6, 0, 0)
            C.orc_rope_qknorm_bwd_batched(_fp(dko), _fp(dwq), _fp(u["dk"]), _fp(u["k"]), _fp(wq), B, KVd // hd, hd, S, 1e-6, 1e6, 0, 0)
            C.orc_rmsnorm_bwd_batched(_fp(tmp), _fp(dw), _fp(u["dxa"]), _fp(xs[l]), _fp(w), B, D, S, 1e-5, 0)
            C.orc_add(_fp(nxt), _fp(tmp), _fp(dx2), nD)                                # train.m:721
            cur, nxt = nxt, cur
        for b in range(B):
            C.orc_embed_backward(_fp(dE), _fp(cur[b]), _ip(tok[b]), D, S, V)

    def adam_part():
        nsq = orc.grad_norm_sq(ag, 1.0 / 2560.0)
        cf = orc.clip_factor(np.float32(nsq), 1.0)
        orc.adam(aw, ag, am, av, 1, 3e-4, 0.9, 0.95, 1e-8, wd=0.1, variant=1, gscale=1.0 / 2560.0, clip=cf)

    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        chain()
        t1 = time.perf_counter()
        adam_part()
        t2 = time.perf_counter()
        if i >= warmup:
            times.append((t1 - t0, t2 - t1))
    t_chain = statistics.mean(t[0] for t in times)
    t_adam = statistics.mean(t[1] for t in times)
    full = t_chain * (cfg_kw["seqs"] / n_seqs) + t_adam * 32
    return {
        "tokens_per_s": cfg_kw["seqs"] * S / full,
        "ms_per_step_extrapolated": full * 1e3,
        "sample_ms": (t_chain + t_adam) * 1e3,
        "cores": nthreads,
        "sample": f"{n_seqs} of {cfg_kw['seqs']} sequences x 2048 tokens through all {L} layers in fp32 "
                  f"({t_chain:.2f} s) + Adam on 1/32 of 596M params ({t_adam:.2f} s), {nthreads} threads; step time = chain x "
                  f"{cfg_kw['seqs'] // n_seqs} + Adam x 32",
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg_kw = {"layers": args.layers, "seqs": args.seqs}
    r = cpu_chain(cfg_kw, args.cpu_seqs, max(1, args.steps), max(0, min(args.warmup, 1)))
    line = {
        "impl": "reference",
        "metric": "layer-op tokens/sec (Qwen3-0.6B non-matmul layer chain + Adam)",
        "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_per_step_extrapolated"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "extrapolated": True, "sample_ms": round(r["sample_ms"], 1),
        "note": "ms_per_step and value are EXTRAPOLATED from a bounded sample (see cpu_baseline.sample): the timed work per step "
                "is sample_ms, scaled linearly in sequences and parameters to the full step",
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    return {
        "workload": "configs[4]: Qwen3-0.6B non-matmul layer chain (28 layers, dim 1024, hidden 3072, GQA 16/8, "
                    "head_dim 128, bf16 activations) + Adam on 596M fp32 params",
        "sequences": args.seqs, "seq_len": 2048, "layers": args.layers,
        "micro_batch_per_gpu": min(args.micro_batch, max(1, args.seqs // world)),
        "parallelism": f"dp{world} (sequences sharded, ZeRO-1 Adam)",
        "launch": "host launches" if getattr(args, "no_graph", False) else "CUDA graph replay per micro-batch (the first micro-batch of the first timed step runs eagerly, with events around the dominant kernel)",
        "l2_policy": f"inputs larger than L2: every operator reads per-layer buffers ({4 * min(args.micro_batch, max(1, args.seqs // world))}-"
                     f"{12 * min(args.micro_batch, max(1, args.seqs // world))} MiB each) last touched GBs of traffic earlier",
    }


def pcie_copy_only(torch, device, seconds: float = 1.0):
    """Diagnostic for the multi-GPU e2e figure: this rank's host <-> device copy rate with nothing else running on the GPU --
    256 MiB page-locked buffers, upload and download concurrently on two streams.  GB/s over both directions."""
    n = 256 << 20
    h_in, h_out = torch.empty(n, dtype=torch.uint8).pin_memory(), torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in, d_out = torch.empty(n, dtype=torch.uint8, device=device), torch.empty(n, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    torch.cuda.synchronize()
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        with torch.cuda.stream(s1):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(s2):
            h_out.copy_(d_out, non_blocking=True)
        s1.synchronize()
        s2.synchronize()
        reps += 1
    return 2 * n * reps / (time.perf_counter() - t0) / 1e9


# ------------------------------------------------------------------------------------- e2e (host buffers)
def e2e_chain(torch, cfg, params, device, n_seqs, steps, warmup):
    """The chain with host buffers on the contraction side (ane_b200.host_chain.HostLayerChain): every tensor a matmul
    or SDPA produces or consumes crosses PCIe inside the timed region, from / to page-locked host memory."""
    from ane_b200.host_chain import CHostLayerChain, HostLayerChain

    def timed(chain):
        for _ in range(warmup):
            chain.step()
        chain.synchronize()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            chain.step()
        chain.synchronize()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps

    hc = HostLayerChain(cfg, n_seqs, params, device)
    dt_py = timed(hc)
    # the headline: the same step through the C ABI's chain object (ane_cuda_chain_step), from the same host buffers
    del hc.chain.q, hc.chain.k, hc.chain.h1, hc.chain.h3, hc.chain.o_out, hc.chain.ffn_out, hc.chain.layer_in, hc.chain.x2
    torch.cuda.empty_cache()
    cc = CHostLayerChain(hc, params)
    dt = timed(cc)
    h2d, d2h = cc.h2d_bytes_per_step, cc.d2h_bytes_per_step
    cc.close()
    return n_seqs * cfg.seq / dt, h2d, d2h, dt, n_seqs * cfg.seq / dt_py


def e2e_per_op(torch, cfg, n_seqs, steps, warmup):
    """The same chain, every operator called on its own through the host-buffer entry points (ane_cuda_*_host): each call
    stages its own inputs and outputs, so tensors the operators hand to each other cross PCIe too."""
    from ane_b200 import host_ops as hop

    S, D, H, Qd, KVd, hd = cfg.seq, cfg.dim, cfg.hidden, cfg.q_dim, cfg.kv_dim, cfg.head_dim
    B = n_seqs
    bf = cfg.dtype

    def pin(ch, fill=True):
        t = torch.empty((B, ch, S), dtype=bf).pin_memory()
        if fill:
            t.normal_()
        return t

    x, o, f, h1, h3, q, k = pin(D), pin(D), pin(D), pin(H), pin(H), pin(Qd), pin(KVd)
    xn, x2, x2n, gate, xo, qr, kr = (pin(c, False) for c in (D, D, D, H, D, Qd, KVd))
    ds, dxf, dqi, dki, dxa, dy = pin(H), pin(D), pin(Qd), pin(KVd), pin(D), pin(D)
    dh1, dh3, dx2, dq, dk, dyo = (pin(c, False) for c in (H, H, D, Qd, KVd, D))
    w = torch.ones(D)
    wq = torch.ones(hd)
    dw = torch.zeros(D)
    dwq = torch.zeros(hd)
    e = 2
    h2d = cfg.layers * e * B * S * ((D) + (Qd + KVd) + 2 * D + 2 * H + 2 * D + 3 * H + 3 * D + 2 * (Qd + KVd) + 3 * D) + e * B * S * (D + 2 * D)
    d2h = cfg.layers * e * B * S * ((D) + (Qd + KVd) + 2 * D + H + D + 2 * H + D + (Qd + KVd) + D) + e * B * S * (D + D)

    def step():
        for _ in range(cfg.layers):
            hop.rmsnorm(xn, x, w, cfg.eps)
            hop.qknorm_rope(qr, q, wq, hd, cfg.qk_eps, cfg.rope_base)
            hop.qknorm_rope(kr, k, wq, hd, cfg.qk_eps, cfg.rope_base)
            hop.residual_rmsnorm(x2, x2n, x, o, w, cfg.alpha, cfg.eps)
            hop.swiglu(gate, h1, h3)
            hop.residual(xo, x2, f, cfg.alpha)
        hop.rmsnorm(xn, xo, w, cfg.eps)
        hop.rmsnorm_bwd(dyo, dw, dy, xo, w, eps=cfg.eps)
        for _ in range(cfg.layers):
            hop.swiglu_bwd(dh1, dh3, h1, h3, ds)
            hop.rmsnorm_bwd(dx2, dw, dxf, x2, w, add=dyo, eps=cfg.eps)
            hop.rope_qknorm_bwd(dq, dwq, dqi, q, wq, hd, cfg.qk_eps, cfg.rope_base)
            hop.rope_qknorm_bwd(dk, dwq, dki, k, wq, hd, cfg.qk_eps, cfg.rope_base)
            hop.rmsnorm_bwd(dyo, dw, dxa, x, w, add=dx2, eps=cfg.eps)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    return B * S / dt, h2d, d2h, dt


def cpu_reference_ops():
    """The reference's own compiled CPU functions (oracle/_ref, built from stories_cpu_ops.h and training_dynamic/cpu_ops.h
    with a portable stand-in for Accelerate) on their native shapes, one thread -- the way the reference calls them.
    Returns {} when the compiled reference is not present."""
    import numpy as np

    from oracle.oracle import Reference
    try:
        ref = Reference(fast=True)
    except Exception:
        return {}
    rng = np.random.default_rng(1234)
    out = {}

    def best_of(fn, n=3):
        ts = []
        for _ in range(n):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts)

    D, S, V = 768, 256, 32000
    x = rng.standard_normal((D, S)).astype(np.float32)
    dy = rng.standard_normal((D, S)).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(D)).astype(np.float32)
    t = best_of(lambda: ref.rmsnorm(x, w))
    out["rmsnorm [768,256] f32"] = {"ms": round(t * 1e3, 4), "GB/s": round(2 * D * S * 4 / t / 1e9, 2)}
    t = best_of(lambda: ref.rmsnorm_bwd(dy, x, w))
    out["rmsnorm_bwd [768,256] f32"] = {"ms": round(t * 1e3, 4), "GB/s": round(3 * D * S * 4 / t / 1e9, 2)}
    logits = rng.standard_normal((V, S)).astype(np.float32)
    tg = rng.integers(0, V, S).astype(np.uint16)
    t = best_of(lambda: ref.cross_entropy_loss(logits, tg), 2)
    out["cross_entropy [32000,256] f32"] = {"ms": round(t * 1e3, 3), "GB/s": round(2 * V * S * 4 / t / 1e9, 2)}
    table = rng.standard_normal((V, D)).astype(np.float32)
    tok = rng.integers(0, V, S).astype(np.uint16)
    t = best_of(lambda: ref.embed_lookup(table, tok))
    out["embed_lookup [32000x768] S=256"] = {"ms": round(t * 1e3, 4), "GB/s": round((S * 2 + 2 * D * S * 4) / t / 1e9, 2)}
    n = V * D                                             # one Stories110M embedding tensor: 24.6 M parameters
    wv, gv = (rng.standard_normal(n).astype(np.float32) * 0.01 for _ in range(2))
    mv, vv = np.zeros(n, np.float32), np.zeros(n, np.float32)
    t = best_of(lambda: ref.adam_update(wv, gv, mv, vv, 1, 3e-4, 0.9, 0.999, 1e-8), 2)
    out["adam 24.6M params"] = {"ms": round(t * 1e3, 2), "GB/s": round(28 * n / t / 1e9, 2)}
    return {"threads": 1, "kind": "reference", "build": "gcc -O3 -march=native, Accelerate calls through a portable C stand-in", "ops": out}


def cross_rank_checks(torch, dist, params, opt, t_last, gscale, world, rank, peer_mode):
    """Outside the timed region, world > 1: (a) every rank ends the timed steps with the same parameters -- a 64-bit sum
    of the parameter bits, MIN and MAX over the ranks; (b) one optimizer step from the same parameters and gradients, with
    cleared moments (the two forms keep the moments of different ranges on a rank), through both forms of the exchange
    (peer memory, then NCCL reduce-scatter / all-gather on restored buffers) and the largest difference between the two
    results relative to the largest parameter.  NCCL adds the ranks' gradients in its own order, the peer kernels in rank
    order, and the squared norm is summed over different partitions: fp32 rounding apart, the same step."""
    from ane_b200.sharded import ShardedAdam

    def checksum():
        c = params.w[:params.n].view(torch.int32).to(torch.int64).sum().reshape(1)
        lo, hi = c.clone(), c.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return int(lo[0]) == int(hi[0])

    out = {"params_equal_across_ranks": checksum()}
    if not peer_mode:
        return out
    w0 = params.w.clone()
    params.m.zero_()
    params.v.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    opt.begin_step(gscale)
    opt.step(1, gscale)
    opt.flush()
    torch.cuda.synchronize()
    dist.barrier()
    w_peer = params.w.clone()
    out["params_equal_across_ranks_after_peer_step"] = checksum()
    dist.barrier()
    params.w.copy_(w0)
    params.m.zero_()
    params.v.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    nccl = ShardedAdam(params.w, params.g, params.m, params.v, params.n_decay, params.n, world, rank,
                       lr=opt.lr, b1=opt.b1, b2=opt.b2, eps=opt.eps, wd=opt.wd, clip=opt.clip)
    nccl.step(1, gscale)
    torch.cuda.synchronize()
    dist.barrier()
    diff = (params.w[:params.n] - w_peer[:params.n]).abs().max() / w_peer[:params.n].abs().max()
    moved = (w_peer[:params.n] - w0[:params.n]).abs().max() / w0[:params.n].abs().max()
    d = torch.stack([diff, -moved]).float()
    dist.all_reduce(d, op=dist.ReduceOp.MAX)
    out["optimizer_forms_max_rel_diff"] = float(d[0])
    out["optimizer_step_moved_params_rel"] = float(-d[1])
    out["params_equal_across_ranks_after_nccl_step"] = checksum()
    return out


# ------------------------------------------------------------------------------------- main (ours)
def run_ours(args):
    import torch
    import torch.distributed as dist

    from ane_b200 import dev_ops as ops
    from ane_b200 import lib
    from ane_b200.layer_chain import ChainConfig, FlatParams, LayerChain
    from ane_b200.sharded import RegionShardedAdam, ShardedAdam, padded_length, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs CUDA devices: libane_cuda has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib.init(local)
    peak_gbs, peak_kind = measured_peak()

    cfg = ChainConfig(layers=args.layers, alpha=(2.0 * args.layers) ** -0.5, fuse_layer_boundary=not args.no_boundary_fusion)
    lo, hi = shard_range(args.seqs, world, rank)
    my_seqs = hi - lo
    M = min(args.micro_batch, max(my_seqs, 1))
    n_micro = (my_seqs + M - 1) // M
    if my_seqs % M:
        raise SystemExit(f"sequences per rank ({my_seqs}) must be a multiple of the micro-batch ({M})")

    peer_ptrs, exchange = None, "none (one rank)"
    wg = None
    if world > 1:
        exchange = "NCCL reduce-scatter and all-gather around the Adam kernel"
        if not args.no_p2p:
            try:
                from ane_b200.sharded import symmetric_buffers
                w_s, g_s, peer_ptrs = symmetric_buffers(FlatParams.padded_count(cfg, world * 256), device)
                wg = (w_s, g_s)
                exchange = "peer memory: the reduce kernel reads every rank's gradients, the Adam kernel stores the new weights to every rank"
            except Exception as exc:       # no peer mapping on this machine: the NCCL path computes the same step
                peer_ptrs, wg = None, None
                exchange += f" (peer mapping unavailable: {str(exc)[:120]})"
    params = FlatParams(cfg, device, pad_to=world * 256, wg_buffers=wg)
    params.init_random()
    chain = LayerChain(cfg, M, params, device)
    opt = ShardedAdam(params.w, params.g, params.m, params.v, params.n_decay, params.n, world, rank,
                      lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=1.0, peer_ptrs=peer_ptrs, n_early=params.n_matrix if args.early_reduce else 0)
    gscale = 1.0 / (10 * 256.0)       # 1/(accum_steps*loss_scale), train.m:750
    tstep = [0]
    use_graph = not args.no_graph
    if use_graph:
        chain.capture()
    per_mb = chain.launches_per_microbatch()
    graph_launches = [0]
    # The gradient exchange beside the backward pass: a layer's weight gradients are final once the step's last micro-batch
    # has run that layer's backward operators (in a full loop the dW contractions sit there), so the reduce of a finished
    # group of layers can run while the remaining groups are computed.  Every rank owns a share of every group.
    groups, region_of_group = None, None
    if world > 1 and peer_ptrs is not None and args.overlap_groups > 1 and not args.early_reduce:
        try:
            groups = chain.capture_segments(args.overlap_groups) if use_graph else chain.layer_groups(args.overlap_groups)
            per_layer = cfg.matrix_params_per_layer()
            edges = sorted({lo_ * per_layer for _, lo_ in groups} | {params.n_matrix, params.n_padded})
            region_of_group = [edges.index(lo_ * per_layer) for _, lo_ in groups]
            from ane_b200.sharded import symmetric_buffer
            opt = RegionShardedAdam(params.w, params.g, params.m, params.v, params.n_decay, params.n, world, rank, peer_ptrs, edges,
                                    lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=1.0,
                                    staging=symmetric_buffer(RegionShardedAdam.staging_floats(edges, world), device),
                                    deferred_broadcast=not args.no_deferred_broadcast)
            exchange = (f"peer memory: every rank owns a share of every layer group; the gradients of {len(groups) - 1} of {len(groups)} groups are pushed "
                        "to their owners by the copy engines (side stream) while the rest of the backward pass runs and are added from local "
                        "memory in rank order, the last group, embedding and norm weights are read from the peers by the reduce kernel")
            if not args.no_deferred_broadcast:
                exchange += ("; Adam writes the new weights locally, the norm weights are copied to the peers at once and the matrices and the "
                             "embedding table by the copy engines beside the next step's operator chain (landed before the next optimizer step)")
            else:
                exchange += "; the Adam kernel stores the new weights to every rank"
        except Exception as exc:       # staging memory or graph capture unavailable: the one-slice peer form computes the same step
            groups, region_of_group = None, None
            exchange += f" (exchange beside the backward pass unavailable: {str(exc)[:120]})"

    def step():
        params.zero_produced_grads()
        opt.begin_step(gscale)
        for mb in range(n_micro):
            eager = not use_graph or (mb == 0 and chain.timed_op is not None)   # the first micro-batch of a timed step runs eagerly, with events around the dominant kernel
            if groups is not None and mb == n_micro - 1:
                for i in range(len(groups)):
                    if eager:
                        chain.run_segment(groups, i)
                    else:
                        chain.segment_graphs[i].replay()
                    if i + 1 < len(groups):
                        ev = torch.cuda.Event()
                        ev.record()
                        opt.reduce_region(region_of_group[i], ev)
                if not eager:
                    graph_launches[0] += per_mb
            elif not eager:
                chain.replay()
                graph_launches[0] += per_mb
            else:
                chain.forward()
                chain.backward()
        tstep[0] += 1
        opt.step(tstep[0], gscale)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    chain.timed_op = ("swiglu_bwd", [])
    lib.reset_launch_count()
    graph_launches[0] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    timed = chain.timed_op
    opt.phase_events = []
    for i in range(args.steps):
        chain.timed_op = timed if i == 0 else None       # events around the dominant kernel in the first timed step only
        step()
    opt.flush()       # the last step's deferred weight copies land inside the timed region
    chain.timed_op = timed
    e1.record()
    barrier()
    launches = lib.launch_count() + graph_launches[0]     # graph replays do not pass through the host-side counter
    phases = {}
    for name, s_ev, e_ev in opt.phase_events:
        phases.setdefault(name, []).append(s_ev.elapsed_time(e_ev))
    opt.phase_events = None
    optimizer_ms = {k: round(statistics.mean(v), 3) for k, v in phases.items()}
    if "all_gather" in optimizer_ms:       # nested inside the update phase: report the local part on its own
        optimizer_ms["norm_clip_adam_local"] = round(optimizer_ms["norm_clip_adam_gather"] - optimizer_ms["all_gather"], 3)
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0]) / args.steps
    tokens = args.seqs * cfg.seq
    value = tokens / (ms_step * 1e-3)

    # roofline of the dominant kernel, timed live inside the timed region
    ev = chain.timed_op[1]
    chain.timed_op = None
    k_ms = statistics.mean(s.elapsed_time(e) for s, e in ev)
    k_bytes = 5 * cfg.hidden * M * cfg.seq * 2
    achieved = k_bytes / k_ms / 1e6
    roofline = {"bound": "hbm", "kernel": "ew_vec_kernel<bf16,3,2,SwigluBwdOp> (swiglu_bwd)", "achieved": round(achieved, 1),
                "peak": peak_gbs, "peak_kind": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650",
                "unit": "GB/s", "frac": round(achieved / peak_gbs, 4), "frac_of_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                "traffic": None, "launch_ms": round(k_ms, 4), "launches_timed": len(ev), "algorithmic_bytes_per_launch": k_bytes}
    # DRAM bytes of this kernel from one profiler capture at 16 sequences (dram__bytes_read + dram__bytes_write = 0.953 of
    # its algorithmic bytes: the inputs are read exactly once, part of the output is still in L2 when the kernel ends);
    # a streaming kernel's traffic grows in proportion to the elements moved, so the ratio carries to this launch size.
    roofline["traffic"] = int(SWIGLU_BWD_DRAM_BYTES_PER_ALGORITHMIC_BYTE * k_bytes)
    roofline["traffic_source"] = "ncu capture at 16 sequences, scaled by elements (profiles/swiglu_bwd_ew_vec_kernel_16seq.md)"
    # the same launch counted in DRAM bytes: what the memory system actually moved per second, against the same copy-rate peak
    roofline["achieved_dram"] = round(roofline["traffic"] / k_ms / 1e6, 1)
    roofline["frac_dram"] = round(roofline["achieved_dram"] / peak_gbs, 4)
    if roofline["frac"] > 1.0:
        roofline["note"] = ("frac > 1: the denominator is a measured plain copy (read + write), not a hardware limit; this kernel reads three "
                            "streams and writes two, part of its output is still in L2 when it ends (frac_dram), and its clocks under "
                            "load differ from those of the peak measurement.  Launched back to back for seconds under the 1000 W cap a "
                            "three-stream copy on this board sustains 6.8 TB/s (146 pJ per byte; python -m ane_b200.opbench --sustain), "
                            "which is the ceiling of a long step")

    chain_bytes = tokens * (cfg.layers * cfg.bytes_per_token_layer() + cfg.bytes_per_token_ends()) + 28 * params.n + 4 * params.n
    line = {
        "metric": "layer-op tokens/sec (Qwen3-0.6B non-matmul layer chain + Adam)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 activations / f32 math and optimizer", "data": "synthetic",
        "config": workload_config(args, world),
        "step_algorithmic_GB": round(chain_bytes / 1e9, 2),
        "step_GBps_per_gpu": round(chain_bytes / world / (ms_step * 1e-3) / 1e9, 1),
        "step_frac_of_measured_peak": round(chain_bytes / world / (ms_step * 1e-3) / 1e9 / peak_gbs, 4),
        "roofline": roofline,
        "optimizer_ms_per_step": optimizer_ms,
        "optimizer_exchange": exchange,
        "clocks": clocks,
        "gpu_launches": int(launches),
    }

    line["ms_per_step_x_sm_mhz"] = round(ms_step * clocks["sm_mhz"], 1) if clocks.get("sm_mhz") else None
    if world == 1 and not args.no_ops and use_graph:
        # the same step with the classifier loss after every micro-batch, at the compacted vocabulary (a quarter of the 151,936
        # ids: training_dynamic/cpu_ops.h:96-148 compacts to the ids in use): fp32 logits [M][37984][2048], softmax-CE forward + backward in place
        Vc = cfg.vocab // 4
        logits = torch.randn((M, Vc, cfg.seq), device=device)
        targets = torch.randint(0, Vc, (M, cfg.seq), device=device, dtype=torch.int32)

        def step_with_loss():
            params.zero_produced_grads()
            for _ in range(n_micro):
                chain.replay()
                ops.cross_entropy(logits, targets, dlogits=logits)
            tstep[0] += 1
            opt.step(tstep[0], gscale)

        step_with_loss()
        torch.cuda.synchronize()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for _ in range(2):
            step_with_loss()
        l1.record()
        torch.cuda.synchronize()
        ms_l = l0.elapsed_time(l1) / 2
        line["chain_plus_loss"] = {"value": round(tokens / (ms_l * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms_l, 3),
                                   "loss": f"softmax cross-entropy forward + backward over a compact vocabulary of {Vc} ids, fp32 logits, after every micro-batch"}
        del logits, targets
    del chain
    torch.cuda.empty_cache()
    if world > 1:
        line.update(cross_rank_checks(torch, dist, params, opt, tstep[0], gscale, world, rank, peer_ptrs is not None))
    if not args.no_ops and rank == 0 and world == 1:
        from ane_b200.opbench import per_op_table, reference_shape_table
        line["ops"] = per_op_table(torch, ops, device, peak_gbs, batch=32)
        line["ops_reference_shapes_f32"] = reference_shape_table(torch, ops, device, peak_gbs)
    if world > 1:
        dist.barrier()

    if not args.no_e2e:
        e2e_seqs = args.e2e_seqs
        tps, h2d, d2h, dt, tps_py = e2e_chain(torch, cfg, params, device, e2e_seqs, steps=2, warmup=1)
        t = torch.tensor([tps, tps_py], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        line["e2e"] = {"value": round(float(t[0]), 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                       "python_chain_value": round(float(t[1]), 1),
                       "note": f"ane_cuda_chain_step (the C ABI's chain object): {e2e_seqs} sequences x 2048 tokens per rank and step "
                               f"({dt*1e3:.0f} ms); every contraction-side tensor of every layer is copied from / to page-locked host "
                               f"memory inside the timed region ({(h2d + d2h) / dt / 1e9:.1f} GB/s over PCIe, both directions); "
                               "PCIe-bound.  python_chain_value: the same step driven by ane_b200.host_chain.HostLayerChain over torch streams"}
        torch.cuda.empty_cache()
        if True:            # how much of the per-rank PCIe rate is left when all ranks copy at once, operators aside
            if world > 1:
                dist.barrier()
            r = torch.tensor([pcie_copy_only(torch, device)], device=device)
            lo_, hi_ = r.clone(), r.clone()
            if world > 1:
                dist.all_reduce(lo_, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
            line["e2e"]["copy_only_GBps_per_rank_min_max"] = [round(float(lo_[0]), 1), round(float(hi_[0]), 1)]
            line["e2e"]["chain_GBps_per_rank"] = round((h2d + d2h) / dt / 1e9, 1)
            try:
                line["e2e"]["host"] = {"cpus_visible": len(os.sched_getaffinity(0)), "numa_nodes": len([d_ for d_ in os.listdir("/sys/devices/system/node") if d_.startswith("node")])}
            except OSError:
                pass
        if rank == 0 and world == 1 and not args.no_ops:
            tps2, h2d2, d2h2, dt2 = e2e_per_op(torch, cfg, 4, steps=1, warmup=1)
            line["e2e_per_op_calls"] = {"value": round(tps2, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d2), "d2h_bytes_per_step": int(d2h2),
                                        "note": "the same chain as one ane_cuda_*_host call per operator (4 sequences; each call stages its own "
                                                "operands, also the ones operators hand to each other)"}

    if rank == 0:
        if not args.no_cpu and world == 1:
            r = cpu_chain({"layers": args.layers, "seqs": args.seqs}, args.cpu_seqs, 1, 0)
            line["cpu_baseline"] = {"value": round(r["tokens_per_s"], 1), "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"]}
            try:
                line["cpu_reference_ops"] = cpu_reference_ops()
            except Exception as exc:       # the baseline of record is the chain above; this table is an extra
                line["cpu_reference_ops"] = {"error": str(exc)[:200]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
