"""Per-operator micro-benchmark: achieved GB/s of each device-resident operator on benchmark-sized
tensors, computed from ALGORITHMIC bytes (compulsory HBM traffic with perfect on-chip reuse) and the
CUDA-event time of a launch.

    python -m ane_b200.opbench                       # the whole table, one JSON object
    python -m ane_b200.opbench --op cross_entropy    # one operator (what a profiler run wraps)
    python -m ane_b200.opbench --op rmsnorm --batch 64 --iters 3 --tuning norm_fwd=0

Timing: CUDA events around each of 20 back-to-back launches after 5 warm-ups, median reported (best beside
it).  Every operator rotates through four input/output sets so that consecutive launches do not find their
operands in the 126 MB L2 (each set is 128 MiB or more at the default batch of 32 sequences).

    python -m ane_b200.opbench --dim 768 --hidden 2048 --seq 256 --dtype float32 --batch 1024 \
        --op rmsnorm --op rmsnorm_bwd --op swiglu --op swiglu_bwd --op residual      # Stories110M shapes
"""
from __future__ import annotations

import argparse
import json

NOMINAL_HBM_GBS = 8000.0
SEQ, DIM, HIDDEN, QD, KVD, HD, VOCAB = 2048, 1024, 3072, 2048, 1024, 128, 151936
DEFAULT_SETS = 4


def _cases(torch, ops, device, M, shape=None):
    """name -> (builder) ; builder() returns (fn(i), algorithmic bytes per launch, default iterations).
    shape: optional dict(dim=, hidden=, seq=, dtype=) for the norm / residual / SwiGLU rows (the reference-native
    Stories110M shapes are dim 768, hidden 2048, seq 256, float32)."""
    shape = shape or {}
    S, D, H = shape.get("seq", SEQ), shape.get("dim", DIM), shape.get("hidden", HIDDEN)
    bf = shape.get("dtype", torch.bfloat16)
    e = torch.empty((), dtype=bf).element_size()
    T = M * S
    NSET = shape.get("sets", DEFAULT_SETS)      # input/output sets an operator rotates through

    def mk(ch, dtype=bf, n=NSET, b=M):
        return [torch.randn((b, ch, S), device=device, dtype=dtype) for _ in range(n)]

    def norm_w():
        return torch.ones(D, device=device), torch.zeros(D, device=device)

    def head_w():
        return torch.ones(HD, device=device), torch.zeros(HD, device=device)

    def rmsnorm():
        (w, _), xs, os_ = norm_w(), mk(D), mk(D)
        return (lambda i: ops.rmsnorm(xs[i % NSET], w, out=os_[i % NSET])), 2 * D * T * e, 20

    def rmsnorm_bwd():
        (w, dw), xs, ys, os_ = norm_w(), mk(D), mk(D), mk(D)
        return (lambda i: ops.rmsnorm_bwd(ys[i % NSET], xs[i % NSET], w, dw, out=os_[i % NSET])), 3 * D * T * e, 20

    def rmsnorm_bwd_add():
        (w, dw), xs, ys, zs, os_ = norm_w(), mk(D), mk(D), mk(D), mk(D)
        return (lambda i: ops.rmsnorm_bwd(ys[i % NSET], xs[i % NSET], w, dw, add=zs[i % NSET], out=os_[i % NSET])), 4 * D * T * e, 20

    def residual_rmsnorm():
        (w, _), xs, ys, os_, o2 = norm_w(), mk(D), mk(D), mk(D), mk(D)
        return (lambda i: ops.residual_rmsnorm(xs[i % NSET], ys[i % NSET], w, 0.13, x2=os_[i % NSET], x2norm=o2[i % NSET])), 4 * D * T * e, 20

    def residual():
        xs, ys, os_ = mk(D), mk(D), mk(D)
        return (lambda i: ops.residual(xs[i % NSET], ys[i % NSET], 0.13, out=os_[i % NSET])), 3 * D * T * e, 20

    def swiglu():
        h1, h3, g1 = mk(H), mk(H), mk(H)
        return (lambda i: ops.swiglu(h1[i % NSET], h3[i % NSET], out=g1[i % NSET])), 3 * H * T * e, 20

    def swiglu_bwd():
        h1, h3, dd, g1, g3 = mk(H), mk(H), mk(H), mk(H), mk(H)
        return (lambda i: ops.swiglu_bwd(h1[i % NSET], h3[i % NSET], dd[i % NSET], dh1=g1[i % NSET], dh3=g3[i % NSET])), 5 * H * T * e, 20

    def rope():
        q, qo = mk(QD), mk(QD)
        return (lambda i: ops.rope(q[i % NSET], HD, base=1e6, out=qo[i % NSET])), 2 * QD * T * e, 20

    def qknorm_rope():
        (wq, _), q, qo = head_w(), mk(QD), mk(QD)
        return (lambda i: ops.qknorm_rope(q[i % NSET], wq, HD, out=qo[i % NSET])), 2 * QD * T * e, 20

    def rope_qknorm_bwd():
        (wq, dwq), q, dq, qo = head_w(), mk(QD), mk(QD), mk(QD)
        return (lambda i: ops.rope_qknorm_bwd(dq[i % NSET], q[i % NSET], wq, dwq, HD, out=qo[i % NSET])), 3 * QD * T * e, 20

    # the K side of the attention prep on its own (8 KV heads of 128): half the bytes of the Q side per launch
    def qknorm_rope_k():
        (wq, _), k, ko = head_w(), mk(KVD, n=2 * NSET), mk(KVD, n=2 * NSET)
        return (lambda i: ops.qknorm_rope(k[i % (2 * NSET)], wq, HD, out=ko[i % (2 * NSET)])), 2 * KVD * T * e, 20

    def rope_qknorm_bwd_k():
        (wq, dwq), k, dk, ko = head_w(), mk(KVD, n=2 * NSET), mk(KVD, n=2 * NSET), mk(KVD, n=2 * NSET)
        return (lambda i: ops.rope_qknorm_bwd(dk[i % (2 * NSET)], k[i % (2 * NSET)], wq, dwq, HD, out=ko[i % (2 * NSET)])), 3 * KVD * T * e, 20

    # Q and K of one layer in one call (what the layer chain issues): bytes of the Q and the K operator together
    def qknorm_rope_pair():
        (wq, _), q, qo, k, ko = head_w(), mk(QD), mk(QD), mk(KVD), mk(KVD)
        return (lambda i: ops.qknorm_rope_pair(q[i % NSET], k[i % NSET], wq, wq, HD, out_q=qo[i % NSET], out_k=ko[i % NSET])), 2 * (QD + KVD) * T * e, 20

    def rope_qknorm_bwd_pair():
        (wq, dwq), q, dq, qo, k, dk, ko = head_w(), mk(QD), mk(QD), mk(QD), mk(KVD), mk(KVD), mk(KVD)
        dwk = torch.zeros_like(dwq)
        return (lambda i: ops.rope_qknorm_bwd_pair(dq[i % NSET], dk[i % NSET], q[i % NSET], k[i % NSET], wq, wq, dwq, dwk, HD,
                                                   out_q=qo[i % NSET], out_k=ko[i % NSET])), 3 * (QD + KVD) * T * e, 20

    # embedding: batch sequences of 2048 tokens, table [151936, 1024] bf16
    def _embed_common():
        Be = M
        table = (0.02 * torch.randn(VOCAB, D, device=device)).to(bf)
        tok = torch.randint(0, VOCAB, (Be, S), device=device, dtype=torch.int32)
        xe = [torch.empty((Be, D, S), device=device, dtype=bf) for _ in range(2)]
        return Be, table, tok, xe

    def embed_lookup():
        Be, table, tok, xe = _embed_common()
        return (lambda i: ops.embed_lookup(table, tok, out=xe[i % 2])), Be * S * 4 + 2 * D * Be * S * e, 20

    def embed_backward():
        Be, table, tok, xe = _embed_common()
        ops.embed_lookup(table, tok, out=xe[0])
        ops.embed_lookup(table, tok, out=xe[1])
        del table
        dE = torch.zeros(VOCAB, D, device=device)
        uniq = int(torch.unique(tok).numel())
        return (lambda i: ops.embed_backward(dE, xe[i % 2], tok)), Be * S * 4 + D * Be * S * e + 2 * uniq * D * 4, 10

    # cross-entropy: fp32 logits [batch/4][151936][2048] (10 GB at the default batch), written in place
    def cross_entropy():
        Bc = max(1, M // 4)
        logits = torch.randn((Bc, VOCAB, S), device=device)
        tg = torch.randint(0, VOCAB, (Bc, S), device=device, dtype=torch.int32)
        return (lambda i: ops.cross_entropy(logits, tg, dlogits=logits)), 2 * VOCAB * Bc * S * 4, 3

    # the vocabulary after compaction to the ids a corpus uses (a quarter of the full one here)
    def cross_entropy_compact():
        Vc = VOCAB // 4
        logits = torch.randn((M, Vc, S), device=device)
        tg = torch.randint(0, Vc, (M, S), device=device, dtype=torch.int32)
        return (lambda i: ops.cross_entropy(logits, tg, dlogits=logits)), 2 * Vc * M * S * 4, 3

    # the compact vocabulary of the reference's own run (training/README.md: 9.2 k of 32 k ids in use)
    def cross_entropy_9200():
        Vc = 9200
        sets = [torch.randn((M, Vc, S), device=device) for _ in range(2)]
        tg = torch.randint(0, Vc, (M, S), device=device, dtype=torch.int32)
        return (lambda i: ops.cross_entropy(sets[i % 2], tg, dlogits=sets[i % 2])), 2 * Vc * M * S * 4, 6

    def _flat():
        n = 2 * M << 20
        wv, gv, mv, vv = (torch.randn(n, device=device) * 0.01 for _ in range(4))
        vv.abs_()
        return n, wv, gv, mv, vv

    def adam():
        n, wv, gv, mv, vv = _flat()
        return (lambda i: ops.adam(wv, gv, mv, vv, 1 + i, 3e-4, 0.9, 0.95, 1e-8, wd=0.1)), 28 * n, 20

    def grad_norm_sq():
        n, wv, gv, mv, vv = _flat()
        del wv, mv, vv
        nsq = torch.zeros(1, device=device)
        return (lambda i: ops.grad_norm_sq(gv, 1.0, out=nsq)), 4 * n, 20

    # layout helpers beside the operators (GQA 16/8 heads of 128; fp32 -> bf16 cast; compact table of a quarter of the ids)
    def gqa_tile():
        k = mk(KVD)
        o = [torch.empty((M, QD, S), dtype=bf, device=device) for _ in range(NSET)]
        return (lambda i: ops.gqa_tile(k[i % NSET], 8, 2, out=o[i % NSET])), (KVD + QD) * T * e, 20

    def gqa_reduce():
        q = mk(QD)
        o = [torch.empty((M, KVD, S), dtype=bf, device=device) for _ in range(NSET)]
        return (lambda i: ops.gqa_reduce(q[i % NSET], 8, 2, out=o[i % NSET])), (KVD + QD) * T * e, 20

    def qknorm_rope_tiled():
        (wq, _), k = head_w(), mk(KVD)
        o = [torch.empty((M, QD, S), dtype=bf, device=device) for _ in range(NSET)]
        return (lambda i: ops.qknorm_rope_tiled(k[i % NSET], wq, HD, 2, out=o[i % NSET])), (KVD + QD) * T * e, 20

    def rope_qknorm_bwd_gqa():
        (wq, dwq), k, dyt, o = head_w(), mk(KVD), mk(QD), mk(KVD)
        return (lambda i: ops.rope_qknorm_bwd_gqa(dyt[i % NSET], k[i % NSET], wq, dwq, HD, 2, out=o[i % NSET])), (QD + 2 * KVD) * T * e, 20

    def convert_f32_bf16():
        x = mk(D, dtype=torch.float32)
        o = [torch.empty((M, D, S), dtype=torch.bfloat16, device=device) for _ in range(NSET)]
        return (lambda i: ops.convert(x[i % NSET], torch.bfloat16, out=o[i % NSET])), 6 * D * T, 20

    def vocab_compact_embed():
        Vc = VOCAB // 4
        full = torch.randn(VOCAB, D, device=device)
        tok = (torch.randperm(VOCAB, device=device)[:Vc]).to(torch.int32).repeat(2)
        f2c, c2f, cnt = ops.vocab_map_build(tok, VOCAB)
        out = [torch.empty((Vc, D), device=device) for _ in range(2)]
        return (lambda i: ops.vocab_compact_embed(full, c2f, cnt, Vc, out=out[i % 2])), 2 * Vc * D * 4 + Vc * 4, 20

    return {
        "gqa_tile": gqa_tile, "gqa_reduce": gqa_reduce, "qknorm_rope_tiled(K)": qknorm_rope_tiled,
        "rope_qknorm_bwd_gqa(K)": rope_qknorm_bwd_gqa, "convert_f32_bf16": convert_f32_bf16,
        "vocab_compact_embed": vocab_compact_embed,
        "rmsnorm": rmsnorm, "rmsnorm_bwd": rmsnorm_bwd, "rmsnorm_bwd_add": rmsnorm_bwd_add,
        "residual_rmsnorm": residual_rmsnorm, "residual": residual, "swiglu": swiglu, "swiglu_bwd": swiglu_bwd,
        "rope": rope, "qknorm_rope(Q)": qknorm_rope, "rope_qknorm_bwd(Q)": rope_qknorm_bwd,
        "qknorm_rope(K)": qknorm_rope_k, "rope_qknorm_bwd(K)": rope_qknorm_bwd_k,
        "qknorm_rope(Q+K)": qknorm_rope_pair, "rope_qknorm_bwd(Q+K)": rope_qknorm_bwd_pair,
        "embed_lookup": embed_lookup, "embed_backward": embed_backward,
        "cross_entropy": cross_entropy, "cross_entropy_compact": cross_entropy_compact, "cross_entropy_9200": cross_entropy_9200,
        "adam": adam, "grad_norm_sq": grad_norm_sq,
    }


def time_op(torch, builder, peak_gbs, iters=None, warmup=5):
    """CUDA events around every one of `iters` back-to-back launches after `warmup` untimed ones; the reported time
    is the median launch (the best one is given beside it)."""
    fn, nbytes, default_iters = builder()
    iters = iters or default_iters
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    ev[0].record()
    for i in range(iters):
        fn(i)
        ev[i + 1].record()
    torch.cuda.synchronize()
    per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(iters))
    ms = per[len(per) // 2]
    gbs = nbytes / ms / 1e6
    return {"ms": round(ms, 4), "ms_best": round(per[0], 4), "GB/s": round(gbs, 1), "frac_measured": round(gbs / peak_gbs, 3),
            "frac_8TBs": round(gbs / NOMINAL_HBM_GBS, 3), "bytes": nbytes}


def sustain_op(torch, builder, peak_gbs, seconds):
    """The operator launched back to back for `seconds`, with the board power and the SM clock sampled through NVML every
    50 ms (the first third of the samples, while the clocks settle, is dropped).  A 20-launch timing shows what the kernel does
    at the clock the GPU happens to hold; this shows what it does once the 1000 W power cap has set the clock -- the state a
    long training step runs in -- and what a byte costs in energy (power x time / algorithmic bytes)."""
    import threading
    import time
    import pynvml
    pynvml.nvmlInit()
    handle = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    fn, nbytes, _ = builder()
    for i in range(10):
        fn(i)
    torch.cuda.synchronize()
    samples, stop = [], threading.Event()

    def sampler():
        while not stop.is_set():
            samples.append((pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0, pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
            time.sleep(0.05)

    th = threading.Thread(target=sampler)
    th.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.perf_counter()
    e0.record()
    while time.perf_counter() - t0 < seconds:
        for i in range(200):
            fn(n + i)
        n += 200
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    stop.set()
    th.join()
    ms = e0.elapsed_time(e1) / n
    kept = samples[len(samples) // 3:] or samples or [(0.0, 0)]
    watts = sum(p for p, _ in kept) / len(kept)
    mhz = sorted(c for _, c in kept)[len(kept) // 2]
    gbs = nbytes / ms / 1e6
    return {"ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_measured": round(gbs / peak_gbs, 3), "frac_8TBs": round(gbs / NOMINAL_HBM_GBS, 3),
            "power_w": round(watts), "sm_mhz": mhz, "pJ_per_byte": round(watts * ms * 1e-3 / nbytes * 1e12, 1), "launches": n, "bytes": nbytes}


def per_op_table(torch, ops, device, peak_gbs, batch=32, only=None, iters=None, warmup=5, shape=None, sustain=0.0):
    """Achieved GB/s per operator on benchmark-sized bf16 tensors (algorithmic bytes / time)."""
    res = {}
    for name, builder in _cases(torch, ops, device, batch, shape).items():
        if only and name not in only:
            continue
        res[name] = sustain_op(torch, builder, peak_gbs, sustain) if sustain > 0 else time_op(torch, builder, peak_gbs, iters, warmup)
        torch.cuda.empty_cache()
    return res


REFERENCE_SHAPE_OPS = ("rmsnorm", "rmsnorm_bwd", "rmsnorm_bwd_add", "residual_rmsnorm", "residual", "swiglu", "swiglu_bwd")


def reference_shape_table(torch, ops, device, peak_gbs, batches=(1, 64, 1024, 4096)):
    """The norm / residual / SwiGLU rows at the reference's own shapes (Stories110M: fp32, DIM 768, HIDDEN 2048, SEQ 256;
    stories_config.h), batched over B sequences.  B = 1 is one reference call: everything fits in L2, so the row is a
    latency (its GB/s is not an HBM figure); at B = 1024 and 4096 a tensor is 0.8-8.6 GB and fewer buffer sets are
    rotated (every launch still reads data last touched gigabytes earlier)."""
    out = {}
    for B in batches:
        sets = 4 if B <= 64 else 2 if B <= 1024 else 1
        shape = dict(dim=768, hidden=2048, seq=256, dtype=torch.float32, sets=sets)
        rows = per_op_table(torch, ops, device, peak_gbs, batch=B, only=REFERENCE_SHAPE_OPS, iters=10 if B >= 1024 else 20, shape=shape)
        if B == 1:
            rows = {k: {"latency_us": round(v["ms"] * 1e3, 2), "latency_us_best": round(v["ms_best"] * 1e3, 2), "bytes": v["bytes"]}
                    for k, v in rows.items()}
        out[f"B={B}"] = rows
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", action="append", help="operator name (repeatable); default: all")
    ap.add_argument("--batch", type=int, default=32, help="sequences of 2048 tokens per launch")
    ap.add_argument("--dim", type=int, default=None, help="channels of the norm / residual rows (default 1024)")
    ap.add_argument("--hidden", type=int, default=None, help="channels of the SwiGLU rows (default 3072)")
    ap.add_argument("--seq", type=int, default=None, help="tokens per sequence (default 2048)")
    ap.add_argument("--dtype", default=None, choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--sets", type=int, default=None, help="buffer sets to rotate through (default 4; fewer for multi-GB tensors)")
    ap.add_argument("--iters", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--peak-gbs", type=float, default=None, help="roofline denominator (default: MEASURED_PEAKS.json)")
    ap.add_argument("--tuning", default="", help="comma-separated knob=value pairs")
    ap.add_argument("--sustain", type=float, default=0.0, help="launch every operator back to back for this many seconds and "
                    "report time, board power, SM clock and energy per byte under the power cap instead of the 20-launch timing")
    a = ap.parse_args(argv)
    import torch
    from . import dev_ops as ops, lib
    from .peaks import hbm_peak_gbs

    if not torch.cuda.is_available():
        raise SystemExit("opbench needs a CUDA device")
    lib.init(0)
    for item in filter(None, a.tuning.split(",")):
        k, _, v = item.partition("=")
        lib.set_tuning(k, int(v))
    peak, kind = hbm_peak_gbs()
    if a.peak_gbs:
        peak, kind = a.peak_gbs, "given"
    shape = {k: v for k, v in (("dim", a.dim), ("hidden", a.hidden), ("seq", a.seq), ("sets", a.sets)) if v}
    if a.dtype:
        shape["dtype"] = getattr(torch, a.dtype)
    table = per_op_table(torch, ops, torch.device("cuda:0"), peak, a.batch, a.op, a.iters, a.warmup, shape or None, a.sustain)
    print(json.dumps({"batch": a.batch, "peak_gbs": peak, "peak_kind": kind, "sustain_s": a.sustain, "ops": table}))


if __name__ == "__main__":
    main()
