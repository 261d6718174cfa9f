"""Device-timed micro-benchmarks of the native kernels with their roofline
fractions: ``python -m sga_b200.utils.kernel_bench --kernel attention|gemm|adam|
index_sync|elementwise|replay [--small]``.

Each case warms up, then times with CUDA events on the launching stream
between synchronisations, on inputs larger than the 126 MB L2 (or flushes L2
between iterations when they are not), and prints one JSON line with the
achieved rate and its fraction of the measured peak (``MEASURED_PEAKS.json``
beside the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).
``--small`` keeps the footprint to a few GB and a handful of launches so the
same command can run under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return p["hbm_gbs"] * 1e9, p["bf16_tflops"] * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


def timed(fn, iters, warmup=3, flush=None, pre=None):
    """Mean device time of ``fn`` over ``iters`` launches. Every launch is bracketed by its own pair
    of events, and the whole series is enqueued before the one synchronisation at the end, so the
    host's launch latency hides behind the previous kernel (or the L2 flush) instead of being timed
    as an idle GPU."""
    for _ in range(warmup):
        if pre is not None:
            pre()
        fn()
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    pad = flush if flush is not None else None
    for s, e in pairs:
        if pad is not None:
            pad.zero_()
        if pre is not None:
            pre()  # untimed set-up of the launch (restores its input)
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in pairs) / iters


def emit(kernel, case, ms, bytes_=None, flops=None, **extra):
    bw, tf, src = peaks()
    rec = {"kernel": kernel, "case": case, "ms": round(ms, 4)}
    if bytes_ is not None:
        rec["GBps"] = round(bytes_ / ms / 1e6, 1)
        rec[f"frac_of_{src}_hbm"] = round(bytes_ / (ms / 1e3) / bw, 3)
    if flops is not None:
        rec["TFLOPs"] = round(flops / ms / 1e9, 1)
        rec[f"frac_of_{src}_bf16"] = round(flops / (ms / 1e3) / tf, 3)
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def bench_gemm(small):
    from .. import kernels as K

    dev = "cuda"
    shapes = [("fwd qkv+o", 8192, 3072, 2048, 0, 0, 0), ("fwd fc1", 8192, 16384, 2048, 0, 0, 0),
              ("fwd fc2", 8192, 2048, 8192, 0, 0, 0), ("dgrad fc1", 8192, 2048, 16384, 0, 1, 0),
              ("wgrad fc1", 16384, 2048, 8192, 1, 1, 2), ("lm head", 8192, 128256, 2048, 0, 0, 0),
              ("square", 8192, 8192, 8192, 0, 0, 0)]
    if small:
        shapes = [("fwd fc1", 8192, 16384, 2048, 0, 0, 0)]
    for name, M, N, Kd, a_mn, b_mn, epi in shapes:
        A = torch.randn((Kd, M) if a_mn else (M, Kd), device=dev).to(torch.bfloat16)
        B = torch.randn((Kd, N) if b_mn else (N, Kd), device=dev).to(torch.bfloat16)
        C = torch.zeros(M, N, device=dev, dtype=torch.bfloat16 if epi == 0 else torch.float32)
        for pair in (True,) if small else (False, True):
            ms = timed(lambda: K.gemm_bf16(A, B, C, a_mn=bool(a_mn), b_mn=bool(b_mn), epi=epi, pair=pair),
                       2 if small else 20, warmup=1 if small else 3)
            emit("gemm_bf16_pair" if pair else "gemm_bf16", f"{name} M={M} N={N} K={Kd}", ms, flops=2.0 * M * N * Kd)
        if not small:
            At, Bt = (A.t() if a_mn else A), (B.t() if b_mn else B)
            ms = timed(lambda: torch.matmul(At, Bt.t()), 20)
            emit("library matmul (reference point)", f"{name} M={M} N={N} K={Kd}", ms, flops=2.0 * M * N * Kd)
    assert int(K.gemm_err_word(dev).item()) == 0


def bench_adam(small):
    from .. import kernels as K

    n = (64 if small else 256) * 1024 * 1024
    dev = "cuda"
    w, g, m, v = (torch.randn(n, device=dev) * 1e-2 for _ in range(4))
    v.abs_()
    model = torch.empty(n, dtype=torch.bfloat16, device=dev)
    table = K.SegmentTable([0], [0], n, dev)
    ms = timed(lambda: K.adam_step(w, g, m, v, table, [3e-4], [0.1], beta1=0.9, beta2=0.95, eps=1e-8, step=3,
                                   model=model, clear=True), 2 if small else 10, warmup=1)
    emit("sga_adam_kernel", f"n={n} sparse-step form (read w,g,m,v; write w,m,v,g,bf16)", ms, bytes_=n * 34.0)


def bench_index_sync(small):
    from ..parallel import p2p
    from ..parallel.symm import SymmPool

    pool = SymmPool(device="cuda:0")
    ch = p2p.PeerChannel(pool)
    # up to the bucket size the training step uses for this mode (1.24 G parameters in 7 buckets of about 176 M)
    for mi in ((32,) if small else (8, 16, 32, 64, 128, 168)):
        _index_sync_case(pool, ch, p2p, mi * 1024 * 1024, small)
    pool.close()


def _index_sync_case(pool, ch, p2p, n, small):
    k = n // 100
    acc0 = torch.randn(n, device="cuda") * 1e-3
    acc = acc0.clone()
    slots = p2p.IndexSyncSlots(pool, k, n)
    comm = torch.zeros(n, device="cuda")
    scratch = p2p.IndexSyncScratch("cuda:0", n)
    sq = torch.zeros(1, device="cuda")

    def restore():
        acc.copy_(acc0)   # the launch zeroes what it selects; also pushes the bucket out of L2
        comm.zero_()

    def run():
        p2p.bucket_index_sync_(ch, scratch, acc, k, slots=slots, comm=comm, scale=1.0, sumsq_out=sq)

    ms = timed(run, 2 if small else 10, warmup=1, pre=restore)
    ch.check()
    cands = int(scratch.state[2].item())
    # bound of the path as the step accounts it: three reads of the bucket + the payload written,
    # read back and scattered; the chain itself reads the bucket once
    emit("index_sync chain (sample, filter, digits, count, emit, reduce)", f"n={n} k={k} (1 rank)", ms,
         bytes_=n * 4.0 * 3 + k * 8.0 * 3, frac_of_one_pass_bound=round((n * 4.0 + k * 8.0 * 3) / (ms / 1e3) / peaks()[0], 3),
         candidates=cands)


def bench_elementwise(small):
    from ..ops import functional as F

    T, H, Fd = 8192, 2048, 8192
    dev = "cuda"
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(T, H, device=dev).to(torch.bfloat16)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    it = 2 if small else 20
    y, rstd = F.rmsnorm_fwd(x, w, 1e-5)
    emit("rmsnorm_fwd_kernel", f"T={T} H={H}", timed(lambda: F.rmsnorm_fwd(x, w, 1e-5, out=y), it, flush=flush),
         bytes_=T * H * 4.0)
    dw = torch.zeros(H, device=dev)
    dx = torch.empty_like(x)
    emit("rmsnorm_bwd_kernel", f"T={T} H={H}",
         timed(lambda: F.rmsnorm_bwd(x, w, dy, rstd, dw_out=dw, dx_out=dx), it, flush=flush), bytes_=T * H * 6.0)
    gu = torch.randn(T, 2 * Fd, device=dev).to(torch.bfloat16)
    out = torch.empty(T, Fd, device=dev, dtype=torch.bfloat16)
    emit("swiglu_fwd_kernel", f"T={T} F={Fd}", timed(lambda: F.swiglu_fwd(gu, out=out), it, flush=flush),
         bytes_=T * Fd * 6.0)
    din = torch.empty_like(gu)
    emit("swiglu_bwd_kernel", f"T={T} F={Fd}", timed(lambda: F.swiglu_bwd(gu, out, out=din), it, flush=flush),
         bytes_=T * Fd * 10.0)
    qkv = torch.randn(T, 3072, device=dev).to(torch.bfloat16)
    cs, sn = F.rope_tables(2048, 64, 500000.0, dev)
    emit("rope_kernel", f"T={T} heads=40 hd=64", timed(lambda: F.rope_(qkv, cs, sn, 2048, 40, 64, 0, 1.0), it,
                                                       flush=flush), bytes_=T * 2560 * 4.0)
    if not small:
        bench_ce(False)


def bench_ce(small):
    """Fused cross-entropy forward + backward over bf16 logits, in place (2.1 GB of logits at the Llama-3
    vocabulary: larger than L2 by itself)."""
    from ..ops import functional as F

    dev = "cuda"
    T, V = (4096 if small else 8192), 128256
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    z = torch.randn(T, V, device=dev, dtype=torch.bfloat16)
    tgt = torch.randint(0, V, (T,), device=dev)
    # the logits are read once (a row's second visit comes from L2 / shared memory) and overwritten with
    # their gradient in place: 2 B read + 2 B written per element
    emit("ce_fwd_bwd_kernel", f"T={T} V={V}", timed(lambda: F.cross_entropy_(z, tgt, 1.0 / T), 2 if small else 5,
                                                     warmup=1 if small else 3, flush=flush), bytes_=T * V * 4.0)


def bench_peer(small):
    """The fused peer-memory kernels on one rank (peer = self): their local work without the link.
    Reduce-scatter form of the all-reduce, mask-union reduce, sharded AdamW + bf16 parameter push."""
    from .. import kernels as K
    from ..parallel import p2p
    from ..parallel.symm import SymmPool

    dev = "cuda"
    n = (48 if small else 64) * 1024 * 1024   # 192 MB of fp32 even in the small case: larger than L2
    pool = SymmPool(device="cuda:0")
    ch = p2p.PeerChannel(pool)
    it = 2 if small else 10
    buf = pool.alloc(4 * n)
    buf.view(torch.float32, 0, n).normal_()
    sq = torch.zeros(1, device=dev)
    ms = timed(lambda: p2p.allreduce_(ch, buf, 0, n, scale=0.5, rs_only=True, sumsq_out=sq), it, warmup=1)
    emit("p2p_allreduce_kernel (rs_only)", f"n={n} fp32 (1 rank: read, scale, write back, norm)", ms, bytes_=n * 8.0)
    nw = (n + 31) // 32
    grad, bits, ubits = pool.alloc(4 * n), pool.alloc(4 * nw), pool.alloc(4 * nw)
    grad.view(torch.float32, 0, n).normal_()
    sel = (torch.rand(nw, 32, device=dev) < 0.0625).to(torch.int64)
    words = (sel << torch.arange(32, device=dev)).sum(1)
    bits.view(torch.int32, 0, nw).copy_((words - (words >= 2 ** 31).to(torch.int64) * 2 ** 32).to(torch.int32))
    del sel, words
    mu8 = torch.empty(n, dtype=torch.uint8, device=dev)
    ms = timed(lambda: p2p.mask_union_reduce_(ch, grad, 0, bits, 0, ubits, 0, n, scale=0.5, mask_u8=mu8, sumsq_out=sq),
               it, warmup=1)
    # mask words read and written, 1/16 of the entries read and written back (32-byte sectors: about
    # 40 % of the bucket's sectors are touched), the byte mask written
    emit("p2p_mask_union_kernel", f"n={n} fp32, 6 % of the entries in the union (1 rank)", ms,
         bytes_=n * (2 / 8.0 + 1.0 + 0.4 * 8.0))
    w, g, m, v = (torch.randn(n, device=dev) * 1e-3 for _ in range(4))
    v.abs_()
    model = pool.alloc(2 * n)
    table = K.SegmentTable([0], [0], n, dev)
    bs = torch.tensor([0], dtype=torch.int64, device=dev)
    bl = torch.tensor([n], dtype=torch.int64, device=dev)
    ms = timed(lambda: p2p.dense_adamw_ag_(ch, w, g, m, v, model, bs, bl, table, [3e-4], [0.1], beta1=0.9, beta2=0.95,
                                           eps=1e-8, step=3), it, warmup=1)
    emit("dense_adamw_ag_kernel", f"n={n} (1 rank: read w,g,m,v; write w,m,v and the bf16 copy)", ms, bytes_=n * 30.0)
    ch.check()
    pool.close()


def bench_replay(small):
    import ctypes

    from .. import kernels as _k  # noqa: F401  (declares the launchers' argument types)
    from ..csrc import lib
    from ..replay.fused import _CfgStruct

    L = lib()
    R, n = 18, (8 if small else 64) * 1024 * 1024
    dev = "cuda"
    g = (torch.randn(n, device=dev) * 1e-3).to(torch.bfloat16)
    W, M, V, RES = (torch.randn(R, n, device=dev) * 1e-3 for _ in range(4))
    V.abs_()
    SEL = (torch.rand(R, n, device=dev) < 0.01).to(torch.uint8)
    wd = torch.full((n,), 0.1, device=dev)
    arr = (_CfgStruct * R)()
    for r in range(R):
        arr[r].boundary, arr[r].coef, arr[r].lr, arr[r].bc1, arr[r].bc2, arr[r].fold_div = r % 3 == 0, 0.9, 3e-4, 0.5, 0.4, 4.0
    cfg = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev)
    nb = L.sga_replay_blocks()
    partials = torch.zeros(R * nb, dtype=torch.float64, device=dev)
    out = torch.zeros(R, dtype=torch.float64, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    def p3():
        assert L.sga_replay_pass3(g.data_ptr(), 1, 1.0, W.data_ptr(), M.data_ptr(), V.data_ptr(), RES.data_ptr(),
                                  SEL.data_ptr(), wd.data_ptr(), None, cfg.data_ptr(), R, n, 0.9, 0.1, 0.95, 0.05,
                                  1e-8, None, None, st) == 0

    ms = timed(p3, 2 if small else 5, warmup=1)
    emit("replay_pass3_kernel", f"R={R} n={n} bf16 g", ms, bytes_=n * (2.0 + 4.0 + R * 33.0))


def bench_attention(small):
    from ..ops import attention as A

    dev = "cuda"
    cases = [(4, 2048, 32, 8, 64)] if small else [(4, 2048, 32, 8, 64), (2, 4096, 16, 8, 128), (1, 4096, 32, 8, 128)]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # the operands fit in L2: flush it
    for B, S, nq, nkv, hd in cases:
        T = B * S
        qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=dev).to(torch.bfloat16)
        dctx = torch.randn(T, nq * hd, device=dev).to(torch.bfloat16)
        fl_f = 4.0 * B * nq * hd * S * S / 2
        for impl in ("native", "library"):
            A._IMPL = impl
            ctx, saved = A.attn_fwd(qkv, B, S, nq, nkv, hd)
            it = 2 if small else 10
            ms_f = timed(lambda: A.attn_fwd(qkv, B, S, nq, nkv, hd), it, warmup=1 if small else 3, flush=flush)
            dq = torch.empty_like(qkv)
            ms_b = timed(lambda: A.attn_bwd(dctx, qkv, saved, B, S, nq, nkv, hd, dq), it, warmup=1 if small else 3,
                         flush=flush)
            name = "attn_fwd_kernel" if impl == "native" else "library flash fwd (reference point)"
            emit(name, f"B={B} S={S} heads={nq}:{nkv} hd={hd} causal", ms_f, flops=fl_f)
            name = "attn_dq+dkv kernels" if impl == "native" else "library flash bwd (reference point)"
            emit(name, f"B={B} S={S} heads={nq}:{nkv} hd={hd} causal (2.5x forward FLOPs)", ms_b, flops=2.5 * fl_f)
        A._IMPL = "auto"


def bench_mask_stats(small):
    """Support count and position checksums of a byte mask (the consistency checks' kernel): 1 byte per element."""
    from .. import kernels as K

    n = (64 if small else 512) * 1024 * 1024
    mask = (torch.rand(n, device="cuda") < 0.01).to(torch.uint8)
    out = torch.zeros(3, dtype=torch.int64, device="cuda")
    ms = timed(lambda: K.mask_stats(mask, out), 2 if small else 10, warmup=1)
    emit("mask_stats_kernel", f"n={n} 1% set", ms, bytes_=float(n))


CASES = {"mask_stats": bench_mask_stats, "attention": bench_attention, "gemm": bench_gemm, "adam": bench_adam, "index_sync": bench_index_sync, "elementwise": bench_elementwise,
         "replay": bench_replay, "peer": bench_peer, "ce": bench_ce}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", choices=["all"] + sorted(CASES))
    ap.add_argument("--small", action="store_true")
    ns = ap.parse_args(argv)
    for name, fn in CASES.items():
        if ns.kernel == name or (ns.kernel == "all" and name != "ce"):  # "elementwise" already runs the CE case
            fn(ns.small)
    return 0


if __name__ == "__main__":
    sys.exit(main())
