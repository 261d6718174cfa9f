"""Worker for the tensor-parallel GPU tests (run under torchrun, one rank per GPU).

Checks the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels bit for
bit against the same GEMM kernel around library collectives (with the
kernel's own order of summation), then the sharded model against the
unsharded one, and prints ``TP_GPU_OK`` on rank 0. With ``--bench`` it also
times the fused kernels against the library path on Llama-3-8B shapes.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sga_b200 import kernels as K  # noqa: E402
from sga_b200.models.gpt import GPT, get_config  # noqa: E402
from sga_b200.parallel.tp import TPContext  # noqa: E402


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def bf(*shape, dev, scale=1.0):
    return (torch.randn(*shape, device=dev) * scale).to(torch.bfloat16)


def check_ag(tp, dev, M, N, Kd, b_mn):
    W_ = tp.world
    slot = tp.slot(("t_ag", M, Kd), M, Kd)
    Wt = bf(Kd, N, dev=dev, scale=0.1) if b_mn else bf(N, Kd, dev=dev, scale=0.1)
    for rep in range(3):
        x = bf(M // W_, Kd, dev=dev)
        slot.local.copy_(x)
        torch.cuda.synchronize()
        dist.barrier()
        y = tp.ag_linear(slot, Wt, b_mn=b_mn)
        torch.cuda.synchronize()
        tp.check()
        full = torch.cat(gather(x), 0)
        assert torch.equal(slot.full, full), f"gathered rows differ (rep {rep})"
        ref = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        K.gemm_bf16(full, Wt, ref, b_mn=b_mn)
        assert torch.equal(y, ref), f"ag_gemm differs from the GEMM of the gathered input (rep {rep})"
        dist.barrier()


def check_rs(tp, dev, M, N, Kd, b_mn, with_res):
    W_, rank = tp.world, tp.rank
    rows = M // W_
    Wt = bf(Kd, N, dev=dev, scale=0.1) if b_mn else bf(N, Kd, dev=dev, scale=0.1)
    for rep in range(3):
        a = bf(M, Kd, dev=dev)
        res = bf(rows, N, dev=dev) if with_res else None
        dist.barrier()
        y = tp.linear_rs(a, Wt, b_mn=b_mn, residual=res)
        torch.cuda.synchronize()
        tp.check()
        part = torch.empty(M, N, dtype=torch.float32, device=dev)
        K.gemm_bf16(a, Wt, part, b_mn=b_mn, epi=K.EPI_F32)
        parts = gather(part)
        lo = rank * rows
        exp = parts[rank][lo:lo + rows].clone()
        for s in range(W_):
            if s != rank:
                exp += parts[s][lo:lo + rows].to(torch.bfloat16).float()
        if res is not None:
            exp += res.float()
        exp = exp.to(torch.bfloat16)
        assert torch.equal(y, exp), (f"gemm_rs differs (rep {rep}, b_mn={b_mn}, res={with_res}): "
                                     f"{(y.float() - exp.float()).abs().max().item()}")
        dist.barrier()


def check_model(tp, dev):
    # heads and FFN columns divide over the ranks; B * S rows are a multiple of 256 per rank
    W_ = tp.world
    cfg = get_config("test_tiny", seq_len=128 * W_, n_heads=max(4, W_), n_kv_heads=max(2, W_),
                     hidden=32 * max(4, W_), ffn=256 * max(1, W_ // 2))
    model = GPT(cfg, device=dev, seed=5, tp=tp)
    full = GPT(cfg, device=dev, seed=5)
    g = torch.Generator().manual_seed(21)
    toks = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=g).to(dev)
    before = tp.launches
    l_tp = model.forward_backward(toks[:, :-1], toks[:, 1:])
    l_full = full.forward_backward(toks[:, :-1], toks[:, 1:])
    torch.cuda.synchronize()
    tp.check()
    assert tp.launches - before == 8 * cfg.num_layers
    assert abs(float(l_tp) - float(l_full)) < 5e-3 * max(1.0, float(l_full)), (float(l_tp), float(l_full))
    for slot in model.arena.slots:
        ref = full.arena.by_name[slot.name].grad
        if slot.spec.tp_pieces is not None:
            dim = slot.spec.tp_pieces[0][0]
            ref = torch.cat([ref.narrow(dim, lo, hi - lo) for _, lo, hi in slot.spec.tp_pieces], dim)
        err = float((slot.grad - ref).abs().max())
        scale = float(ref.abs().max()) + 1e-8
        assert err <= 0.08 * scale + 1e-6, (slot.name, err, scale)
    return float(l_tp), float(l_full)


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def bench(dev, rank):
    """Llama-3-8B linears at tp=2, 8192 tokens: fused kernels vs library collectives around the same GEMM."""
    fused = TPContext(device=dev, transport="fused")
    libc = TPContext(device=dev, transport="library")
    W_ = fused.world
    M, H, QKV, F2, F_ = 8192, 4096, 6144 // W_, 2 * 14336 // W_, 14336 // W_
    rows = []
    for name, Kd, N in (("qkv (all-gather -> GEMM)", H, QKV), ("fc1 (all-gather -> GEMM)", H, F2)):
        Wt = bf(N, Kd, dev=dev, scale=0.05)
        res = {}
        for tag, ctx in (("fused", fused), ("library", libc)):
            slot = ctx.slot(("b", Kd), M, Kd)
            slot.local.copy_(bf(M // W_, Kd, dev=dev))
            res[tag] = timed(lambda: ctx.ag_linear(slot, Wt))
        flops = 2.0 * M * N * Kd
        rows.append({"op": name, "M": M, "N": N, "K": Kd, "fused_ms": round(res["fused"], 4),
                     "library_ms": round(res["library"], 4), "fused_TFLOPs": round(flops / res["fused"] / 1e9, 1),
                     "nvlink_GBps_fused": round((W_ - 1) * (M // W_) * Kd * 2 / res["fused"] / 1e6, 1)})
    for name, Kd, N in (("proj (GEMM -> reduce-scatter)", H // W_, H), ("fc2 (GEMM -> reduce-scatter)", F_, H)):
        Wt = bf(N, Kd, dev=dev, scale=0.05)
        a = bf(M, Kd, dev=dev)
        r = bf(M // W_, N, dev=dev)
        res = {}
        for tag, ctx in (("fused", fused), ("library", libc)):
            res[tag] = timed(lambda: ctx.linear_rs(a, Wt, residual=r))
        flops = 2.0 * M * N * Kd
        rows.append({"op": name, "M": M, "N": N, "K": Kd, "fused_ms": round(res["fused"], 4),
                     "library_ms": round(res["library"], 4), "fused_TFLOPs": round(flops / res["fused"] / 1e9, 1),
                     "nvlink_GBps_fused": round((W_ - 1) * (M // W_) * N * 2 / res["fused"] / 1e6, 1)})
    fused.check()
    if rank == 0:
        for r in rows:
            print("TP_BENCH " + json.dumps(r), flush=True)
    fused.close()


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank()
    torch.manual_seed(7 + rank)
    tp = TPContext(device=dev, transport="fused")
    # the fused kernels work on CTA-pair tiles of 256 rows per rank's chunk: M is a multiple of 256 * ranks
    unit = 256 * tp.world
    for b_mn in (False, True):
        check_ag(tp, dev, 2 * unit, 384, 256, b_mn)
        check_ag(tp, dev, 4 * unit, 1024, 160, b_mn)
    for b_mn in (False, True):
        for with_res in (False, True):
            check_rs(tp, dev, 2 * unit, 384, 320, b_mn, with_res)
    check_rs(tp, dev, 4 * unit, 128, 1024, False, True)
    losses = check_model(tp, dev)
    dist.barrier()
    if rank == 0:
        print("tp model loss (sharded, unsharded):", losses)
        print("TP_GPU_OK", flush=True)
    if "--bench" in sys.argv:
        bench(dev, rank)
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
