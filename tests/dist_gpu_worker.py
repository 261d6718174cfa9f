"""Worker for the multi-GPU tests (run under torchrun, one rank per GPU).

Checks the peer-memory kernels against references built from NCCL
all-gathers with the same fixed rank order of summation (so results must be
bit-identical), then steps the tiny model through every synchronisation path
and checks that all ranks hold identical parameters afterwards.
Prints ``DIST_GPU_OK`` on rank 0 when everything passed.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sga_b200 import kernels_torch as KT  # noqa: E402
from sga_b200.parallel import p2p  # noqa: E402
from sga_b200.parallel.symm import SymmPool  # noqa: E402


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def pack_bits_np(mask_bool):
    packed = np.packbits(mask_bool.cpu().numpy().astype("uint8"), bitorder="little")
    packed = np.concatenate([packed, np.zeros((-len(packed)) % 4, dtype="uint8")]).view("int32")
    return torch.from_numpy(packed.copy())


def check_kernels(rank, world, dev):
    pool = SymmPool(device=dev)
    ch = p2p.PeerChannel(pool)
    n = 300007
    torch.manual_seed(100 + rank)
    # ---- all-reduce
    buf = pool.alloc(4 * n)
    v = buf.view(torch.float32, 0, n)
    x = torch.randn(n, device=dev)
    v.copy_(x)
    sq = torch.zeros(1, device=dev)
    dist.barrier()
    p2p.allreduce_(ch, buf, 0, n, scale=1.0 / world, sumsq_out=sq)
    torch.cuda.synchronize()
    ch.check("allreduce")
    xs = gather(x)
    ref = xs[0].clone()
    for r in range(1, world):
        ref += xs[r]
    ref *= 1.0 / world
    assert torch.equal(v, ref), "p2p all-reduce differs from the rank-ordered sum"
    sqs = gather(sq)
    assert all(torch.equal(sqs[0], s) for s in sqs), "norm must be identical on every rank"
    assert abs(sq.item() - (ref.double() ** 2).sum().item()) <= 1e-4 * sq.item()
    # ---- reduce-scatter only
    v.copy_(x)
    dist.barrier()
    p2p.allreduce_(ch, buf, 0, n, scale=1.0 / world, rs_only=True)
    torch.cuda.synchronize()
    ch.check("reduce-scatter")
    n4 = (n + 3) // 4
    per = (n4 + world - 1) // world
    lo, hi = min(n, per * rank * 4), min(n, per * (rank + 1) * 4)
    assert torch.equal(v[lo:hi], ref[lo:hi])
    # ---- mask union reduce
    gb = pool.alloc(4 * n)
    nw = (n + 31) // 32
    bb, ub = pool.alloc(4 * nw), pool.alloc(4 * nw)
    g = gb.view(torch.float32, 0, n)
    g.copy_(x)
    m = torch.rand(n, device=dev) < 0.03
    bb.view(torch.int32, 0, nw).copy_(pack_bits_np(m))
    mu8 = torch.empty(n, dtype=torch.uint8, device=dev)
    dist.barrier()
    p2p.mask_union_reduce_(ch, gb, 0, bb, 0, ub, 0, n, scale=1.0 / world, mask_u8=mu8, sumsq_out=sq)
    torch.cuda.synchronize()
    ch.check("mask union")
    ms = gather(m.to(torch.uint8))
    union = ms[0].clone()
    for r in range(1, world):
        union |= ms[r]
    assert torch.equal(mu8, union)
    exp = torch.where(union.bool(), ref, x)
    assert torch.equal(g, exp), "masked entries must hold the mean, the rest the local value"
    # ---- bucket index sync (exact rank-local top-k, (idx, val) exchange, ordered scatter-add)
    for nb, k in ((200003, 2000), (3 * (1 << 20) + 5, 40000)):
        acc = torch.randn(nb, device=dev) * 1e-3
        acc[::53] = 0.25  # ties at the top
        a0 = acc.clone()
        slots = p2p.IndexSyncSlots(pool, k, nb)
        comm = torch.zeros(nb, device=dev)
        scratch = p2p.IndexSyncScratch(dev, nb)
        for rep in range(3):
            acc.copy_(a0)
            comm.zero_()
            # poison the receive area: a pair that survives from an earlier launch or is read before
            # the peers' payload has landed shows up as NaN in the staging buffer
            slots.buf.view(torch.int32, 0, 2 * k * world).fill_(0x7FC00000)
            dist.barrier()
            p2p.bucket_index_sync_(ch, scratch, acc, k, slots=slots, comm=comm, scale=1.0 / world, sumsq_out=sq)
            torch.cuda.synchronize()
            ch.check("bucket index sync")
            mask = KT.topk_rank_local(a0.abs(), k)
            idx = KT.compact_mask_idx(mask)
            vals = a0[idx.long()]
            assert torch.equal(acc, torch.where(mask.bool(), torch.zeros_like(a0), a0))
            idxs, valss = gather(idx), gather(vals)
            refc = torch.zeros(nb, device=dev)
            for r in range(world):
                refc.index_add_(0, idxs[r].long(), valss[r] * (1.0 / world))
            assert not torch.isnan(comm).any(), "a poisoned receive slot reached the staging buffer"
            assert torch.equal(comm, refc), "reduced sparse gradient differs from the rank-ordered reference"
            assert abs(sq.item() - (refc.double() ** 2).sum().item()) <= 1e-4 * max(sq.item(), 1e-30)
    dist.barrier()
    pool.close()


def check_trainer(rank, world, dev):
    from sga_b200.runtime.trainer import Trainer, default_args

    common = dict(model="test_tiny", micro_batch_size=2, global_batch_size=4 * world, train_iters=6, lr=1e-3,
                  sga_bucket_elems=30000, log_interval=0)
    cases = {
        "dense_fused": dict(),
        "dense_allreduce": dict(dense_mode="allreduce"),
        "rank_local_index": dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="exact",
                                 sga_selection_ratio_percent=2.0, sga_backend="torch_pipelined_index",
                                 sga_selection_locality="rank_local", sga_cycle_period=3),
        "rank_local_mask": dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="exact",
                                sga_selection_ratio_percent=5.0, sga_backend="torch_pipelined_mask",
                                sga_selection_locality="rank_local", sga_cycle_period=4),
        "shared_index": dict(sga_enabled=True, sga_score="update", sga_selection_method="histogram",
                             sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                             sga_backend="torch_pipelined_index", sga_cycle_period=3, sga_cycle_start_iter=1),
        "shared_mask": dict(sga_enabled=True, sga_score="abs_m", sga_selection_method="histogram",
                            sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                            sga_backend="torch_pipelined_mask", sga_cycle_period=2),
        "shared_nccl_index": dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="histogram",
                                  sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                                  sga_backend="nccl_pipelined_index", sga_cycle_period=2),
    }
    final = {}
    for name, kw in cases.items():
        tr = Trainer(default_args(**common, **kw), quiet=True)
        losses = []
        for s in range(6):
            losses.append(float(tr.train_step(tr.host_batch(0)).item()))
        tr.check()
        w = tr.model.arena.model_param.clone()
        ws = gather(w)
        assert all(torch.equal(ws[0], t) for t in ws), f"{name}: ranks hold different parameters"
        assert losses[-1] < losses[0], f"{name}: loss did not decrease {losses}"
        assert all(l == l for l in losses)
        final[name] = losses
        tr.close()
        dist.barrier()
    # the two dense paths compute the same update (different execution strategy)
    a, b = final["dense_fused"], final["dense_allreduce"]
    assert all(abs(x - y) < 2e-2 for x, y in zip(a, b)), (a, b)
    return final


def _run_steps(args, steps, batches=None):
    from sga_b200.runtime.trainer import Trainer

    tr = Trainer(args, quiet=True)
    losses = [float(tr.train_step(tr.host_batch(s if batches is None else batches[s])).item()) for s in range(steps)]
    tr.check()
    return tr, losses


def check_trajectories(rank, world, dev):
    """The same configuration over the peer-memory kernels and over the library collectives must give
    the same loss trajectory up to the order of the fp32 / bf16 sums: SGA rank-local index mode and
    the dense step, 20 steps each."""
    from sga_b200.runtime.trainer import default_args

    common = dict(model="test_tiny", micro_batch_size=2, global_batch_size=4 * world, train_iters=20, lr=1e-3,
                  sga_bucket_elems=30000, log_interval=0)
    sga = dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="exact", sga_selection_ratio_percent=2.0,
               sga_backend="torch_pipelined_index", sga_selection_locality="rank_local", sga_cycle_period=0)
    out = {}
    for name, kw in (("sga_p2p", dict(sga, transport="p2p")), ("sga_nccl", dict(sga, transport="nccl")),
                     ("dense_p2p", dict(transport="p2p")), ("dense_nccl", dict(transport="nccl"))):
        tr, losses = _run_steps(default_args(**common, **kw), 20)
        out[name] = losses
        tr.close()
        dist.barrier()
    for a, b in (("sga_p2p", "sga_nccl"), ("dense_p2p", "dense_nccl")):
        worst = max(abs(x - y) / max(abs(y), 1e-6) for x, y in zip(out[a], out[b]))
        assert worst < 1e-3, f"{a} vs {b}: loss trajectories differ by {worst:.2e} relative: {out[a]} {out[b]}"
    return out


def check_sharded_step(rank, world, dev):
    """The sharded SGA step (each rank updates the bucket slices it owns, bf16 parameters pushed to the
    peers) against the replicated one: bit-identical bf16 parameters, and after the gather bit-identical
    fp32 weights and moments."""
    from sga_b200.runtime.trainer import default_args

    kw = dict(model="test_tiny", micro_batch_size=2, global_batch_size=4 * world, train_iters=8, lr=1e-3,
              sga_bucket_elems=30000, log_interval=0, sga_enabled=True, sga_score="abs_g",
              sga_selection_method="exact", sga_selection_ratio_percent=2.0, sga_backend="torch_pipelined_index",
              sga_selection_locality="rank_local", sga_cycle_period=3)
    got = {}
    for mode in ("1", "0"):
        os.environ["SGA_SHARDED_STEP"] = mode
        tr, losses = _run_steps(default_args(**kw), 8)
        assert tr.sharded_state == (mode == "1" and world > 1)
        tr.gather_optimizer_state()
        a = tr.model.arena
        got[mode] = (losses, a.model_param.clone(), a.main_param.clone(), a.exp_avg.clone(), a.exp_avg_sq.clone())
        tr.close()
        dist.barrier()
    os.environ.pop("SGA_SHARDED_STEP")
    assert got["1"][0] == got["0"][0], (got["1"][0], got["0"][0])
    for i, what in ((1, "bf16 parameters"), (2, "fp32 weights"), (3, "exp_avg"), (4, "exp_avg_sq")):
        assert torch.equal(got["1"][i], got["0"][i]), f"sharded vs replicated step: {what} differ"


def check_resume(rank, world, dev):
    """Checkpoint of a run whose optimizer state lives in owner slices (fused dense step, sharded SGA
    step): save at step 3, resume in a fresh trainer, continue; bit-identical with the uninterrupted run."""
    import tempfile

    from sga_b200.runtime import checkpoint as ckpt
    from sga_b200.runtime.trainer import Trainer, default_args

    root = [tempfile.mkdtemp(prefix="sga_resume_") if rank == 0 else None]
    dist.broadcast_object_list(root, src=0)
    base = dict(model="test_tiny", micro_batch_size=2, global_batch_size=4 * world, train_iters=6, lr=1e-3,
                sga_bucket_elems=30000, log_interval=0)
    for name, kw in (("dense_fused", dict()),):
        args = default_args(**base, **kw)
        full, _ = _run_steps(args, 6)
        full.gather_optimizer_state()
        ref = (full.model.arena.model_param.clone(), full.model.arena.main_param.clone(),
               full.model.arena.exp_avg.clone())
        full.close()
        dist.barrier()
        first, _ = _run_steps(args, 3)
        assert first.sharded_state == (world > 1)
        d = os.path.join(root[0], name)
        first.gather_optimizer_state()
        ckpt.save_checkpoint(d, 3, args, first.model, first.optimizer, first.rank, first.tp_rank, first.dp_rank,
                             first.pp_rank, first.pp_size, tracker=False)
        dist.barrier()
        if rank == 0:
            ckpt.write_tracker(d, 3)
        dist.barrier()
        first.close()
        second = Trainer(args, quiet=True)
        it = ckpt.load_checkpoint(d, second.model, second.optimizer)
        assert it == 3
        second.iteration = it
        for s in range(3, 6):
            second.train_step(second.host_batch(s))
        second.check()
        second.gather_optimizer_state()
        a = second.model.arena
        assert torch.equal(a.model_param, ref[0]), f"{name}: resumed bf16 parameters differ"
        assert torch.equal(a.main_param, ref[1]), f"{name}: resumed fp32 weights differ"
        assert torch.equal(a.exp_avg, ref[2]), f"{name}: resumed moments differ"
        second.close()
        dist.barrier()


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    check_kernels(rank, world, dev)
    final = check_trainer(rank, world, dev)
    check_sharded_step(rank, world, dev)
    check_resume(rank, world, dev)
    final.update(check_trajectories(rank, world, dev))
    dist.barrier()
    if rank == 0:
        for k, v in final.items():
            print(k, [round(x, 4) for x in v])
        print("DIST_GPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
