"""Two-rank gloo runs on CPU: the plumbing of the sparse step without a GPU.

Case 1 is the plumbing benchmark configuration: a flat fp32 gradient of
4,194,304 elements in 4 buckets of 1,048,576, N(0, 1e-3^2) gradients fresh
every step, rank-local exact top-1 % per bucket of |grad + residual|, (int32
index, fp32 value) exchange summed and divided by the world size, residual
write-back, residual-aware AdamW; 10 steps, compared with a dense
all-reduce + AdamW run of the same data.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sga_b200 import config as C
from sga_b200.runtime.arena import FlatArena, ParamSpec
from sga_b200.runtime.builder import build_engine
from sga_b200.runtime.ddp import DataParallel, DDPConfig
from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _FlatModel:
    def __init__(self, n_buckets, bucket_elems, seed):
        specs = [ParamSpec(f"p{i}.weight", (bucket_elems,), 0, "normal", 0.02) for i in range(n_buckets)]
        self.arena = FlatArena(specs, bucket_elems=bucket_elems, device="cpu")
        self.arena.init_parameters(seed)

    def named_parameters(self):
        for s in self.arena.slots:
            yield s.name, s.model


def _sga_args(**kw):
    base = dict(sga_enabled=True, sga_score="abs_g", sga_selection_method="exact", sga_selection_ratio_percent=1.0,
                sga_backend="torch_pipelined_index", sga_selection_locality="rank_local", sga_cycle_period=0)
    base.update(kw)
    return C.make_args(**base)


def _cfg1_worker(rank, world, port, n_buckets, bucket_elems, steps, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        n = n_buckets * bucket_elems
        opt_cfg = OptimizerConfig(lr=1e-4, weight_decay=0.1, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8,
                                  clip_grad=0.0)
        # sparse run
        C.set_args(_sga_args())
        model = _FlatModel(n_buckets, bucket_elems, seed=0)
        ddp = DataParallel(model, transport="gloo", ddp_config=DDPConfig(average_in_collective=False,
                                                                         overlap_grad_reduce=False))
        opt = FlatOptimizer(model.arena, opt_cfg)
        eng = build_engine(quiet=True)
        eng.log_interval = 0
        eng.attach(ddp)
        # dense reference on the same data
        ref = _FlatModel(n_buckets, bucket_elems, seed=0)
        ref_ddp = DataParallel(ref, transport="gloo", ddp_config=DDPConfig(average_in_collective=False,
                                                                           overlap_grad_reduce=False))
        ref_opt = FlatOptimizer(ref.arena, opt_cfg)
        from sga_b200.plugins.optimizer.reference import grad_correct_torch

        total_sent = torch.zeros(n, dtype=torch.float64)
        total_grad = torch.zeros(n, dtype=torch.float64)
        for step in range(1, steps + 1):
            g = torch.Generator().manual_seed(1000 * step + rank)
            grad = torch.randn(n, generator=g) * 1e-3
            model.arena.main_grad[:n] += grad
            ref.arena.main_grad[:n].copy_(grad)
            total_grad += grad.double()
            eng.begin_step(ddp, step)
            assert eng.grad_sync(ddp, False)
            total_sent += model.arena.comm[:n].double() * world  # what this step applied, summed over ranks
            ok, gn, _ = eng.optimizer_step(opt, [ddp], step)
            assert ok
            ref_ddp.finish_grad_sync()
            b1, b2 = 0.9, 0.95
            grad_correct_torch(ref.arena.main_param, ref.arena.main_grad, ref.arena.exp_avg, ref.arena.exp_avg_sq,
                               1e-4, b1, b2, 1e-8, 0.1, 1 - b1 ** step, 1 - b2 ** step, None, None)
            ref.arena.main_grad.zero_()
        # invariants
        w = model.arena.main_param.clone()
        gathered = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(gathered, w)
        replicas_equal = all(torch.equal(gathered[0], x) for x in gathered)
        # conservation: sum over ranks of (residual + everything sent) == sum over ranks of all gradients
        resid = model.arena.main_grad[:n].double()
        lhs = resid.clone()
        dist.all_reduce(lhs)
        tg = total_grad.clone()
        dist.all_reduce(tg)
        conservation = float(((lhs + total_sent) - tg).abs().max())
        drift = float((model.arena.main_param - ref.arena.main_param).abs().max())
        ref_move = float((ref.arena.main_param - _FlatModel(n_buckets, bucket_elems, 0).arena.main_param).abs().max())
        nnz = int((model.arena.comm != 0).sum())
        if rank == 0:
            out.put(dict(replicas_equal=replicas_equal, conservation=conservation, drift=drift, ref_move=ref_move,
                         comm_cleared=nnz == 0, step_count=opt.step_count))
    finally:
        dist.destroy_process_group()


def _spawn(fn, world, *args):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=fn, args=(r, world, port) + args + (q,)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0, f"worker exited with {p.exitcode}"
    return q.get()


@pytest.mark.timeout(900)
def test_cfg1_rank_local_index_sparse_allreduce_world2():
    res = _spawn(_cfg1_worker, 2, 4, 1 << 20, 10)
    assert res["replicas_equal"], "ranks must hold bit-identical parameters"
    assert res["conservation"] < 1e-6, res
    assert res["comm_cleared"]
    assert res["step_count"] == 10
    # the sparse trajectory stays within the distance the dense run itself moved
    assert res["drift"] <= 2.5 * res["ref_move"], res


def _rank_local_score_worker(rank, world, port, score, out):
    """Rank-local selection by a score that reads the optimizer state: every step's support must be
    the exact top-k of the registry formula over (gradient + residual), and the replicas stay equal."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sga_b200 import kernels_torch as KT
        from sga_b200.plugins.scores import compute_score

        n_buckets, be = 2, 30000
        C.set_args(_sga_args(sga_score=score, sga_selection_ratio_percent=2.0))
        model = _FlatModel(n_buckets, be, seed=0)
        ddp = DataParallel(model, transport="gloo", ddp_config=DDPConfig(average_in_collective=False,
                                                                         overlap_grad_reduce=False))
        opt = FlatOptimizer(model.arena, OptimizerConfig(lr=1e-3, clip_grad=1.0))
        eng = build_engine(quiet=True)
        eng.log_interval = 0
        eng.attach(ddp)
        eng.bind_optimizer(opt)
        n = n_buckets * be
        a = model.arena
        exact = True
        for step in range(1, 6):
            g = torch.Generator().manual_seed(31 * step + rank)
            a.main_grad[:n] += torch.randn(n, generator=g) * 1e-2
            before = a.main_grad.clone()
            st = opt.peek_step()
            sc = compute_score(score, a.main_param, a.exp_avg, a.exp_avg_sq, before, beta1=0.9, beta2=0.95,
                               eps=1e-8, weight_decay=0.1, bc1=1 - 0.9 ** st, bc2=1 - 0.95 ** st).abs()
            eng.begin_step(ddp, step)
            eng.grad_sync(ddp, False)
            if not eng._step_full:
                for b in a.buckets:
                    k = eng._k_for_bucket(b.numel)
                    ref = KT.topk_rank_local(sc[b.start:b.end], k).bool()
                    sent = (before[b.start:b.end] != 0) & (a.main_grad[b.start:b.end] == 0)
                    exact &= bool(torch.equal(sent, ref))
            eng.optimizer_step(opt, [ddp], step)
        w = a.main_param.clone()
        gathered = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(gathered, w)
        if rank == 0:
            out.put(dict(exact=exact, replicas_equal=all(torch.equal(gathered[0], x) for x in gathered)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("score", ["abs_m", "update", "coi"])
def test_rank_local_scores_world2(score):
    res = _spawn(_rank_local_score_worker, 2, score)
    assert res["exact"], "the support is not the exact top-k of the score"
    assert res["replicas_equal"]


def _shared_worker(rank, world, port, backend_name, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        os.environ["SGA_ALLOW_FROZEN_SELECTION"] = "1"
        n_buckets, be = 3, 40000
        C.set_args(C.make_args(sga_enabled=True, sga_score="abs_g", sga_selection_method="histogram",
                               sga_selection_histogram_mode="exact", sga_selection_ratio_percent=5.0,
                               sga_backend=backend_name, sga_cycle_period=4, sga_cycle_start_iter=1))
        model = _FlatModel(n_buckets, be, seed=0)
        ddp = DataParallel(model, transport="gloo", ddp_config=DDPConfig(average_in_collective=False,
                                                                         overlap_grad_reduce=False))
        opt = FlatOptimizer(model.arena, OptimizerConfig(lr=1e-3, clip_grad=1.0))
        eng = build_engine(quiet=True)
        eng.log_interval = 0
        eng.attach(ddp)
        n = n_buckets * be
        phases = []
        for step in range(1, 11):
            g = torch.Generator().manual_seed(77 * step + rank)
            model.arena.main_grad[:n] += torch.randn(n, generator=g) * 1e-2
            eng.begin_step(ddp, step)
            eng.grad_sync(ddp, False)
            phases.append("full" if eng._step_full else "sparse")
            if not eng._step_full:
                # a power-of-two factor makes the reduction exact: residual coordinates are untouched
                mask = eng._active_mask_arena()
                assert int(mask.sum()) == eng._active_support.total_selected
            eng.optimizer_step(opt, [ddp], step)
        w = model.arena.main_param.clone()
        gathered = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(gathered, w)
        if rank == 0:
            out.put(dict(phases=phases, replicas_equal=all(torch.equal(gathered[0], x) for x in gathered),
                         ratio=eng.last_ratio))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("backend_name", ["torch_pipelined_index", "torch_pipelined_mask"])
def test_shared_support_cycle_world2(backend_name):
    res = _spawn(_shared_worker, 2, backend_name)
    # start_iter 1, period 4: steps 1 (warm-up), 5, 9 are boundaries; no support before step 5
    assert res["phases"] == ["full"] * 5 + ["sparse"] * 3 + ["full", "sparse"], res["phases"]
    assert res["replicas_equal"]
    assert 0.04 < res["ratio"] < 0.07
