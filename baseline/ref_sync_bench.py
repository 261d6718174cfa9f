"""Same-box comparison of the part of a training step that the reference
implements itself: gradient synchronisation (full or sparse, by the cycle
calendar) plus the optimizer step, over a flat parameter vector with the
geometry of a model (default: Llama-3-1B's 1.24 B parameters in 16 Mi-element
buckets), on 1..N GPUs::

    torchrun --nnodes=1 --nproc-per-node=N --master-addr 127.0.0.1 baseline/ref_sync_bench.py --impl both

``--impl reference`` drives the unmodified reference engine (``sga.engine``
from ``baseline/_ref``: its backends, its selection plugin, its Triton
optimizer kernels, NCCL through ``torch.distributed``) with a stand-in for the
external training stack's data-parallel chunk and optimizer wrapper: the
attributes the engine reads (``sga/engine.py:318-396``) and nothing else. The
two predicates the engine imports from that stack are stubbed to "count every
parameter" (one model-parallel rank). ``--impl ours`` drives this framework's
engine, data-parallel layer and optimizer on the same geometry, the same
shared-support configuration and the same per-step gradients. Both arms are
timed with CUDA events around ``grad_sync`` + ``optimizer_step`` (the gradient
fill is outside), max over ranks; each arm prints one JSON line with every
step's time, the medians of the full and the sparse steps and the per-step
cost of one cycle built from those medians.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import types

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SGA = dict(sga_score="abs_g", sga_selection="topk", sga_selection_method="histogram",
           sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=1.0, sga_optimizer="adamw",
           sga_backend="torch_pipelined_index", sga_cycle_start_iter=0, sga_cycle_period=4)
HP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0)


def geometry(total: int, bucket: int, param: int):
    """Parameters of ``param`` elements packed into buckets of ``bucket`` elements (the last ones smaller)."""
    buckets, left = [], total
    while left > 0:
        b = min(bucket, left)
        sizes, bl = [], b
        while bl > 0:
            sizes.append(min(param, bl))
            bl -= sizes[-1]
        buckets.append(sizes)
        left -= b
    return buckets


def fill_grads(views, step: int, rank: int) -> None:
    g = torch.Generator(device=views[0].device).manual_seed(1000 * step + rank)
    for v in views:
        v.add_(torch.randn(v.numel(), generator=g, device=v.device, dtype=torch.float32) * 1e-3)


def timed_steps(step_fn, fill_fn, steps: int, warmup: int, world: int):
    dev = torch.cuda.current_device()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s in range(1, warmup + steps + 1):
        fill_fn(s)
        if s > warmup:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)
            ev[s - warmup - 1][0].record()
        step_fn(s)
        if s > warmup:
            ev[s - warmup - 1][1].record()
    torch.cuda.synchronize(dev)
    ms = torch.tensor([a.elapsed_time(b) for a, b in ev], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.tolist()


# ------------------------------------------------------------------ reference arm
def run_reference(ns, rank, world, dev):
    if not os.path.isdir(os.path.join(REF, "sga")):
        return {"impl": "reference", "unavailable": "baseline/_ref/sga is not present on this machine"}
    for n in ("megatron", "megatron.core", "megatron.core.tensor_parallel", "megatron.core.transformer",
              "megatron.core.transformer.module"):
        sys.modules.setdefault(n, types.ModuleType(n))
    sys.modules["megatron.core.tensor_parallel"].param_is_not_tensor_parallel_duplicate = lambda p, g=None: True
    sys.modules["megatron.core.transformer.module"].param_is_not_shared = lambda p: True
    sys.path.insert(0, REF)
    from sga.config import set_args
    from sga.config.validation import sga_defaults, validate_sga_args
    from sga.engine import SGAEngine
    from sga.plugins import build_backend_plugin, build_optimizer, build_selection, register_default_plugins

    args = types.SimpleNamespace(**{**sga_defaults(), **SGA, "sga_enabled": True})
    args.train_iters, args.pipeline_model_parallel_size = 10 ** 6, 1
    validate_sga_args(args)
    set_args(args)
    register_default_plugins()
    group = dist.group.WORLD

    class Bucket:
        def __init__(self, sizes, bid):
            n = sum(sizes)
            self.grad_data = torch.zeros(n, dtype=torch.float32, device=dev)
            self.params_list, self.param_to_index, off = [], {}, 0
            for sz in sizes:
                p = torch.nn.Parameter(torch.randn(sz, device=dev, dtype=torch.float32).mul_(0.02).to(torch.bfloat16),
                                       requires_grad=False)
                p.main_grad = self.grad_data[off:off + sz]
                self.params_list.append(p)
                self.param_to_index[p] = (off, off + sz)
                off += sz
            self.gradient_scaling_factor = 1.0 / world
            self.bucket_id = bid

    class Group:
        def __init__(self, bucket):
            self.buckets, self.data_parallel_group = [bucket], group

        def reset(self):
            pass

    class Chunk:
        def __init__(self):
            self.bucket_list = [Bucket(sizes, i) for i, sizes in enumerate(geometry(ns.elems, ns.bucket, ns.param))]
            self.bucket_groups = [Group(b) for b in self.bucket_list]
            self.expert_parallel_bucket_groups, self.expert_parallel_buffers = [], []
            self.buffers = [types.SimpleNamespace(buckets=self.bucket_list, extra_main_grads=[])]
            self.params = [p for b in self.bucket_list for p in b.params_list]
            names = [f"decoder.layers.{i}.weight" for i in range(len(self.params))]
            self.module = types.SimpleNamespace(named_parameters=lambda: list(zip(names, self.params)))
            self.ddp_config = types.SimpleNamespace(average_in_collective=False)
            self.params_with_grad = list(self.params)

        def finish_grad_sync(self, force_all_reduce=False):
            # the dense path of the external stack: average every bucket over the data-parallel group
            for b in self.bucket_list:
                if world > 1:
                    dist.all_reduce(b.grad_data, group=group)
                    b.grad_data.mul_(1.0 / world)

    class MixedPrecisionOptimizer:
        def __init__(self, chunk):
            self.config = types.SimpleNamespace(clip_grad=HP["clip"])
            self.float16_groups = [list(chunk.params)]
            self.main_params = [p.detach().float().clone() for p in chunk.params]
            for mp, p in zip(self.main_params, chunk.params):
                p.main_param = mp
            self.fp32_from_float16_groups = [self.main_params]
            self.optimizer = torch.optim.Adam(self.main_params, lr=HP["lr"], betas=(HP["beta1"], HP["beta2"]),
                                              eps=HP["eps"], weight_decay=HP["wd"], foreach=True)

        def prepare_grads(self):
            for mp, p in zip(self.main_params, self.float16_groups[0]):
                mp.grad = p.main_grad
            return False

        def _copy_main_params_to_model_params(self):
            torch._foreach_copy_(self.float16_groups[0], self.main_params)

    torch.manual_seed(1234)  # data-parallel replicas start from the same weights
    chunk = Chunk()
    opt = MixedPrecisionOptimizer(chunk)
    p0 = [m.cpu() for m in opt.main_params] if ns.check else None
    eng = SGAEngine(SGA["sga_score"], build_selection(SGA["sga_selection"]), build_optimizer(SGA["sga_optimizer"]),
                    build_backend_plugin(SGA["sga_backend"]))
    eng._dp_cp_group = lambda: group
    eng._tp_group = lambda: None
    eng.attach(chunk)
    views = [b.grad_data for b in chunk.bucket_list]
    phases = []

    probe = []

    def lane_state(lane):
        b, off = divmod(lane, ns.bucket)
        j, o = divmod(off, ns.param)
        mp = opt.main_params[sum(len(x.params_list) for x in chunk.bucket_list[:b]) + j]
        st = opt.optimizer.state.get(mp, {})
        mask = eng._bucket_states[b].active_mask_u8
        return [float(mp[o]), float(st["exp_avg"][o]) if "exp_avg" in st else 0.0,
                float(st["exp_avg_sq"][o]) if "exp_avg_sq" in st else 0.0,
                float(chunk.bucket_list[b].grad_data[off]), int(mask.view(-1)[off]) if mask is not None else -1]

    def step(s):
        pre = [float(chunk.bucket_list[l // ns.bucket].grad_data[l % ns.bucket]) for l in ns.lanes]
        handled = eng.grad_sync(chunk, force_all_reduce=False)
        if not handled:
            chunk.finish_grad_sync()
        phases.append("full" if eng._step_full else "sparse")
        ok, _gn, _nz = eng.optimizer_step(opt, [chunk], s)
        assert ok
        if ns.lanes:
            probe.append({"step": s, "phase": phases[-1], "grad_norm": float(_gn), "local_grad": pre,
                          "w_m_v_buf_active": [lane_state(l) for l in ns.lanes]})

    ms = timed_steps(step, lambda s: fill_grads(views, s, rank), ns.steps, ns.warmup, world)
    out = {"impl": "reference", "ms": ms, "phases": phases[ns.warmup:],
           "kernels": "reference engine + backends + its Triton optimizer kernels; NCCL via torch.distributed"}
    if ns.lanes:
        out["probe"] = probe
    if ns.check:
        out["_state"] = (p0, torch.cat([m.reshape(-1) for m in opt.main_params]).cpu(),
                         torch.cat([b.grad_data for b in chunk.bucket_list]).cpu())
    return out


# ------------------------------------------------------------------------ our arm
def run_ours(ns, rank, world, dev, p0=None):
    from sga_b200 import config as C
    from sga_b200.runtime.arena import FlatArena, ParamSpec
    from sga_b200.runtime.builder import build_engine
    from sga_b200.runtime.ddp import DataParallel, DDPConfig
    from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig

    pool = None
    if ns.transport == "p2p":
        from sga_b200.parallel.symm import SymmPool

        pool = SymmPool(device=dev)
    C.set_args(C.make_args(sga_enabled=True, sga_checks=True, **SGA))
    specs = [ParamSpec(f"decoder.layers.{i}.weight", (sz,), 0, "normal", 0.02)
             for i, sz in enumerate(s for sizes in geometry(ns.elems, ns.bucket, ns.param) for s in sizes)]
    model = types.SimpleNamespace()
    model.arena = FlatArena(specs, bucket_elems=ns.bucket, device=dev, pool=pool)
    model.arena.init_parameters(0, on_device=True)
    if p0 is not None:  # start from the reference arm's weights
        for slot, p in zip(model.arena.slots, p0):
            slot.main.copy_(p.to(dev))
        model.arena.sync_model_from_main()
    model.named_parameters = lambda: [(s.name, s.model) for s in model.arena.slots]
    ddp = DataParallel(model, transport=ns.transport if world > 1 or pool is not None else "local",
                       ddp_config=DDPConfig(average_in_collective=True, overlap_grad_reduce=False), pool=pool)
    opt = FlatOptimizer(model.arena, OptimizerConfig(lr=HP["lr"], weight_decay=HP["wd"], adam_beta1=HP["beta1"],
                                                     adam_beta2=HP["beta2"], adam_eps=HP["eps"], clip_grad=HP["clip"]))
    eng = build_engine(quiet=True)
    eng.log_interval = 0
    eng.attach(ddp)
    views = [model.arena.main_grad[b.start:b.end] for b in model.arena.buckets]
    phases = []

    probe = []
    per_bucket = [len(sizes) for sizes in geometry(ns.elems, ns.bucket, ns.param)]

    def flat(lane):
        b, off = divmod(lane, ns.bucket)
        j, o = divmod(off, ns.param)
        return model.arena.slots[sum(per_bucket[:b]) + j].start + o

    def step(s):
        a = model.arena
        pre = [float(a.main_grad[flat(l)]) for l in ns.lanes]
        ddp.begin_step()
        eng.begin_step(ddp, s)
        if not eng.grad_sync(ddp, False):
            ddp.finish_grad_sync()
        phases.append("full" if eng._step_full else "sparse")
        ok, _gn, _nz = eng.optimizer_step(opt, [ddp], s)
        assert ok
        if ns.lanes:
            mask = eng._active_mask_arena() if eng._active_support is not None else None
            probe.append({"step": s, "phase": phases[-1], "grad_norm": float(_gn), "local_grad": pre,
                          "w_m_v_buf_active": [[float(a.main_param[flat(l)]), float(a.exp_avg[flat(l)]),
                                                float(a.exp_avg_sq[flat(l)]), float(a.main_grad[flat(l)]),
                                                int(mask[flat(l)]) if mask is not None else -1] for l in ns.lanes]})

    ms = timed_steps(step, lambda s: fill_grads(views, s, rank), ns.steps, ns.warmup, world)
    ddp.check()
    out = {"impl": "ours", "ms": ms, "phases": phases[ns.warmup:], "transport": ddp.transport}
    if ns.lanes:
        out["probe"] = probe
    if ns.check:
        out["_state"] = (None, torch.cat([sl.main.reshape(-1) for sl in model.arena.slots]).cpu(),
                         torch.cat([model.arena.main_grad[sl.start:sl.end] for sl in model.arena.slots]).cpu())
    if pool is not None:
        pool.close()
    return out


def _median(xs):
    xs = sorted(xs)
    if not xs:
        return float("nan")
    mid = len(xs) // 2
    return xs[mid] if len(xs) % 2 else 0.5 * (xs[mid - 1] + xs[mid])


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="both", choices=("ours", "reference", "both"))
    ap.add_argument("--elems", type=int, default=1235814400)
    ap.add_argument("--bucket", type=int, default=16 * 1024 * 1024)
    ap.add_argument("--param", type=int, default=4 * 1024 * 1024)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--transport", default="p2p", choices=("p2p", "nccl"))
    ap.add_argument("--check", action="store_true",
                    help="with --impl both: start our arm from the reference arm's weights and report how far the "
                         "two arms' weights and residual buffers are apart after the run")
    ap.add_argument("--lanes", type=lambda t: [int(x) for x in t.split(",") if x], default=[],
                    help="comma list of flat element numbers: each arm also reports, after every step, the weight, "
                         "both moments, the gradient-buffer value and the support bit there (a diagnostic; the "
                         "per-step device reads make the timings meaningless)")
    ap.add_argument("--clip", type=float, default=HP["clip"], help="gradient-norm clip of both arms (0 = off)")
    ns = ap.parse_args()
    HP["clip"] = ns.clip
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # a process group even for one rank: the reference backends call all_reduce unconditionally
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank()
    states = {}
    for impl in (("reference", "ours") if ns.impl == "both" else (ns.impl,)):
        if impl == "reference":
            res = run_reference(ns, rank, world, dev)
        else:
            res = run_ours(ns, rank, world, dev, p0=states["reference"][0] if "reference" in states else None)
        if "_state" in res:
            states[impl] = res.pop("_state")
        if "ms" in res:
            ms, ph = res["ms"], res["phases"]
            res.update(n_gpus=world, elems=ns.elems, bucket_elems=ns.bucket, steps=ns.steps, warmup=ns.warmup,
                       ms_full_median=round(_median([m for m, p in zip(ms, ph) if p == "full"]), 3),
                       ms_sparse_median=round(_median([m for m, p in zip(ms, ph) if p == "sparse"]), 3),
                       config="score |g|, shared support top-1 % (balanced histogram), index backend, cycle 4, "
                              "residual-aware AdamW, clip 1.0",
                       timing="CUDA events around grad_sync + optimizer_step, max over ranks")
            period = SGA["sga_cycle_period"]
            res["ms_per_step_cycle"] = round((res["ms_full_median"] + (period - 1) * res["ms_sparse_median"]) / period, 3)
            res["ms"] = [round(m, 3) for m in ms]
        if rank == 0:
            print(json.dumps(res), flush=True)
        torch.cuda.empty_cache()
    if ns.check and len(states) == 2:
        (_, rw, rr), (_, ow, orr) = states["reference"], states["ours"]
        moved = float((rw - torch.cat([p.reshape(-1) for p in states["reference"][0]])).abs().max())
        cmp = {"check": "reference vs ours after the run", "max_abs_dw": float((rw - ow).abs().max()),
               "max_weight_movement": moved, "residual_lanes_differing": int((rr != orr).sum()),
               "residual_lanes": int(rr.numel()), "max_abs_dresidual": float((rr - orr).abs().max()),
               "weight_lanes_off_by_1e-6": int(((rw - ow).abs() > 1e-6).sum())}
        off = ((rw - ow).abs() > 1e-6).nonzero().view(-1)[:8]
        w0 = torch.cat([p.reshape(-1) for p in states["reference"][0]])
        cmp["lanes_off"] = [{"lane": int(i), "w0": float(w0[i]), "reference": float(rw[i]), "ours": float(ow[i])} for i in off]
        t = torch.tensor([cmp["max_abs_dw"], float(cmp["residual_lanes_differing"]), cmp["max_abs_dresidual"]],
                         dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        cmp["max_abs_dw"], cmp["residual_lanes_differing"], cmp["max_abs_dresidual"] = t[0].item(), int(t[1]), t[2].item()
        if rank == 0:
            print(json.dumps(cmp), flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
