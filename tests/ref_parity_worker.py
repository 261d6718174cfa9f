"""Worker of the multi-rank parity test: two or more ``gloo`` ranks on CPU drive the unmodified
reference engine (``sga/engine.py``, from the local copy of the reference package) and this
framework's engine over the same initial weights and the same per-rank gradients (each rank's
gradients differ in seed and scale), and compare calendars, gradient norms, weights and the
residual left in the gradient buffer. The stand-ins for the external training stack expose the
attributes the reference engine reads (``sga/engine.py:318-396``) and nothing else.

Launched by ``tests/test_reference_parity.py`` through ``torch.distributed.run``."""
import os
import sys
import types

sys.modules["triton"] = None  # the reference takes its torch paths
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
sys.path.insert(0, REF)
sys.path.insert(0, ROOT)
os.environ["SGA_ALLOW_FROZEN_SELECTION"] = "1"
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

# the two predicates the reference engine imports from its external training stack
for _name in ("megatron", "megatron.core", "megatron.core.tensor_parallel", "megatron.core.transformer",
              "megatron.core.transformer.module"):
    sys.modules.setdefault(_name, types.ModuleType(_name))
sys.modules["megatron.core.tensor_parallel"].param_is_not_tensor_parallel_duplicate = lambda p, g=None: True
sys.modules["megatron.core.transformer.module"].param_is_not_shared = lambda p: True

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
HP = dict(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01, clip=1.0)
BUCKETS = [[1000, 24], [512, 512, 300], [700]]  # parameter sizes per bucket
TOTAL = sum(sum(b) for b in BUCKETS)
STEPS = 14


def grads_for(step, r):
    g = torch.Generator().manual_seed(1000 * step + r)
    return torch.randn(TOTAL, generator=g) * (1.0 + 0.5 * r)


class _Bucket:
    def __init__(self, sizes, bid):
        self.grad_data = torch.zeros(sum(sizes))
        self.params_list, self.param_to_index = [], {}
        off = 0
        for sz in sizes:
            p = torch.nn.Parameter((torch.randn(sz) * 0.5).to(torch.bfloat16), requires_grad=False)
            p.main_grad = self.grad_data[off:off + sz]
            self.params_list.append(p)
            self.param_to_index[p] = (off, off + sz)
            off += sz
        self.gradient_scaling_factor = 1.0 / world
        self.bucket_id = bid


class _Group:
    def __init__(self, bucket, group):
        self.buckets, self.data_parallel_group = [bucket], group

    def reset(self):
        pass


class _Chunk:
    """The data-parallel model chunk as the reference engine sees it."""

    def __init__(self, group):
        self.group = group
        self.bucket_list = [_Bucket(s, i) for i, s in enumerate(BUCKETS)]
        self.bucket_groups = [_Group(b, group) for b in self.bucket_list]
        self.expert_parallel_bucket_groups, self.expert_parallel_buffers = [], []
        self.buffers = [types.SimpleNamespace(buckets=self.bucket_list, extra_main_grads=[])]
        self.params = [p for b in self.bucket_list for p in b.params_list]
        names = [f"decoder.layers.{i}.weight" for i in range(len(self.params))]
        self.module = types.SimpleNamespace(named_parameters=lambda: list(zip(names, self.params)))
        self.ddp_config = types.SimpleNamespace(average_in_collective=False)
        self.params_with_grad = list(self.params)

    def finish_grad_sync(self, force_all_reduce=False):
        for b in self.bucket_list:  # the stock dense path: scale, then sum over the group
            b.grad_data.mul_(1.0 / world)
            dist.all_reduce(b.grad_data, group=self.group)


class _MixedPrecisionOptimizer:
    """The optimizer wrapper as the reference engine sees it (hyper-parameters and lazy Adam state)."""

    def __init__(self, chunk):
        self.config = types.SimpleNamespace(clip_grad=HP["clip"])
        self.float16_groups = [list(chunk.params)]
        self.main_params = [p.detach().float().clone() for p in chunk.params]
        for mp, p in zip(self.main_params, chunk.params):
            p.main_param = mp
        self.fp32_from_float16_groups = [self.main_params]
        self.optimizer = torch.optim.Adam(self.main_params, lr=HP["lr"], betas=(HP["beta1"], HP["beta2"]),
                                          eps=HP["eps"], weight_decay=HP["wd"])

    def prepare_grads(self):
        for mp, p in zip(self.main_params, self.float16_groups[0]):
            mp.grad = p.main_grad
        return False

    def _copy_main_params_to_model_params(self):
        for p, mp in zip(self.float16_groups[0], self.main_params):
            p.data.copy_(mp)


def run_reference(SGA):
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
    torch.manual_seed(5)  # replicas start from the same weights
    chunk = _Chunk(group)
    opt = _MixedPrecisionOptimizer(chunk)
    p0 = [m.clone() for m in opt.main_params]
    eng = SGAEngine(SGA["sga_score"], build_selection(SGA["sga_selection"]), build_optimizer(SGA["sga_optimizer"]),
                    build_backend_plugin(SGA["sga_backend"]))
    eng._dp_cp_group = lambda: group
    eng._tp_group = lambda: None
    eng.attach(chunk)
    log = []
    for s in range(1, STEPS + 1):
        g, off = grads_for(s, rank), 0
        for b in chunk.bucket_list:
            n = b.grad_data.numel()
            b.grad_data += g[off:off + n]
            off += n
        if not eng.grad_sync(chunk, force_all_reduce=False):
            chunk.finish_grad_sync()
        full = bool(eng._step_full)
        _ok, gn, _nz = eng.optimizer_step(opt, [chunk], s)
        log.append((s, full, float(gn)))
    return p0, log, torch.cat(opt.main_params), torch.cat([b.grad_data for b in chunk.bucket_list])


def run_ours(SGA, p0):
    from sga_b200 import config as C
    from sga_b200.runtime.arena import FlatArena, ParamSpec
    from sga_b200.runtime.builder import build_engine
    from sga_b200.runtime.ddp import DataParallel, DDPConfig
    from sga_b200.runtime.optimizer import FlatOptimizer, OptimizerConfig

    C.set_args(C.make_args(sga_enabled=True, **SGA))
    sizes = [s for b in BUCKETS for s in b]
    specs = [ParamSpec(f"decoder.layers.{i}.weight", (sz,), 0, "zeros") for i, sz in enumerate(sizes)]
    model = types.SimpleNamespace()
    model.arena = FlatArena(specs, bucket_elems=1024, device="cpu")
    model.named_parameters = lambda: [(s.name, s.model) for s in model.arena.slots]
    slots = model.arena.slots
    for s, p in zip(slots, p0):
        s.main.copy_(p)
    model.arena.sync_model_from_main()
    ddp = DataParallel(model, transport="gloo",
                       ddp_config=DDPConfig(average_in_collective=False, overlap_grad_reduce=False))
    opt = FlatOptimizer(model.arena, OptimizerConfig(lr=HP["lr"], weight_decay=HP["wd"], adam_beta1=HP["beta1"],
                                                     adam_beta2=HP["beta2"], adam_eps=HP["eps"], clip_grad=HP["clip"]))
    eng = build_engine(quiet=True)
    eng.log_interval = 0
    eng.attach(ddp)
    log = []
    for s in range(1, STEPS + 1):
        g, off = grads_for(s, rank), 0
        for sl in slots:
            n = sl.end - sl.start
            model.arena.main_grad[sl.start:sl.end] += g[off:off + n]
            off += n
        ddp.begin_step()
        eng.begin_step(ddp, s)
        if not eng.grad_sync(ddp, False):
            ddp.finish_grad_sync()
        full = bool(eng._step_full)
        _ok, gn, _nz = eng.optimizer_step(opt, [ddp], s)
        log.append((s, full, float(gn)))
    return (log, torch.cat([sl.main.reshape(-1) for sl in slots]),
            torch.cat([model.arena.main_grad[sl.start:sl.end] for sl in slots]))


BASE = dict(sga_score="abs_g", sga_selection="topk", sga_selection_method="histogram",
            sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0, sga_optimizer="adamw",
            sga_backend="torch_pipelined_index", sga_cycle_start_iter=2, sga_cycle_period=3)
VARIANTS = {
    "index": {},
    "mask": {"sga_backend": "torch_pipelined_mask", "sga_score": "update", "sga_cycle_start_iter": 0},
    "index fold adams": {"sga_optimizer": "adams", "sga_optimizer_residual_mean": True},
    "index writeback": {"sga_backend_emission": "writeback"},
    "index dual": {"sga_optimizer_full_sync_inactive_lr_scale": 0.5, "sga_score": "abs_m"},
    "exact kth": {"sga_selection_method": "exact", "sga_score": "coi"},
    "adaptive": {"sga_selection_method": "adaptive"},
    "hist allreduce": {"sga_selection_topk_histogram_add_global_allreduce": True,
                       "sga_selection_histogram_mode": "exact"},
    "fast": {"sga_selection_histogram_mode": "fast", "sga_backend_index_slices": 3},
    "block8": {"sga_selection_block_size": 8, "sga_selection_histogram_mode": "exact",
               "sga_backend_emission": "writeback"},
    "always": {"sga_always_sync_layers": ["layers.1."], "sga_backend": "torch_pipelined_mask"},
    "decoupled": {"sga_cycle_period": 6, "sga_cycle_full_sync_interval": 3,
                  "sga_cycle_decouple_full_sync_interval_and_period": True},
}


def main() -> int:
    bad = []
    for name, override in VARIANTS.items():
        SGA = {**BASE, **override}
        p0, rlog, rw, rr = run_reference(SGA)
        olog, ow, orr = run_ours(SGA, p0)
        if [(s, f) for s, f, _ in rlog] != [(s, f) for s, f, _ in olog]:
            bad.append((name, "calendar"))
        if max(abs(a[2] - b[2]) / max(a[2], 1e-9) for a, b in zip(rlog, olog)) > 5e-7:
            bad.append((name, "norm"))
        if float((rw - ow).abs().max()) > 3e-7:
            bad.append((name, "weights"))
        if not torch.equal(rr, orr):
            bad.append((name, "residual"))
    flag = torch.tensor([len(bad)])
    dist.all_reduce(flag)
    if rank == 0:
        print("PARITY OK" if int(flag) == 0 else f"PARITY FAILED {bad}", flush=True)
    dist.destroy_process_group()
    return 0 if int(flag) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
