"""Headline benchmark: Llama-3-1B SGA training throughput (tokens/s).

Config (the benchmark's named one): 16 layers, hidden 2048, SwiGLU 8192,
32 query / 8 KV heads of 64, RoPE theta 5e5, vocab 128256 tied, sequence 2048,
micro-batch 4, global batch 256 sequences (fixed as GPUs are added: strong
scaling), bf16 compute with fp32 master weights and gradients, synthetic
uniform tokens (seed 1234), random-init weights N(0, 0.02^2). SGA: score
|grad + residual|, exact per-bucket top-1 %, index backend, residual-aware
AdamW lr 3e-4, rank-local exchange over peer memory.

    python bench.py --gpus N --steps K --warmup W          # our framework
    python bench.py --impl reference ...                     # the reference arm

For N > 1 launch under torchrun (one rank per GPU). Rank 0 prints one JSON line.
Timing: W untimed warm-up steps, then K steps between barrier + synchronize,
CUDA events on the compute stream, max over ranks. ``value`` is the device-side
number with batches already on the GPU; ``e2e`` repeats K steps through the
public ``Trainer.train_step`` with the batch copied from pinned host memory and
the loss read back every step. Working set (2.5 GB of bf16 weights, 5 GB of
fp32 gradients) is far larger than the 126 MB L2, so no explicit flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _reference_arm(ns) -> int:
    """The reference cannot be installed or run here: it has no setup.py /
    pyproject.toml, and its training path needs an external Megatron-LM fork,
    TransformerEngine and flash-attn, none of which are present offline."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    why = ("reference is not installable offline (pip: neither setup.py nor pyproject.toml) and its training "
           "entry needs the external Megatron-LM fork + TransformerEngine, absent from this image")
    if os.path.isdir(os.path.join(ref_dir, "sga")):
        why = ("the reference's training entry (forward / backward, data-parallel buckets) is an external Megatron-LM "
               "fork + TransformerEngine + flash-attn, absent from this image; the part it implements itself is "
               "measured on the same box by baseline/ref_sync_bench.py (gradient sync + optimizer step) and "
               "sga_b200/replay/bench.py --impl both (offline replay)")
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.fh,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            self.fh.close()
            sm, mx, reasons, power = [], [], set(), []
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                    power.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            if sm:
                busy = [s for s, p in zip(sm, power) if p > 0.5 * max(power)] or sm
                out = {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                       "samples": len(sm), "power_w_max": max(power)}
            os.unlink(self.path)
        except Exception:
            pass
        return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=("ours", "reference"))
    ap.add_argument("--model", type=str, default="llama3_1b")
    ap.add_argument("--mode", type=str, default="sga", choices=("sga", "dense", "nccl_baseline"))
    ap.add_argument("--global-batch", type=int, default=256)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--ratio-percent", type=float, default=1.0)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--sga-backend", type=str, default="index", choices=("index", "mask"),
                    help="index: rank-local exact top-k, (index, value) exchange; mask: shared support, mask-union reduce")
    ap.add_argument("--cycle-period", type=int, default=None, help="dense flush every N steps (mask backend default 4)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (with sequence-parallel activations)")
    ap.add_argument("--tp-comm", type=str, default="auto", choices=("auto", "fused", "library"))
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages (untied embeddings; 1F1B over NCCL p2p)")
    ap.add_argument("--bucket-elems", type=int, default=None,
                    help="gradient bucket size in elements (default: 128 Mi for the rank-local index mode, whose "
                         "per-bucket chain of kernels has a fixed cost; the trainer's 16 Mi otherwise)")
    ap.add_argument("--sga-score", type=str, default="abs_g", choices=("abs_g", "abs_m", "update", "coi"))
    ap.add_argument("--sga-checks", action="store_true",
                    help="accepted for older command lines: the engine's cross-rank checks are at their defaults (on) anyway")
    ap.add_argument("--no-sga-checks", action="store_true",
                    help="switch every cross-rank consistency check of the engine off (the engine prints its escape-hatch warning)")
    ap.add_argument("--no-exposed", action="store_true", help="skip the exposed-synchronisation measurement")
    ns = ap.parse_args()
    if ns.impl == "reference":
        return _reference_arm(ns)
    if ns.warmup < 3:
        ns.warmup = 3

    import torch
    import torch.distributed as dist

    from sga_b200 import kernels
    from sga_b200.runtime.trainer import Trainer, default_args

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != ns.gpus and int(os.environ.get("RANK", "0")) == 0:
        print(f"[bench] note: --gpus {ns.gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)
    over = dict(model=ns.model, micro_batch_size=ns.micro_batch, global_batch_size=ns.global_batch,
                train_iters=ns.steps + ns.warmup, lr=3e-4, seed=1234, data_seed=1234, log_interval=0)
    if ns.seq_len:
        over["seq_length"] = ns.seq_len
    if ns.tp > 1:
        over.update(tensor_model_parallel_size=ns.tp, tp_comm=ns.tp_comm, init_on_device=True)
    if ns.pp > 1:
        over.update(pipeline_model_parallel_size=ns.pp, untie_embeddings_and_output_weights=True)
    if ns.mode == "sga" and ns.sga_backend == "index":
        over.update(sga_enabled=True, sga_score=ns.sga_score, sga_selection="topk", sga_selection_method="exact",
                    sga_selection_ratio_percent=ns.ratio_percent, sga_backend="torch_pipelined_index",
                    sga_optimizer="adamw", sga_selection_locality="rank_local",
                    sga_cycle_period=ns.cycle_period or 0, sga_cycle_start_iter=0,
                    sga_bucket_elems=ns.bucket_elems or (128 << 20))
        if ns.no_sga_checks:
            over.update(sga_checks=False)
    elif ns.mode == "sga":
        over.update(sga_enabled=True, sga_score="abs_g", sga_selection="topk", sga_selection_method="histogram",
                    sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=ns.ratio_percent,
                    sga_backend="torch_pipelined_mask", sga_optimizer="adamw", sga_cycle_period=ns.cycle_period or 4,
                    sga_cycle_start_iter=0, sga_checks=False)
    elif ns.mode == "nccl_baseline":
        over.update(transport="nccl", dense_mode="allreduce")
    if ns.bucket_elems and "sga_bucket_elems" not in over:
        over["sga_bucket_elems"] = ns.bucket_elems
    args = default_args(**over)
    tr = Trainer(args, quiet=True)
    rank, world = tr.rank, tr.world
    dev = tr.device
    K, W = ns.steps, ns.warmup

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- warm-up (untimed) and device-resident batches for the kernel-side number
    step_id = 0
    for _ in range(W):
        tr.train_step(tr.host_batch(step_id))
        step_id += 1
    tr.check()
    dev_batches = [tr.host_batch(step_id + i).to(dev) for i in range(K)]
    sampler = ClockSampler(dev.index or 0)
    barrier()
    launches0 = kernels.launch_count()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        tr.train_step(dev_batches[i])
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else {}
    launches = kernels.launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    step_id += K
    tr.check()
    del dev_batches

    # ---- end-to-end: pinned host batch -> H2D every step, loss D2H every step
    e2e = None
    if not ns.no_e2e:
        host = [tr.host_batch(step_id + i) for i in range(K)]
        barrier()
        e0.record()
        last_loss = 0.0
        for i in range(K):
            loss = tr.train_step(host[i])
            last_loss = float(loss.item())
        e1.record()
        barrier()
        ms2 = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        tokens = tr.tokens_per_step() * K
        e2e = {"value": tokens / (float(ms2.item()) / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(host[0].numel() * host[0].element_size() * tr.dp_world),
               "d2h_bytes_per_step": 4 * world, "last_loss": last_loss}
        tr.check()

    # ---- gradient synchronisation: device time of the per-bucket sync launches, outside the timed regions
    grad_sync = None
    if tr.tp_size == 1 and tr.pp_size == 1:
        # the index backend's exchange kernels count the time they stand waiting for peers' flags
        scratch = getattr(getattr(tr.engine, "backend", None), "_scratch", None) if tr.engine is not None else None
        wait_ctr = getattr(scratch, "wait_ns", None)
        if wait_ctr is not None:
            torch.cuda.synchronize(dev)
            wait_ctr.zero_()
        tr.ddp.time_syncs = True
        for i in range(2):
            tr.train_step(tr.host_batch(step_id + K + i))
        tr.ddp.time_syncs = False
        try:
            local_ms = tr.ddp.sync_device_ms() / 2
        except Exception:  # a rank without a reading still joins the reduction below
            local_ms = 0.0
        wait_ms = float(wait_ctr.item()) / 2e6 if wait_ctr is not None else 0.0
        # max over ranks of the whole time, and of the time not spent waiting for peers
        sync_ms = torch.tensor([local_ms, max(local_ms - wait_ms, 0.0), wait_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(sync_ms, op=dist.ReduceOp.MAX)
        busy_ms, peer_wait_ms = float(sync_ms[1].item()), float(sync_ms[2].item())
        sync_ms = sync_ms[:1]
        if float(sync_ms.item()) > 0.0:
            grad_sync = {"ms_per_step": float(sync_ms.item()), "buckets": len(tr.model.arena.buckets),
                         "what": "sum over buckets of the device time of each bucket's sync launch on the "
                                 "communication stream (event pairs), mean of 2 untimed steps, max over ranks; "
                                 "runs under the backward pass"}
            if wait_ctr is not None:
                grad_sync["peer_wait_ms_per_step"] = peer_wait_ms
                grad_sync["busy_ms_per_step"] = busy_ms
                grad_sync["busy_what"] = ("ms_per_step minus the time this rank's exchange kernels stood waiting for "
                                          "peers' flags (device timer around the wait, max over ranks): ranks reach "
                                          "the end of a step milliseconds apart, and whoever is first waits")
    if grad_sync is not None and ns.mode == "sga" and ns.sga_backend == "index":
        try:
            hbm = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]) * 1e9
        except Exception:
            hbm = 6.65e12
        # per bucket: the slower of three passes over the fp32 bucket at the measured copy rate and the
        # (index, value) payload of the other ranks over NVLink at the measured peer-copy rate (770 GB/s)
        bound = 0.0
        for b in tr.model.arena.buckets:
            n = b.end - b.start
            k = max(1, round(n * ns.ratio_percent / 100.0))
            bound += max(3 * 4.0 * n / hbm, (world - 1) * k * 8.0 / 770e9)
        grad_sync["roofline_ms"] = bound * 1e3
        grad_sync["frac_of_roofline"] = bound * 1e3 / max(grad_sync["ms_per_step"], 1e-9)
        if "busy_ms_per_step" in grad_sync:
            grad_sync["frac_of_roofline_excluding_peer_wait"] = bound * 1e3 / max(grad_sync["busy_ms_per_step"], 1e-9)
        grad_sync["roofline"] = "per bucket max(3 x 4 B x n / measured HBM, (W-1) x k x 8 B / 770 GB/s)"

    # ---- exposed synchronisation: step time minus the same step with every bucket's sync skipped.
    # Runs last: the skipped steps feed the optimizer nothing, so the weights after them mean nothing.
    if grad_sync is not None and not ns.no_exposed:
        def _timed_steps(n, first):
            barrier()
            e0.record()
            for i in range(n):
                tr.train_step(tr.host_batch(first + i))
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1) / n], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        n_exp = 2 if K < 10 else 1  # long runs (many timed steps) keep this side measurement short
        with_sync = _timed_steps(n_exp, step_id + K + 2)
        tr.ddp.null_sync = True
        without = _timed_steps(n_exp, step_id + K + 4)
        tr.ddp.null_sync = False
        grad_sync["exposed_ms_per_step"] = with_sync - without
        grad_sync["exposed_what"] = ("ms per step with the buckets synchronised minus ms per step with every bucket's "
                                     "synchronisation skipped (%d + %d untimed-region steps, host-fed batches, max "
                                     "over ranks); differences below the step-to-step jitter read as zero" % (n_exp, n_exp))

    tokens = tr.tokens_per_step() * K
    value = tokens / (ms_total / 1e3)
    baseline = None
    try:
        pub = json.load(open(os.path.join(ROOT, "BASELINE.json"))).get("published", {})
        baseline = pub.get("tokens_per_sec")
    except Exception:
        pass
    par = f"dp{tr.dp_world}" if tr.tp_size == 1 else f"tp{tr.tp_size}(sp,{tr.tp.transport})xdp{tr.dp_world}"
    if tr.pp_size > 1:
        par = f"pp{tr.pp_size}(1f1b)x" + par
    line = {
        "metric": "train tokens/sec (device-timed, max over ranks)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": (value / baseline) if baseline else None, "dtype": "bf16",
        "data": "synthetic uniform token ids (seed 1234), random-init weights N(0, 0.02^2)",
        "config": {"model": tr.cfg.name, "global_batch": args.global_batch_size, "seq_len": tr.cfg.seq_len,
                   "micro_batch": args.micro_batch_size, "parallelism": par, "mode": ns.mode,
                   "sga": (("score=%s, per-bucket exact top-%g%%, index backend, residual-aware AdamW"
                            % ("|g+residual|" if ns.sga_score == "abs_g" else ns.sga_score, ns.ratio_percent)) if ns.sga_backend == "index" else
                           ("score=|g+residual|, shared support top-%g%% (balanced histogram), mask backend, "
                            "dense flush every %d steps, residual-aware AdamW"
                            % (ns.ratio_percent, ns.cycle_period or 4))) if ns.mode == "sga" else None,
                   "transport": tr.ddp.transport, "bucket_elems": int(getattr(args, "sga_bucket_elems", 0)),
                   "sharded_optimizer_step": bool(tr.sharded_state),
                   "engine_checks": ("defaults (on)" if bool(getattr(args, "sga_checks", True)) else "off")
                   if ns.mode == "sga" else None,
                   "l2": "inputs larger than L2 (weights %.1f GB, grads %.1f GB per rank)" % (
                       2e-9 * tr.model.arena.numel, 4e-9 * tr.model.arena.numel),
                   "params": tr.cfg.num_params()},
        "clocks": clocks, "e2e": e2e, "grad_sync": grad_sync, "gpu_launches": int(launches),
        "mfu_bf16_of_measured_burst": None,
    }
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        flops = tr.cfg.flops_per_token() * value / world
        line["mfu_bf16_of_measured_burst"] = flops / (peaks["bf16_tflops"] * 1e12)
        line["mfu_bf16_of_measured_sustained"] = flops / (peaks["bf16_tflops_sustained"] * 1e12)
    except Exception:
        pass
    if rank == 0:
        print(json.dumps(line), flush=True)
    tr.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
