"""Training entry (the torchrun target): ``python -m sga_b200.train_gpt --model
llama3_1b --sga-enabled true ...``.

Parses the trainer and ``--sga-*`` flags, installs the backend timer when
asked, runs the resume guard, builds the trainer, optionally loads a
checkpoint, trains on synthetic tokens, logs throughput, saves checkpoints.
Counterpart of ``sga/train_gpt.py:212-252``.
"""
from __future__ import annotations

import sys
import time

import torch

from .runtime import checkpoint as ckpt
from .runtime.trainer import Trainer, build_parser


def _save(args, tr, iteration: int) -> None:
    """One complete checkpoint: owner slices of the optimizer state gathered, every shard and every
    rank's SGA state file written, and only then (after a barrier) the tracker."""
    import torch.distributed as dist

    tr.gather_optimizer_state()
    ckpt.save_checkpoint(args.save, iteration, args, tr.model, tr.optimizer, tr.rank, tr.tp_rank, tr.dp_rank,
                         tr.pp_rank, tr.pp_size, tracker=False)
    if args.save_sga_state and tr.engine is not None:
        ckpt.save_sga_state(args.save, iteration, tr.engine, tr.rank)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if tr.rank == 0:
        ckpt.write_tracker(args.save, iteration)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    ckpt.sga_resume_guard(args)
    tr = Trainer(args)
    start = 0
    if args.load:
        start = ckpt.load_checkpoint(args.load, tr.model, tr.optimizer, tr.tp_rank, tr.pp_rank, tr.pp_size)
        tr.iteration = start
        warm = bool(start and args.save_sga_state and tr.engine is not None
                    and ckpt.sga_state_present_everywhere(args.load, start, tr.rank, tr.device)
                    and ckpt.load_sga_state(args.load, start, tr.engine, tr.rank))
        if tr.rank == 0 and start:
            print(f"[train] resumed from iteration {start} " + (
                "with the saved residual and support" if warm else
                "(the SGA cycle cold-starts: dense steps until the next boundary; discard the first post-resume "
                "timing)"), flush=True)
    cuda = tr.device.type == "cuda"
    tb = None
    if getattr(args, "tensorboard_dir", None) and tr.rank == 0:
        try:
            from torch.utils.tensorboard import SummaryWriter

            tb = SummaryWriter(args.tensorboard_dir)
        except ImportError:
            print("[train] --tensorboard-dir given but tensorboard is not installed: no scalars are written", flush=True)
    t_last = time.perf_counter()
    for it in range(start + 1, args.train_iters + 1):
        loss = tr.train_step(tr.host_batch(it - 1))
        if args.log_interval and it % args.log_interval == 0:
            lv = float(loss.item())
            if cuda:
                torch.cuda.synchronize()
            now = time.perf_counter()
            dt = (now - t_last) / args.log_interval
            t_last = now
            if tr.rank == 0:
                gn = tr.last_grad_norm
                gn = float(gn.item()) if hasattr(gn, "item") else (float(gn) if gn is not None else float("nan"))
                extra = ""
                if getattr(args, "log_params_norm", False):  # this rank's parameters (a shard under TP / PP)
                    # the bf16 copies are complete on every rank; the fp32 masters may live in owner slices
                    extra += f" | params norm {float(tr.model.arena.model_param.float().norm()):.4f}"
                extra += f" | lr {tr.optimizer.param_groups[0]['lr']:.3e}"
                print(f"[train] iteration {it}/{args.train_iters} | loss {lv:.6f} | grad norm {gn:.4f}{extra} | "
                      f"{dt * 1e3:.1f} ms/step | {tr.tokens_per_step() / dt:.0f} tokens/s", flush=True)
                if tb is not None:
                    for tag, val in (("lm loss", lv), ("grad-norm", gn), ("learning-rate", tr.optimizer.param_groups[0]["lr"]),
                                     ("iteration-time", dt), ("tokens-per-second", tr.tokens_per_step() / dt)):
                        tb.add_scalar(tag, val, it)
        if args.eval_interval and it % args.eval_interval == 0:
            val = tr.evaluate(args.eval_iters)
            if tr.rank == 0:
                print(f"[train] validation loss at iteration {it} | {val:.6f} | {args.eval_iters} batches", flush=True)
                if tb is not None:
                    tb.add_scalar("lm loss validation", val, it)
        if args.save and args.save_interval and it % args.save_interval == 0:
            _save(args, tr, it)
        if args.exit_interval and it % args.exit_interval == 0 and it < args.train_iters:
            if args.save:
                _save(args, tr, it)
            if tr.rank == 0:
                print(f"[train] exiting at iteration {it} (--exit-interval {args.exit_interval})", flush=True)
            if tb is not None:
                tb.close()
            tr.check()
            tr.close()
            return 0
    if args.save:
        _save(args, tr, args.train_iters)
    if tb is not None:
        tb.close()
    tr.check()
    tr.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
