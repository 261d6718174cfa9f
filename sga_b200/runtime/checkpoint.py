"""Checkpoint writer / loader and the SGA resume guard.

Layout (the Megatron one the reference's resume guard reads,
``sga/train_gpt.py:49-194``, ``tests/test_resume_guard.py:87-114``)::

    <dir>/latest_checkpointed_iteration.txt
    <dir>/iter_0000500/mp_rank_00/model_optim_rng.pt
        {"args": Namespace (carries every sga_* attribute),
         "iteration": int, "checkpoint_version": 3.0,
         "model": {name: bf16 tensor},
         "optimizer": {"optimizer": {"state": {i: {"exp_avg", "exp_avg_sq"}},
                                     "param_groups": [{..., "step"}]},
                       "fp32_from_fp16_params": {name: fp32 tensor}},
         "rng_state": {...}}

The optimizer part is exactly ``torch.optim.Adam``'s layout. The residual (the
grad arena), the active support, the adaptive threshold and the cycle position
are not saved: a resumed engine cold-starts its calendar and runs dense steps
until the next boundary.

Guard: a resume with SGA enabled is refused unless the saved ``sga_*``
attributes equal the current ones, compared raw (defaults filled, sorted-key
JSON, spelled as given). A checkpoint with no saved SGA attributes, with
retired keys, or one that cannot be read is refused too;
``--sga-allow-config-override`` is the single escape. A missing tracker file
is a cold start and passes.
"""
from __future__ import annotations

import json
import os
import pickle
from pathlib import Path

import torch

from .. import config as C

TRACKER = "latest_checkpointed_iteration.txt"


def tracker_path(root: str) -> str:
    return os.path.join(root, TRACKER)


def checkpoint_dir(root: str, iteration: int) -> str:
    return os.path.join(root, f"iter_{iteration:07d}")


def checkpoint_name(root: str, iteration: int, tp_rank: int = 0, pp_rank: int = 0, pp_size: int = 1) -> str:
    sub = f"mp_rank_{tp_rank:02d}" if pp_size == 1 else f"mp_rank_{tp_rank:02d}_{pp_rank:03d}"
    return os.path.join(checkpoint_dir(root, iteration), sub, "model_optim_rng.pt")


def latest_iteration(root: str):
    tp = tracker_path(root)
    if not os.path.exists(tp):
        return None
    with open(tp) as fh:
        its = [int(tok) for tok in fh.read().split() if tok.isdigit()]
    return max(its) if its else None


def write_tracker(root: str, iteration: int) -> None:
    """Point ``latest_checkpointed_iteration.txt`` at ``iteration``. With several writers (tensor /
    pipeline shards, per-rank SGA state files) call it on one rank, after a barrier that follows
    every writer's last file, so that the tracker never names a checkpoint that is still incomplete."""
    os.makedirs(root, exist_ok=True)
    with open(tracker_path(root) + ".tmp", "w") as fh:
        fh.write(str(iteration))
    os.replace(tracker_path(root) + ".tmp", tracker_path(root))


def save_checkpoint(root: str, iteration: int, args, model, optimizer, rank: int = 0, tp_rank: int = 0,
                    dp_rank: int | None = None, pp_rank: int = 0, pp_size: int = 1, tracker: bool = True) -> str:
    """The first data-parallel replica writes (every replica holds the same state; a run whose
    optimizer state lives in per-rank owner slices gathers it first, ``Trainer.gather_optimizer_state``):
    one ``mp_rank_XX[_YYY]`` file per tensor-parallel rank (and pipeline stage). ``tracker`` false leaves
    the tracker file to the caller (``write_tracker`` after a barrier)."""
    path = checkpoint_name(root, iteration, tp_rank, pp_rank, pp_size)
    if (dp_rank if dp_rank is not None else rank) != 0:
        return path
    os.makedirs(os.path.dirname(path), exist_ok=True)
    state = {
        "args": args, "iteration": int(iteration), "checkpoint_version": 3.0,
        "model": {name: p.detach().cpu().clone() for name, p in model.named_parameters()},
        "optimizer": {"optimizer": {k: v for k, v in optimizer.state_dict().items() if k != "fp32_from_fp16_params"},
                      "fp32_from_fp16_params": optimizer.state_dict()["fp32_from_fp16_params"]},
        "rng_state": {"torch": torch.get_rng_state()},
    }
    tmp = path + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, path)
    if tracker and tp_rank == 0 and pp_rank == 0:
        write_tracker(root, iteration)
    return path


def sga_state_name(root: str, iteration: int, rank: int) -> str:
    return os.path.join(checkpoint_dir(root, iteration), f"sga_state_rank{rank:05d}.pt")


def save_sga_state(root: str, iteration: int, engine, rank: int) -> str:
    """Every rank writes its own file: the residual is this rank's unsent gradient mass."""
    path = sga_state_name(root, iteration, rank)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save(engine.state_dict(), path + ".tmp")
    os.replace(path + ".tmp", path)
    return path


def load_sga_state(root: str, iteration: int, engine, rank: int) -> bool:
    path = sga_state_name(root, iteration, rank)
    if not os.path.exists(path):
        return False
    engine.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
    return True


def sga_state_present_everywhere(root: str, iteration: int, rank: int, device=None) -> bool:
    """True only when every rank finds its own SGA state file: a warm resume on some ranks and a
    cold start on others would issue mismatched collectives."""
    import torch.distributed as dist

    here = os.path.exists(sga_state_name(root, iteration, rank))
    if not (dist.is_available() and dist.is_initialized()):
        return here
    dev = device if (device is not None and dist.get_backend() == "nccl") else "cpu"
    flag = torch.tensor([1 if here else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok = bool(flag.item())
    if here and not ok and rank == 0:
        print("[train] some rank has no saved SGA state: every rank cold-starts its cycle", flush=True)
    return ok


def load_checkpoint(root: str, model, optimizer, tp_rank: int = 0, pp_rank: int = 0, pp_size: int = 1):
    """Loads the latest checkpoint; returns its iteration (0 when there is none)."""
    it = latest_iteration(root)
    if it is None:
        return 0
    state = torch.load(checkpoint_name(root, it, tp_rank, pp_rank, pp_size), map_location="cpu",
                       weights_only=False)
    sd = dict(state["optimizer"]["optimizer"])
    sd["fp32_from_fp16_params"] = state["optimizer"]["fp32_from_fp16_params"]
    optimizer.load_state_dict(sd)
    if "rng_state" in state and "torch" in state["rng_state"]:
        torch.set_rng_state(state["rng_state"]["torch"])
    return int(state["iteration"])


def _config_json(owner, fallback_train_iters=None) -> str:
    attrs = dict(C.sga_defaults(), **C.sga_config_attrs(owner))
    if attrs.get("sga_cycle_start_iter_percent") is not None:
        ti = getattr(owner, "train_iters", None)
        attrs["train_iters_for_percent"] = ti if ti is not None else fallback_train_iters
    return json.dumps(attrs, sort_keys=True, default=repr)


def sga_resume_guard(args, log=print) -> None:
    """Raises ``SystemExit(1)`` when the resume must be refused."""
    if not getattr(args, "sga_enabled", False) or not getattr(args, "load", None):
        return
    if getattr(args, "sga_allow_config_override", False):
        return
    try:
        rank = int(os.environ.get("RANK", "0"))
    except ValueError:
        rank = 0
    if rank != 0:
        return
    same, detail = False, ""
    try:
        it = latest_iteration(args.load)
        if it is None:
            return
        shards = sorted(Path(checkpoint_dir(args.load, it)).glob("mp_rank_*/model_optim_rng.pt"))
        if not shards:
            raise OSError(f"no model_optim_rng.pt rank shard under {checkpoint_dir(args.load, it)}")
        state = torch.load(shards[0], map_location="cpu", weights_only=False)
        saved = state.get("args", None)
        legacy = getattr(saved, "sga_config", "") if saved is not None else ""
        saved_attrs = C.sga_config_attrs(saved) if saved is not None else {}
        if legacy:
            detail = "checkpoint predates the flat sga arguments (it saved the retired --sga-config JSON string)"
        elif not saved_attrs:
            detail = "checkpoint carries no saved sga arguments"
        else:
            retired = sorted(set(saved_attrs) - set(C.sga_defaults()))
            if retired:
                detail = (f"checkpoint carries retired sga keys {retired} (removed or renamed since it was saved); "
                          "re-spell the configuration with current names")
            else:
                same = _config_json(saved, getattr(args, "train_iters", None)) == _config_json(args)
                if not same:
                    detail = "checkpoint sga configuration differs from the current --sga-* arguments"
    except (OSError, AttributeError, KeyError, TypeError, ValueError, RuntimeError, pickle.UnpicklingError, EOFError) as e:
        detail = f"could not verify the checkpoint's saved sga configuration ({e})"
    if not same:
        log(f"[SGA] ERROR {detail}; refusing the SGA resume (pass --sga-allow-config-override to override)")
        raise SystemExit(1)
