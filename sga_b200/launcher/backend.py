"""Launcher backend: turns a launch yaml into the trainer's command line and the
per-host run / stop scripts.

``train.{system,model,data}`` keys become trainer flags (``_`` -> ``-``); the
``sga:`` section becomes the flat ``--sga-*`` flags, one to one, and is
pre-validated by parsing exactly the flags about to be emitted with the real
parser and running ``validate_sga_args`` on the result, so a bad config dies
at launch, not on the cluster. Experiment, log and checkpoint directories are
wired under ``experiment.exp_dir``.
Reference: ``sga/launcher/backend_megatron.py:33-342``, ``backend_base.py``.
"""
from __future__ import annotations

import argparse
import os
import shlex

from ..config import sga_actions, validate_sga_args
from ..config.arguments import sga_int_or_null
from .utils import flatten_dict_to_args


class BackendBase:
    def __init__(self, config: dict):
        self.config = config

    def generate_run_script(self, *a, **k):
        raise NotImplementedError

    def generate_stop_script(self, *a, **k):
        raise NotImplementedError


def sga_section_to_flags(config: dict) -> list:
    sga = dict(config.get("sga") or {})
    bad = [k for k in sga if not (isinstance(k, str) and k.startswith("sga_"))]
    if bad:
        raise ValueError(f"sga: keys must be the full flat sga_* names (got {sorted(bad)})")
    acts = sga_actions()
    unknown = sorted(k for k in sga if k not in acts)
    if unknown:
        raise ValueError(f"sga: unknown keys {unknown}")
    flags = []
    for dest in sorted(sga):
        value, action = sga[dest], acts[dest]
        if value is None:
            if dest == "sga_enabled":
                raise ValueError("sga_enabled is explicitly null in the sga: section; spell it true or false")
            if action.type is sga_int_or_null:
                flags += [action.option_strings[0], "null"]
            continue
        if isinstance(value, bool):
            value = "true" if value else "false"
        elif isinstance(value, (list, tuple)):
            value = ",".join(str(v) for v in value)
        else:
            value = str(value)
        flags += [action.option_strings[0], value]
    return flags


def prevalidate_sga(flags: list, train_iters=None, pp=1):
    from ..config.arguments import add_sga_args

    p = argparse.ArgumentParser(add_help=False)
    add_sga_args(p)
    try:
        ns = p.parse_args(flags)
    except SystemExit:
        raise ValueError(f"sga: section does not parse as flags: {flags}") from None
    ns.train_iters = train_iters
    ns.pipeline_model_parallel_size = pp
    validate_sga_args(ns)
    return ns


class TrainBackend(BackendBase):
    def __init__(self, config: dict):
        super().__init__(config)
        self._prepare()

    def _prepare(self) -> None:
        exp = self.config.setdefault("experiment", {})
        exp_dir = os.path.abspath(exp.get("exp_dir", "./outputs"))
        exp["exp_dir"] = exp_dir
        train = self.config.setdefault("train", {})
        system = train.setdefault("system", {})
        ckpt = system.setdefault("checkpoint", {}) if isinstance(system.get("checkpoint", {}), dict) else {}
        self.log_dir = os.path.join(exp_dir, "logs")
        self.ckpt_dir = os.path.join(exp_dir, "checkpoints")
        self.script_dir = os.path.join(self.log_dir, "scripts")
        self.pid_dir = os.path.join(self.log_dir, "pids")
        if ckpt.get("save", True) and "save" not in system:
            system["save"] = self.ckpt_dir
        if ckpt.get("load") and "load" not in system:
            system["load"] = ckpt["load"] if isinstance(ckpt["load"], str) else self.ckpt_dir
        system.pop("checkpoint", None)
        # scalars go under the experiment directory unless the yaml names another place
        # (sga/launcher/backend_megatron.py:180-190)
        logging_cfg = system.get("logging") if isinstance(system.get("logging"), dict) else None
        if "tensorboard_dir" not in system and not (logging_cfg and logging_cfg.get("tensorboard_dir")):
            system["tensorboard_dir"] = os.path.join(exp_dir, "tensorboard")
        self.train_args = self._train_args()

    def _train_args(self) -> list:
        train = self.config.get("train", {})
        flat = {}
        for section in ("system", "model", "data"):
            flat.update(train.get(section) or {})
        args = flatten_dict_to_args(flat)
        sga_flags = sga_section_to_flags(self.config)
        prevalidate_sga(sga_flags, flat.get("train_iters"), flat.get("pipeline_model_parallel_size", 1) or 1)
        # the trainer's own parser must accept what we are about to emit
        from ..runtime.trainer import build_parser

        try:
            build_parser().parse_args(args + sga_flags)
        except SystemExit:
            raise ValueError(f"train: section does not parse as trainer flags: {args}") from None
        return args + sga_flags

    def entrypoint(self) -> str:
        ep = (self.config.get("experiment", {}).get("task", {}) or {}).get("entrypoint")
        return ep or "-m sga_b200.train_gpt"

    def generate_run_script(self, host: str, node_rank: int, runner_cmd: list, envs: dict, background: bool = True,
                            before_start: str = "") -> str:
        os.makedirs(self.script_dir, exist_ok=True)
        os.makedirs(self.pid_dir, exist_ok=True)
        path = os.path.join(self.script_dir, f"host_{node_rank}_{host}_run.sh")
        log = os.path.join(self.log_dir, f"host_{node_rank}_{host}.output")
        pid = os.path.join(self.pid_dir, f"host_{node_rank}_{host}.pid")
        cmd = " ".join(shlex.quote(x) for x in runner_cmd + self.entrypoint().split() + self.train_args)
        lines = ["#!/bin/bash", "set -o pipefail", before_start.strip(),
                 f"mkdir -p {shlex.quote(self.log_dir)} {shlex.quote(self.pid_dir)}"]
        lines += [f"export {k}={shlex.quote(str(v))}" for k, v in envs.items()]
        lines.append(f"cd {shlex.quote(os.getcwd())}")
        if background:
            lines.append(f"nohup {cmd} >> {shlex.quote(log)} 2>&1 & echo $! > {shlex.quote(pid)}")
        else:
            lines.append(f"{cmd} 2>&1 | tee -a {shlex.quote(log)}")
        with open(path, "w") as fh:
            fh.write("\n".join(l for l in lines if l) + "\n")
        os.chmod(path, 0o755)
        return path

    def generate_stop_script(self, host: str, node_rank: int, after_stop: str = "") -> str:
        os.makedirs(self.script_dir, exist_ok=True)
        path = os.path.join(self.script_dir, f"host_{node_rank}_{host}_stop.sh")
        pid = os.path.join(self.pid_dir, f"host_{node_rank}_{host}.pid")
        body = ["#!/bin/bash", f"if [ -f {shlex.quote(pid)} ]; then", f"  pid=$(cat {shlex.quote(pid)})",
                "  kill -- -$(ps -o pgid= $pid | tr -d ' ') 2>/dev/null || kill $pid 2>/dev/null",
                f"  rm -f {shlex.quote(pid)}", "fi", after_stop.strip()]
        with open(path, "w") as fh:
            fh.write("\n".join(l for l in body if l) + "\n")
        os.chmod(path, 0o755)
        return path
