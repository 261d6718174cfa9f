"""``python run.py --config-path DIR --config-name NAME [key=value ...] action=run|test|dryrun|query|stop``.

Loads ``DIR/NAME.yaml``, applies dotted ``key=value`` overrides (values are
parsed as yaml), validates the task, builds the backend and the launcher and
executes the action. ``dryrun`` renders every script and prints the commands
without starting anything; ``test`` runs the job in the foreground on the
local host. Reference: ``run.py``, ``sga/launcher/run.py:47-118``,
``runner_base.py:20-51``.
"""
from __future__ import annotations

import argparse
import os
import sys

import yaml

from .backend import TrainBackend
from .launcher_ssh import SshLauncher

ACTIONS = ("run", "test", "dryrun", "query", "stop")


def load_config(path: str, overrides=()) -> dict:
    with open(path) as fh:
        cfg = yaml.safe_load(fh) or {}
    for ov in overrides:
        if "=" not in ov:
            raise ValueError(f"override '{ov}' is not key=value")
        key, val = ov.split("=", 1)
        node = cfg
        parts = key.split(".")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = yaml.safe_load(val)
    return cfg


def validate_task(cfg: dict) -> None:
    task = (cfg.get("experiment", {}) or {}).get("task", {}) or {}
    if task.get("type", "train") != "train":
        raise ValueError(f"unsupported task type '{task.get('type')}' (only 'train')")
    if cfg.get("action", "run") not in ACTIONS:
        raise ValueError(f"action must be one of {ACTIONS} (got {cfg.get('action')!r})")


class Runner:
    def __init__(self, cfg: dict):
        self.cfg = cfg
        self.backend = TrainBackend(cfg)
        self.launcher = SshLauncher(cfg, self.backend)

    def execute(self, action: str):
        if action == "run":
            return self.launcher.run()
        if action == "dryrun":
            return self.launcher.run(dryrun=True, tail=False)
        if action == "test":
            import subprocess

            host, run_sh, _ = self.launcher.plan()[0]
            script = open(run_sh).read().replace("nohup ", "").rsplit(" >> ", 1)[0]
            return subprocess.run(["bash", "-c", script]).returncode
        if action == "query":
            runner = (self.config.get("experiment", {}) or {}).get("runner", {}) or {}
            if runner.get("query_timeout") is not None or runner.get("query_interval") is not None:
                st = self.launcher.query(interval=float(runner.get("query_interval", 10)),
                                         timeout=runner.get("query_timeout"))
            else:
                st = self.launcher.query_once()
            print(f"[launcher] job status: {st.value}")
            return st
        if action == "stop":
            return self.launcher.stop()
        raise ValueError(action)


def main(argv=None) -> int:
    cwd = os.getcwd()
    ap = argparse.ArgumentParser("run.py")
    ap.add_argument("--config-path", required=True)
    ap.add_argument("--config-name", required=True)
    ap.add_argument("overrides", nargs="*")
    ns = ap.parse_args(argv)
    name = ns.config_name if ns.config_name.endswith((".yaml", ".yml")) else ns.config_name + ".yaml"
    cfg = load_config(os.path.join(ns.config_path, name), ns.overrides)
    validate_task(cfg)
    try:
        Runner(cfg).execute(cfg.get("action", "run"))
    finally:
        os.chdir(cwd)
    return 0


if __name__ == "__main__":
    sys.exit(main())
