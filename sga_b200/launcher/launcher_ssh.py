"""ssh + torchrun launcher: one torchrun per host, started over ssh (or
directly for local hosts), node 0's log tailed to the console, query and stop
through pid files.

Per host the launcher builds the torchrun argv (static or c10d rendezvous,
node rank, master address / port), the environment (``experiment.envs`` plus
per-node overrides), an optional ``nsys profile`` prefix, renders the run
script through the backend and executes it. There is no elastic support: a
node that dies ends the job.
Reference: ``sga/launcher/launcher_ssh.py:30-537``, ``launcher_base.py``.
"""
from __future__ import annotations

from typing import Optional

import enum
import os
import sys
from multiprocessing.pool import ThreadPool

from .utils import (LogTailer, get_free_port, is_local, node_overrides, parse_hostfile, run_local, run_scp, run_ssh)


class JobStatus(enum.Enum):
    RUNNING = "running"
    TRANSITIONAL = "transitional"      # some nodes up, some down
    COMPLETED_OR_IDLE = "completed_or_idle"


class LauncherBase:
    def __init__(self, config, backend):
        self.config, self.backend = config, backend

    def run(self, *a, **k):
        raise NotImplementedError

    def stop(self, *a, **k):
        raise NotImplementedError


def torchrun_argv(runner: dict, nnodes: int, node_rank: int, nproc: int, master_addr: str, master_port: int) -> list:
    argv = [sys.executable, "-m", "torch.distributed.run", "--nnodes", str(nnodes), "--nproc-per-node", str(nproc)]
    rdzv = runner.get("rdzv_backend", "static")
    if rdzv == "static":
        argv += ["--node-rank", str(node_rank), "--master-addr", master_addr, "--master-port", str(master_port)]
    else:
        argv += ["--rdzv-backend", rdzv, "--rdzv-endpoint", f"{master_addr}:{master_port}", "--rdzv-id",
                 str(runner.get("rdzv_id", "sga"))]
    if runner.get("log_dir"):
        argv += ["--log-dir", runner["log_dir"], "--redirects", "3", "--tee", "3"]
    return argv


def nsys_prefix(runner: dict, node_rank: int) -> list:
    if not (runner.get("nsys_bin_path") and runner.get("nsys_rep_file_path")):
        return []
    return [runner["nsys_bin_path"], "profile", "-s", "none", "-t", "nvtx,cuda,osrt", "--capture-range=cudaProfilerApi",
            "-o", f"{runner['nsys_rep_file_path']}_node{node_rank}", "--force-overwrite", "true"]


class SshLauncher(LauncherBase):
    def __init__(self, config, backend):
        super().__init__(config, backend)
        exp = config.get("experiment", {})
        self.runner = exp.get("runner", {}) or {}
        hosts = parse_hostfile(self.runner.get("hostfile"))
        nnodes = int(self.runner.get("nnodes", len(hosts) or 1))
        if hosts:
            self.hosts = hosts[:nnodes]
        else:
            self.hosts = [{"host": "localhost", "slots": int(self.runner.get("nproc_per_node", 1)), "type": None}]
        self.ssh_port = int(self.runner.get("ssh_port", 22))
        self.master_addr = self.runner.get("master_addr") or (
            "127.0.0.1" if is_local(self.hosts[0]["host"]) else self.hosts[0]["host"])
        self.master_port = int(self.runner.get("master_port") or get_free_port())
        self.envs = dict(exp.get("envs", {}) or {})
        self.cmds = exp.get("cmds", {}) or {}
        self._tailer = None

    def plan(self) -> list:
        """Per-node (host, run script path, stop script path); pure rendering."""
        out = []
        for rank, h in enumerate(self.hosts):
            nproc = int(self.runner.get("nproc_per_node", h["slots"]))
            argv = nsys_prefix(self.runner, rank) + torchrun_argv(self.runner, len(self.hosts), rank, nproc,
                                                                  self.master_addr, self.master_port)
            envs = dict(self.envs)
            envs.update(node_overrides(self.config, h["host"], h["type"]))
            run_sh = self.backend.generate_run_script(h["host"], rank, argv, envs, background=True,
                                                      before_start=self.cmds.get("before_start", ""))
            stop_sh = self.backend.generate_stop_script(h["host"], rank, self.cmds.get("after_stop", ""))
            out.append((h["host"], run_sh, stop_sh))
        return out

    def _exec(self, host, script, dryrun):
        if is_local(host):
            return run_local(f"bash {script}", dryrun=dryrun)
        if self.runner.get("no_shared_fs"):
            run_ssh(host, f"mkdir -p {os.path.dirname(script)}", self.ssh_port, dryrun=dryrun)
            run_scp(host, script, script, self.ssh_port, dryrun=dryrun)
        return run_ssh(host, f"bash {script}", self.ssh_port, dryrun=dryrun, background=True)

    def run(self, dryrun: bool = False, tail: bool = True):
        plan = self.plan()
        if tail and not dryrun:
            log0 = os.path.join(self.backend.log_dir, f"host_0_{plan[0][0]}.output")
            os.makedirs(self.backend.log_dir, exist_ok=True)
            open(log0, "a").close()
            self._tailer = LogTailer(log0, prefix="[node0] ").start()
        with ThreadPool(len(plan)) as pool:
            codes = pool.starmap(self._exec, [(h, run_sh, dryrun) for h, run_sh, _ in plan])
        return codes

    def stop(self, dryrun: bool = False):
        with ThreadPool(len(self.hosts)) as pool:
            codes = pool.starmap(self._exec, [(h, stop_sh, dryrun) for h, _, stop_sh in self.plan()])
        if self._tailer:
            self._tailer.stop()
        return codes

    def query(self, interval: float = 10.0, timeout: Optional[float] = None, out=print):
        """Poll the job status every ``interval`` seconds and report it through ``out``; with a
        ``timeout`` stop after that many seconds, without one keep going until interrupted (Ctrl-C).
        Blocking; returns the last status seen. ``query_once`` is the non-blocking form.
        (``sga/launcher/launcher_ssh.py:500-537``.)"""
        import time

        start, last = time.time(), None
        try:
            while timeout is None or time.time() - start < timeout:
                last = self.query_once()
                out(f"Job status: {last.name}")
                time.sleep(max(0.0, float(interval)))
            out(f"Query timeout reached ({timeout}s)")
        except KeyboardInterrupt:
            out("Query interrupted by user")
        return last

    def query_once(self) -> JobStatus:
        alive = 0
        for rank, h in enumerate(self.hosts):
            pid_file = os.path.join(self.backend.pid_dir, f"host_{rank}_{h['host']}.pid")
            cmd = f"test -f {pid_file} && kill -0 $(cat {pid_file}) 2>/dev/null"
            rc = run_local(cmd) if is_local(h["host"]) else run_ssh(h["host"], cmd, self.ssh_port)
            alive += rc == 0
        if alive == len(self.hosts):
            return JobStatus.RUNNING
        return JobStatus.COMPLETED_OR_IDLE if alive == 0 else JobStatus.TRANSITIONAL
