"""Multi-node launcher of the fused replay.

Node 0's parent process writes the job description next to the trace, starts
one *node-worker* per node (over ssh, or as local subprocesses with
``SGA_LAUNCH_EXECUTOR=local`` / ``executor="local"`` so that the whole path can
be exercised on one machine), and supervises them: a bounded pre-flight
rendezvous (every rank joins a gloo group and passes one barrier) before any
real work, the first non-zero exit kills everyone, an optional run deadline
kills everyone, log tails go into the error. A node-worker spawns its local
shards with distinct global ranks; rank 0 writes the result fragment.

The parent never polls a shared filesystem for the workers' files (visibility
lag across NFS clients is unbounded); inputs are confirmed with a one-shot
size probe per node and results come back through rank 0 on node 0.
Reference: ``sga/replay_launch.py:80-812``.
"""
from __future__ import annotations

import argparse
import os
import shlex
import signal
import socket
import subprocess
import sys
import tempfile
import time
from typing import Optional

import torch

SSH_PORT = 2222


def render_ssh_argv(host: str, remote_cmd: str, ssh_key: Optional[str] = None, port: int = SSH_PORT) -> list:
    argv = ["ssh", "-p", str(port), "-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=no",
            "-o", "ServerAliveInterval=15", "-o", "ServerAliveCountMax=4"]
    if ssh_key:
        argv += ["-i", ssh_key]
    return argv + [host, remote_cmd]


def render_worker_cmd(spec_path, node_rank, nnodes, shards_per_node, master_addr, master_port, phase) -> list:
    return [sys.executable, "-m", "sga_b200.replay.launch", "--node-worker", "--spec", spec_path, "--node-rank",
            str(node_rank), "--nnodes", str(nnodes), "--shards-per-node", str(shards_per_node), "--master-addr",
            master_addr, "--master-port", str(master_port), "--phase", phase]


def render_size_probe(host, path, ssh_key=None, executor="ssh") -> list:
    cmd = f"stat -c %s {shlex.quote(path)}"
    return ["bash", "-c", cmd] if executor == "local" else render_ssh_argv(host, cmd, ssh_key)


class LaunchError(RuntimeError):
    pass


class Supervisor:
    """Runs one command per node and enforces all-or-nothing semantics."""

    def __init__(self, log_dir: Optional[str] = None, poll_s: float = 0.2):
        self.log_dir = log_dir or tempfile.mkdtemp(prefix="sga_replay_launch_")
        os.makedirs(self.log_dir, exist_ok=True)
        self.poll_s = poll_s
        self.procs = []

    def _spawn(self, argv, tag):
        log = open(os.path.join(self.log_dir, f"{tag}.log"), "w")
        try:
            p = subprocess.Popen(argv, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
        except OSError as e:
            log.close()
            raise LaunchError(f"could not start {tag}: {e}") from e
        self.procs.append((p, tag, log))
        return p

    def _kill_all(self):
        for p, _tag, _log in self.procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except (ProcessLookupError, PermissionError):
                    pass
        t_end = time.time() + 5
        for p, _tag, _log in self.procs:
            try:
                p.wait(timeout=max(0.1, t_end - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except (ProcessLookupError, PermissionError):
                    pass
                p.wait()

    def tails(self, n=15) -> str:
        out = []
        for _p, tag, log in self.procs:
            if not log.closed:
                log.flush()
            try:
                lines = open(log.name).read().splitlines()[-n:]
            except OSError:
                lines = []
            out.append(f"--- {tag} ---\n" + "\n".join(lines))
        return "\n".join(out)

    def run(self, commands, tags, deadline_s: float = 0.0, what="run") -> None:
        self.procs = []
        t0 = time.time()
        try:
            for argv, tag in zip(commands, tags):
                self._spawn(argv, tag)
            while True:
                codes = [p.poll() for p, _t, _l in self.procs]
                bad = [(c, t) for c, (_p, t, _l) in zip(codes, self.procs) if c not in (None, 0)]
                if bad:
                    self._kill_all()
                    raise LaunchError(f"{what}: {bad[0][1]} exited with code {bad[0][0]}; all workers stopped\n"
                                      + self.tails())
                if all(c == 0 for c in codes):
                    return
                if deadline_s and time.time() - t0 > deadline_s:
                    self._kill_all()
                    raise LaunchError(f"{what}: deadline of {deadline_s:.0f}s exceeded; all workers stopped\n"
                                      + self.tails())
                time.sleep(self.poll_s)
        except KeyboardInterrupt:
            self._kill_all()
            raise
        finally:
            for _p, _t, log in self.procs:
                log.close()


def worker_pid_file(spec_path: str, node_rank: int, phase: str) -> str:
    """Where a node worker records its process-group id: beside the job description, which every
    node sees at the same path."""
    return f"{spec_path}.{phase}.node{node_rank}.pgid"


def render_sweep_argv(host: str, pid_file: str, ssh_key: Optional[str] = None) -> list:
    """ssh command that ends exactly the process group a node worker recorded (and nothing else),
    then removes the record; harmless when the file or the group is already gone."""
    remote = (f"if [ -f {shlex.quote(pid_file)} ]; then kill -TERM -- -$(cat {shlex.quote(pid_file)}) 2>/dev/null; "
              f"rm -f {shlex.quote(pid_file)}; fi; true")
    return render_ssh_argv(host, remote, ssh_key)


def sweep_node_workers(hosts, spec_path: str, phase: str, ssh_key, executor: str) -> None:
    """Best-effort, out-of-band clean-up after a failed or interrupted launch. The supervisor's kill
    took the ssh clients down and a remote worker normally dies with its channel; should one have
    missed the hang-up, its GPUs would stay pinned, so every node is asked once more to end the
    process group its worker recorded at start. Never raises. Skipped for the local executor, where
    the supervisor's own kill of the child process groups is authoritative.
    Counterpart of ``sga/replay_launch.py:480-501`` (which sweeps by command-line pattern; a recorded
    process group cannot hit a stranger's process)."""
    if executor == "local":
        return
    for i, h in enumerate(hosts):
        try:
            subprocess.run(render_sweep_argv(h, worker_pid_file(spec_path, i, phase), ssh_key), capture_output=True,
                           timeout=30)
        except (OSError, subprocess.TimeoutExpired):
            pass


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def confirm_visible(hosts, path, expect_size, ssh_key, executor) -> None:
    """One size probe per node: the job description must be the file we wrote."""
    for h in hosts:
        res = subprocess.run(render_size_probe(h, path, ssh_key, executor), capture_output=True, text=True)
        if res.returncode != 0 or res.stdout.strip() != str(expect_size):
            raise LaunchError(f"{path} is not visible on {h} with the expected size {expect_size} "
                              f"(got {res.stdout.strip()!r}, rc {res.returncode})")


def run_fused_branch_multinode(ns, t0, cfgs, horizons, scores, ratios, executor: Optional[str] = None):
    hosts = [h for h in str(ns.nodes).split(",") if h]
    executor = executor or os.environ.get("SGA_LAUNCH_EXECUTOR", "ssh")
    if executor not in ("ssh", "local"):
        raise ValueError(f"SGA_LAUNCH_EXECUTOR must be ssh or local (got {executor!r})")
    nnodes = len(hosts)
    if ns.fused_shards % nnodes:
        raise ValueError("--fused-shards must be a multiple of the number of nodes")
    spn = ns.fused_shards // nnodes
    work = ns.launch_log_dir or tempfile.mkdtemp(prefix="sga_replay_")
    os.makedirs(work, exist_ok=True)
    spec_path = os.path.join(work, f"job_t{t0}.pt")
    out_path = os.path.join(work, f"frag_t{t0}.pt")
    spec = dict(trace_dir=os.path.abspath(ns.trace_dir), t0=t0, configs=list(cfgs), window=ns.window,
                horizons=list(horizons), device=ns.device, dense_cache=ns.dense_cache,
                max_configs=ns.fused_max_configs, state_budget_mb=ns.fused_state_budget_mb,
                score_names=list(scores), ratios=list(ratios), out_path=out_path)
    torch.save(spec, spec_path)
    confirm_visible(hosts, spec_path, os.path.getsize(spec_path), ns.ssh_key, executor)
    master = "127.0.0.1" if executor == "local" else hosts[0]
    sup = Supervisor(os.path.join(work, "logs"))
    for phase, deadline in (("preflight", ns.preflight_timeout), ("run", ns.run_deadline)):
        port = _free_port()
        cmds = []
        for i, h in enumerate(hosts):
            wc = render_worker_cmd(spec_path, i, nnodes, spn, master, port, phase)
            cmds.append(wc if executor == "local" else render_ssh_argv(h, " ".join(shlex.quote(x) for x in wc),
                                                                       ns.ssh_key))
        try:
            sup.run(cmds, [f"{phase}_node{i}" for i in range(nnodes)], deadline_s=deadline, what=phase)
        except (LaunchError, KeyboardInterrupt):
            sweep_node_workers(hosts, spec_path, phase, ns.ssh_key, executor)
            raise
    return torch.load(out_path, weights_only=False)


# ---------------------------------------------------------------- node worker
def _child(local_rank, node_rank, spn, world, master_addr, master_port, spec, phase):
    import datetime

    import torch.distributed as dist

    from . import fused as RF

    rank = int(os.environ.get("SGA_GLOBAL_RANK", node_rank * spn + local_rank))
    os.environ.update(MASTER_ADDR=master_addr, MASTER_PORT=str(master_port))
    device = spec["device"]
    cuda = str(device).startswith("cuda")
    if cuda:
        torch.cuda.set_device(local_rank)
        device = f"cuda:{local_rank}"
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(hours=2))
    try:
        if phase == "preflight":
            dist.barrier()
            return
        dist.all_reduce(torch.zeros(1, device=device if cuda else "cpu"))  # communicator set-up outside the engine's timers
        kw = {k: v for k, v in spec.items() if k != "out_path"}
        kw["device"] = device
        frag = RF.run_shard(rank, world, **kw)
        if rank == 0:
            tmp = spec["out_path"] + ".tmp"
            torch.save(frag, tmp)
            os.replace(tmp, spec["out_path"])
    finally:
        dist.destroy_process_group()


def node_worker(ns) -> int:
    import torch.multiprocessing as mp

    spec = torch.load(ns.spec, weights_only=False)
    world = ns.nnodes * ns.shards_per_node
    # own process group, recorded for the launcher's out-of-band sweep; the shards spawned below join it
    pid_file = worker_pid_file(ns.spec, ns.node_rank, ns.phase)
    try:
        if os.getpgrp() != os.getpid():
            os.setpgid(0, 0)
        with open(pid_file, "w") as fh:
            fh.write(str(os.getpgrp()))
    except OSError:
        pid_file = None
    try:
        return _run_shards(mp, ns, spec, world)
    finally:
        if pid_file:
            try:
                os.remove(pid_file)
            except OSError:
                pass


def _run_shards(mp, ns, spec, world) -> int:
    mp.spawn(_child, args=(ns.node_rank, ns.shards_per_node, world, ns.master_addr, ns.master_port, spec, ns.phase),
             nprocs=ns.shards_per_node, join=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("sga_b200.replay.launch")
    ap.add_argument("--node-worker", action="store_true")
    ap.add_argument("--spec")
    ap.add_argument("--node-rank", type=int, default=0)
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--shards-per-node", type=int, default=1)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=29555)
    ap.add_argument("--phase", choices=("preflight", "run"), default="run")
    ns = ap.parse_args(argv)
    if not ns.node_worker:
        ap.error("this module is started by the replay CLI (--nodes ...); pass --node-worker to run a node")
    return node_worker(ns)


if __name__ == "__main__":
    sys.exit(main())
