"""Launcher helpers: hostfile parsing, yaml -> flag flattening, ssh / scp / local
command execution, free ports, per-node overrides, log tailing.
Reference: ``sga/launcher/utils.py:16-503``.
"""
from __future__ import annotations

import os
import shlex
import socket
import subprocess
import threading
import time
from typing import Optional


def parse_hostfile(path: Optional[str]) -> list:
    """``<host> slots=<n> [type=<T>]`` per line, ``#`` comments. Returns
    ``[{"host", "slots", "type"}]``; no file means one local node."""
    if not path or not os.path.exists(path):
        return []
    out, seen = [], set()
    with open(path) as fh:
        for ln, raw in enumerate(fh, 1):
            line = raw.split("#", 1)[0].strip()
            if not line:
                continue
            parts = line.split()
            host, slots, typ = parts[0], None, None
            for tok in parts[1:]:
                if tok.startswith("slots="):
                    slots = int(tok[6:])
                elif tok.startswith("type="):
                    typ = tok[5:]
                else:
                    raise ValueError(f"{path}:{ln}: cannot parse '{tok}' (expected slots=<n> or type=<T>)")
            if slots is None or slots < 1:
                raise ValueError(f"{path}:{ln}: host '{host}' needs slots=<n> with n >= 1")
            if host in seen:
                raise ValueError(f"{path}:{ln}: duplicate host '{host}'")
            seen.add(host)
            out.append({"host": host, "slots": slots, "type": typ})
    return out


def flatten_dict_to_args(d: dict, ignore=()) -> list:
    """``{"micro_batch_size": 4, "flag": True}`` -> ``["--micro-batch-size", "4", "--flag"]``.
    ``False`` / ``None`` values are dropped, lists are space-joined arguments, nested dicts are flattened
    in place (``sga/launcher/utils.py:269-290``)."""
    out = []
    for key, val in d.items():
        if key in ignore or val is None or val is False:
            continue
        if isinstance(val, dict):  # nested sections (checkpoint:, logging:) flatten into the same flag list
            out.extend(flatten_dict_to_args(val, ignore))
            continue
        flag = "--" + str(key).replace("_", "-")
        if val is True:
            out.append(flag)
        elif isinstance(val, (list, tuple)):
            out.append(flag)
            out.extend(str(v) for v in val)
        else:
            out.extend([flag, str(val)])
    return out


def get_free_port() -> int:
    s = socket.socket()
    s.bind(("", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def ssh_argv(host: str, cmd: str, port: int = 22, key: Optional[str] = None, background: bool = False) -> list:
    argv = ["ssh"] + (["-f", "-n"] if background else []) + ["-p", str(port), "-o", "BatchMode=yes", "-o",
                                                             "StrictHostKeyChecking=no", "-o",
                                                             "ServerAliveInterval=30"]
    if key or os.environ.get("SGA_SSH_KEY"):
        argv += ["-i", key or os.environ["SGA_SSH_KEY"]]
    return argv + [host, cmd]


def scp_argv(host: str, src: str, dst: str, port: int = 22, key: Optional[str] = None) -> list:
    argv = ["scp", "-P", str(port), "-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=no"]
    if key or os.environ.get("SGA_SSH_KEY"):
        argv += ["-i", key or os.environ["SGA_SSH_KEY"]]
    return argv + [src, f"{host}:{dst}"]


def run_local(cmd: str, dryrun: bool = False, wait: bool = True):
    if dryrun:
        print(f"[dryrun] {cmd}")
        return 0
    p = subprocess.Popen(["bash", "-c", cmd])
    return p.wait() if wait else p


def run_ssh(host, cmd, port=22, key=None, dryrun=False, background=False):
    argv = ssh_argv(host, cmd, port, key, background)
    if dryrun:
        print("[dryrun] " + " ".join(shlex.quote(a) for a in argv))
        return 0
    return subprocess.run(argv).returncode


def run_scp(host, src, dst, port=22, key=None, dryrun=False):
    argv = scp_argv(host, src, dst, port, key)
    if dryrun:
        print("[dryrun] " + " ".join(shlex.quote(a) for a in argv))
        return 0
    return subprocess.run(argv).returncode


def is_local(host: str) -> bool:
    return host in ("localhost", "127.0.0.1", socket.gethostname())


def node_overrides(config: dict, host: str, node_type: Optional[str]) -> dict:
    """Per-host / per-type env overrides: ``experiment.node_envs: {<host or type>: {K: V}}``."""
    table = (config.get("experiment", {}) or {}).get("node_envs", {}) or {}
    out = {}
    for key in (node_type, host):
        if key and key in table:
            out.update(table[key])
    return out


def find_latest_stdout_log(root: str) -> Optional[str]:
    """The ``stdout.log`` to follow on the console: torchrun (with ``--log-dir`` / ``--redirects``)
    writes ``<root>/.../<run>/attempt_<N>/<local rank>/stdout.log``. Of the directories that hold
    attempts the lexicographically last (newest timestamp / run id) wins, inside it the highest
    attempt number, inside that the highest local rank that has a log. ``None`` when there is none yet.
    Same choice as ``sga/launcher/utils.py:397-443``."""
    if not os.path.isdir(root):
        return None
    holders = sorted((d for d, subs, _f in os.walk(root) if any(x.startswith("attempt_") for x in subs)),
                     reverse=True)
    if not holders:
        return None

    def number(name: str, prefix: str = "") -> int:
        tail = name[len(prefix):]
        return int(tail) if tail.isdigit() else -1

    run = holders[0]
    attempts = sorted((x for x in os.listdir(run) if x.startswith("attempt_")),
                      key=lambda x: number(x, "attempt_"), reverse=True)
    if not attempts:
        return None
    attempt = os.path.join(run, attempts[0])
    try:
        ranks = sorted((x for x in os.listdir(attempt) if x.isdigit()), key=int, reverse=True)
    except OSError:
        return None
    for r in ranks:
        log = os.path.join(attempt, r, "stdout.log")
        if os.path.exists(log):
            return log
    return None


class LogTailer:
    """Follows a file from its current end and prints new lines (node 0's log)."""

    def __init__(self, path, prefix: str = "", poll_s: float = 0.5, out=print):
        # ``path``: a file name, or a callable returning the current file to follow (or None while
        # there is none yet), e.g. ``lambda: find_latest_stdout_log(log_dir)``
        self.path, self.prefix, self.poll_s, self.out = path, prefix, poll_s, out
        self._stop = threading.Event()
        self._t = None

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def _run(self):
        pos, current = 0, None
        while not self._stop.is_set():
            path = self.path() if callable(self.path) else self.path
            if path != current:
                pos, current = 0, path  # a new attempt's log: start at its beginning
            if path is None:
                time.sleep(self.poll_s)
                continue
            try:
                with open(path) as fh:
                    fh.seek(pos)
                    for line in fh:
                        self.out(self.prefix + line.rstrip("\n"))
                    pos = fh.tell()
            except OSError:
                pass
            time.sleep(self.poll_s)

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join(2)
