"""Replay CLI and the multi-node launcher with the local executor: node-workers
are local subprocesses that rendezvous on 127.0.0.1 with distinct global
ranks; failure modes are simulated with sleep / exit stand-ins; ssh command
lines are pinned as strings and never executed."""
import json
import os
import sys
import time

import pytest
import torch

from sga_b200.replay import cli, launch
from sga_b200.replay.synth import make_synthetic_trace


@pytest.fixture(scope="module")
def trace(tmp_path_factory):
    return make_synthetic_trace(str(tmp_path_factory.mktemp("trace")), sizes=(4000, 3000, 1700), steps=8,
                                g_dtype="bf16", seed=5)


def _cli(trace, tmp_path, *extra):
    out = tmp_path / "report.json"
    argv = ["--trace-dir", trace, "--ratios", "5,20", "--replay-mode", "cycle", "--cycle-lens", "1,4", "--score-names",
            "abs_g,update", "--window", "8", "--horizons", "4,8", "--out", str(out)] + list(extra)
    assert cli.main(argv) == 0
    return json.load(open(out))


def test_cli_report_shape(trace, tmp_path, capsys):
    rep = _cli(trace, tmp_path)
    assert set(rep) >= {"trace_dir", "config", "branch_results"}
    br = rep["branch_results"]["0"]
    assert br["window_len"] == 8 and br["horizon_steps"] == {"4": 4, "8": 8} and br["cycle_lens"] == [1, 4]
    assert set(br["per_ratio"]) == {"5.0", "20.0"}
    keys = set(br["per_ratio"]["5.0"]["scores"])
    assert keys == {"abs_g@T1", "abs_g@T4", "update@T1", "update@T4"}, "suffix only for multi-valued axes"
    s = br["per_ratio"]["5.0"]["scores"]["abs_g@T4"]
    assert set(s["distortion"]) == {"4", "8"} and 0 < s["distortion"]["8"] < 5
    assert {"ndcg_at_k", "recall_at_k", "missed_label_mass", "missed_score_mass"} <= set(s)
    # more retained coordinates -> less distortion
    assert br["per_ratio"]["20.0"]["scores"]["abs_g@T4"]["distortion"]["8"] < s["distortion"]["8"]
    assert "distortion" in capsys.readouterr().out
    rep2 = _cli(trace, tmp_path, "--cycle-len", "4", "--cycle-lens", "") if False else None  # noqa: F841
    with pytest.raises(ValueError, match="not both"):
        cli.build_configs(cli.build_parser().parse_args(["--trace-dir", trace, "--cycle-len", "2", "--cycle-lens",
                                                         "1,2"]))
    with pytest.raises(ValueError, match="unknown score"):
        cli.build_configs(cli.build_parser().parse_args(["--trace-dir", trace, "--score-names", "nope"]))


def test_cli_absent_branch_point_and_single_axis_keys(trace, tmp_path):
    out = tmp_path / "r.json"
    cli.main(["--trace-dir", trace, "--branch-point", "0,3", "--ratios", "10", "--score-names", "abs_g", "--window",
              "8", "--replay-mode", "cycle", "--out", str(out)])
    rep = json.load(open(out))
    assert rep["branch_results"]["3"] == {"t0": 3, "state_absent": True}
    assert set(rep["branch_results"]["0"]["per_ratio"]["10.0"]["scores"]) == {"abs_g"}
    assert rep["config"]["cycle_lens"] == [20] and rep["config"]["selection_semantics"] == "balanced-histogram"
    # the default mode is zerofill, which exists for exact top-k only: the default selection rule is refused there
    with pytest.raises(ValueError, match="requires --replay-mode cycle"):
        cli.main(["--trace-dir", trace, "--ratios", "10", "--score-names", "abs_g", "--window", "8"])
    with pytest.raises(ValueError, match="only supported with --replay-mode cycle"):
        cli.main(["--trace-dir", trace, "--selection-semantics", "topk", "--fold", "on"])
    cli.main(["--trace-dir", trace, "--ratios", "10", "--score-names", "abs_g", "--window", "8", "--selection-semantics",
              "topk", "--out", str(out)])
    z = json.load(open(out))["branch_results"]["0"]
    assert "cycle_lens" not in z and set(z["per_ratio"]["10.0"]["scores"]) == {"abs_g"}
    assert 0 < z["per_ratio"]["10.0"]["scores"]["abs_g"]["distortion"]["8"] < 5


def test_self_check_on_a_real_trace(tmp_path):
    from sga_b200.runtime.trainer import Trainer, default_args

    tr = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=2, train_iters=8, device="cpu",
                              lr=1e-3, sga_bucket_elems=30000, log_interval=0, sga_enabled=True, sga_shadow=True,
                              sga_score="abs_g", sga_selection_method="histogram",
                              sga_selection_histogram_mode="balanced", sga_selection_ratio_percent=10.0,
                              sga_backend="torch_pipelined_index", sga_cycle_period=2, sga_trace_dir=str(tmp_path),
                              sga_trace_branch_points="1,4", sga_trace_window=4), quiet=True)
    for s in range(8):
        tr.train_step(tr.host_batch(s))
    tr.close()
    res = cli.self_check(str(tmp_path), 1, 4)
    assert res["max_abs_err"] <= 2e-6 * max(res["scale"], 1.0), res


@pytest.mark.timeout(600)
def test_multinode_local_executor_matches_single_process(trace, tmp_path, monkeypatch):
    monkeypatch.setenv("SGA_LAUNCH_EXECUTOR", "local")
    # multi-node replays select by exact top-k (the balanced rule is single-node only): same rule on both arms
    one = _cli(trace, tmp_path, "--fused-shards", "1", "--selection-semantics", "topk")
    two = _cli(trace, tmp_path, "--fused-shards", "2", "--nodes", "nodeA,nodeB", "--launch-log-dir",
               str(tmp_path / "launch"), "--preflight-timeout", "120", "--selection-semantics", "topk")
    a = one["branch_results"]["0"]["per_ratio"]["5.0"]["scores"]
    b = two["branch_results"]["0"]["per_ratio"]["5.0"]["scores"]
    for key in a:
        assert b[key]["distortion"]["8"] == pytest.approx(a[key]["distortion"]["8"], rel=1e-6)
        assert b[key]["recall_at_k"] == a[key]["recall_at_k"]
    logs = os.listdir(tmp_path / "launch" / "logs")
    assert {"preflight_node0.log", "run_node1.log"} <= set(logs)


def test_supervisor_kills_everyone_on_first_failure(tmp_path):
    sup = launch.Supervisor(str(tmp_path), poll_s=0.05)
    t0 = time.time()
    with pytest.raises(launch.LaunchError, match="exited with code 3"):
        sup.run([[sys.executable, "-c", "import time; time.sleep(60)"],
                 [sys.executable, "-c", "import sys; print('boom'); sys.exit(3)"]], ["sleeper", "failer"])
    assert time.time() - t0 < 20
    assert all(p.poll() is not None for p, _t, _l in sup.procs), "no worker may survive"
    assert "boom" in sup.tails()


def test_supervisor_deadline_and_spawn_failure(tmp_path):
    sup = launch.Supervisor(str(tmp_path), poll_s=0.05)
    with pytest.raises(launch.LaunchError, match="deadline"):
        sup.run([[sys.executable, "-c", "import time; time.sleep(60)"]], ["sleeper"], deadline_s=0.5)
    assert sup.procs[0][0].poll() is not None
    with pytest.raises(launch.LaunchError, match="could not start"):
        sup.run([["/nonexistent/binary"]], ["ghost"])
    sup.run([[sys.executable, "-c", "pass"], [sys.executable, "-c", "pass"]], ["a", "b"])


def test_ssh_and_worker_command_rendering():
    argv = launch.render_ssh_argv("node7", "echo hi", ssh_key="/k/id", port=2222)
    assert argv == ["ssh", "-p", "2222", "-o", "BatchMode=yes", "-o", "StrictHostKeyChecking=no", "-o",
                    "ServerAliveInterval=15", "-o", "ServerAliveCountMax=4", "-i", "/k/id", "node7", "echo hi"]
    wc = launch.render_worker_cmd("/w/job.pt", 1, 2, 4, "node0", 29501, "preflight")
    assert wc[1:4] == ["-m", "sga_b200.replay.launch", "--node-worker"]
    assert wc[wc.index("--node-rank") + 1] == "1" and wc[wc.index("--phase") + 1] == "preflight"
    assert launch.render_size_probe("h", "/a b/c", executor="local") == ["bash", "-c", "stat -c %s '/a b/c'"]
    assert launch.render_size_probe("h", "/x")[-1] == "stat -c %s /x"


def test_visibility_probe_refuses_wrong_size(tmp_path):
    f = tmp_path / "job.pt"
    f.write_bytes(b"12345")
    launch.confirm_visible(["n0"], str(f), 5, None, "local")
    with pytest.raises(launch.LaunchError, match="not visible"):
        launch.confirm_visible(["n0"], str(f), 6, None, "local")
    with pytest.raises(launch.LaunchError):
        launch.confirm_visible(["n0"], str(tmp_path / "missing"), 5, None, "local")


@pytest.mark.timeout(900)
def test_multinode_smoke_script_local_executor(tmp_path):
    """The cross-node smoke script end to end with local subprocesses standing in for the two nodes."""
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run(["bash", os.path.join(root, "tests", "smoke_replay_multinode.sh"), "nodeA", "nodeB",
                          str(tmp_path / "work")], env=dict(os.environ, SGA_LAUNCH_EXECUTOR="local"),
                         capture_output=True, text=True, timeout=800)
    assert res.returncode == 0 and "SMOKE PASS" in res.stdout, (res.stdout[-1500:], res.stderr[-1500:])


def test_sweep_is_rendered_by_recorded_process_group_and_skipped_locally(tmp_path, monkeypatch):
    """The out-of-band sweep after a failed launch: one ssh per node that ends the process group the
    node worker recorded (never a pattern match), nothing at all for the local executor."""
    from sga_b200.replay import launch as L

    pf = L.worker_pid_file("/work/job_t5.pt", 2, "run")
    assert pf == "/work/job_t5.pt.run.node2.pgid"
    argv = L.render_sweep_argv("node7", pf, ssh_key="/k/id")
    assert argv[0] == "ssh" and "node7" in argv
    remote = argv[-1]
    assert "kill -TERM -- -$(cat /work/job_t5.pt.run.node2.pgid)" in remote and "pkill" not in remote
    assert remote.rstrip().endswith("true")
    ran = []
    monkeypatch.setattr(L.subprocess, "run", lambda a, **k: ran.append(a))
    L.sweep_node_workers(["a", "b"], "/work/job.pt", "run", None, "local")
    assert ran == []
    L.sweep_node_workers(["a", "b"], "/work/job.pt", "preflight", None, "ssh")
    assert len(ran) == 2 and "/work/job.pt.preflight.node1.pgid" in ran[1][-1]

