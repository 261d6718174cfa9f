"""Launcher: yaml -> flags (dual-form equivalence with the CLI), pre-validation,
torchrun command line and run-script skeleton, hostfile parsing."""
import glob
import json
import os
import sys

import pytest
import yaml

from sga_b200.launcher import backend as B
from sga_b200.launcher import utils as U
from sga_b200.launcher.launcher_ssh import JobStatus, SshLauncher, nsys_prefix, torchrun_argv
from sga_b200.launcher.run import load_config, validate_task, Runner

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_hostfile_parser(tmp_path):
    f = tmp_path / "hosts"
    f.write_text("# cluster\nnode1 slots=8 type=b200\n\nnode2 slots=4   # half\n")
    assert U.parse_hostfile(str(f)) == [{"host": "node1", "slots": 8, "type": "b200"},
                                        {"host": "node2", "slots": 4, "type": None}]
    assert U.parse_hostfile(None) == []
    f.write_text("node1 slots=8\nnode1 slots=8\n")
    with pytest.raises(ValueError, match="duplicate"):
        U.parse_hostfile(str(f))
    f.write_text("node1 gpus=8\n")
    with pytest.raises(ValueError, match="cannot parse"):
        U.parse_hostfile(str(f))
    f.write_text("node1\n")
    with pytest.raises(ValueError, match="slots"):
        U.parse_hostfile(str(f))


def test_flatten_dict_to_args():
    assert U.flatten_dict_to_args({"micro_batch_size": 4, "flag": True, "off": False, "none": None, "xs": [1, 2]}) == \
        ["--micro-batch-size", "4", "--flag", "--xs", "1", "2"]
    # nested sections flatten in place, in order, with the ignore list applied at every level
    assert U.flatten_dict_to_args({"a": 1, "logging": {"log_interval": 5, "log_dir": "x", "deep": {"b_c": True}}, "z": 2},
                                  ignore=("log_dir",)) == ["--a", "1", "--log-interval", "5", "--b-c", "--z", "2"]


def test_sga_section_to_flags_and_nulls():
    cfg = {"sga": {"sga_enabled": True, "sga_score": "abs_m", "sga_trace_branch_points": [30, 10],
                   "sga_selection_adaptive_warmup_syncs": None, "sga_trace_dir": None,
                   "sga_always_sync_layers": ["norm", "embedding"]}}
    flags = B.sga_section_to_flags(cfg)
    assert flags == ["--sga-always-sync-layers", "norm,embedding", "--sga-enabled", "true", "--sga-score", "abs_m",
                     "--sga-selection-adaptive-warmup-syncs", "null", "--sga-trace-branch-points", "30,10"]
    with pytest.raises(ValueError, match="explicitly null"):
        B.sga_section_to_flags({"sga": {"sga_enabled": None}})
    with pytest.raises(ValueError, match="full flat sga_"):
        B.sga_section_to_flags({"sga": {"score": "abs_g"}})
    with pytest.raises(ValueError, match="unknown keys"):
        B.sga_section_to_flags({"sga": {"sga_scoree": "abs_g"}})


def test_yaml_and_flag_routes_resolve_identically():
    cfg = {"sga": {"sga_enabled": True, "sga_score": "update", "sga_selection_method": "histogram",
                   "sga_selection_histogram_mode": "balanced", "sga_selection_ratio_percent": 10,
                   "sga_backend": "torch_pipelined_index", "sga_cycle_period": 8,
                   "sga_cycle_start_iter_percent": 1.0, "sga_trace_dir": "/t", "sga_trace_branch_points": [5, 1]}}
    a = B.prevalidate_sga(B.sga_section_to_flags(cfg), train_iters=2000)
    b = B.prevalidate_sga(["--sga-enabled", "true", "--sga-score", "update", "--sga-selection-method", "histogram",
                           "--sga-selection-histogram-mode", "balanced", "--sga-selection-ratio-percent", "10",
                           "--sga-backend", "torch_pipelined_index", "--sga-cycle-period", "8",
                           "--sga-cycle-start-iter-percent", "1.0", "--sga-trace-dir", "/t",
                           "--sga-trace-branch-points", "5,1"], train_iters=2000)
    assert vars(a) == vars(b)
    assert a.sga_cycle_start_iter == 20 and a.sga_trace_branch_points == [1, 5]


def test_prevalidation_fails_at_launch(tmp_path):
    cfg = load_config(os.path.join(ROOT, "examples/llama3/train_1b_adamw.yaml"),
                      [f"experiment.exp_dir={tmp_path}", "sga.sga_cycle_period=0"])
    with pytest.raises(ValueError, match="sga_cycle_period"):
        B.TrainBackend(cfg)
    cfg = load_config(os.path.join(ROOT, "examples/llama3/train_1b_adamw.yaml"),
                      [f"experiment.exp_dir={tmp_path}", "train.model.no_such_flag=1"])
    with pytest.raises(ValueError, match="trainer flags"):
        B.TrainBackend(cfg)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples/*/*.yaml"))
                                        + glob.glob(os.path.join(ROOT, "experiments/example/configs/*.yaml"))))
def test_every_shipped_config_prevalidates(path, tmp_path, monkeypatch):
    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    cfg = load_config(path, [f"experiment.exp_dir={tmp_path}"])
    validate_task(cfg)
    be = B.TrainBackend(cfg)
    assert "--model" in be.train_args


def test_golden_command_line_and_script_skeleton(tmp_path):
    cfg = load_config(os.path.join(ROOT, "examples/llama3/train_1b_rank_local.yaml"),
                      [f"experiment.exp_dir={tmp_path}", "experiment.runner.nproc_per_node=8"])
    r = Runner(cfg)
    (host, run_sh, stop_sh), = r.launcher.plan()
    text = open(run_sh).read().splitlines()
    assert text[0] == "#!/bin/bash" and text[1] == "set -o pipefail"
    assert any(l.startswith("export NCCL_DEBUG=") for l in text)
    last = text[-1]
    assert last.startswith("nohup ") and last.endswith(f"host_0_{host}.pid")
    assert "-m torch.distributed.run --nnodes 1 --nproc-per-node 8 --node-rank 0 --master-addr 127.0.0.1 " \
           "--master-port 29512 -m sga_b200.train_gpt" in last
    assert "--sga-enabled true" in last and "--sga-selection-locality rank_local" in last
    assert "--global-batch-size 256" in last and f"--save {tmp_path}/checkpoints" in last
    assert f"--tensorboard-dir {tmp_path}/tensorboard" in last
    stop = open(stop_sh).read()
    assert "kill" in stop and f"host_0_{host}.pid" in stop
    assert r.launcher.query_once() == JobStatus.COMPLETED_OR_IDLE
    said = []
    assert r.launcher.query(interval=0.01, timeout=0.05, out=said.append) == JobStatus.COMPLETED_OR_IDLE
    assert said[0] == "Job status: COMPLETED_OR_IDLE" and said[-1].startswith("Query timeout reached")
    assert r.launcher.run(dryrun=True, tail=False) == [0]


def test_torchrun_and_nsys_argv():
    a = torchrun_argv({"rdzv_backend": "static"}, 2, 1, 8, "node0", 29500)
    assert a[1:] == ["-m", "torch.distributed.run", "--nnodes", "2", "--nproc-per-node", "8", "--node-rank", "1",
                     "--master-addr", "node0", "--master-port", "29500"]
    b = torchrun_argv({"rdzv_backend": "c10d", "rdzv_id": "job7"}, 2, 1, 8, "node0", 29500)
    assert "--rdzv-endpoint" in b and "node0:29500" in b and "--node-rank" not in b
    assert nsys_prefix({}, 0) == []
    n = nsys_prefix({"nsys_bin_path": "/opt/nsys", "nsys_rep_file_path": "/tmp/rep"}, 3)
    assert n[:2] == ["/opt/nsys", "profile"] and "--capture-range=cudaProfilerApi" in n and "/tmp/rep_node3" in n


def test_multi_node_plan_and_node_overrides(tmp_path):
    hf = tmp_path / "hosts"
    hf.write_text("nodeA slots=8 type=b200\nnodeB slots=8 type=b200\n")
    cfg = load_config(os.path.join(ROOT, "examples/llama3/train_1b_dense.yaml"),
                      [f"experiment.exp_dir={tmp_path}", f"experiment.runner.hostfile={hf}",
                       "experiment.runner.nnodes=2"])
    cfg["experiment"]["node_envs"] = {"nodeB": {"NCCL_DEBUG": "INFO"}, "b200": {"EXTRA": "1"}}
    L = Runner(cfg).launcher
    plan = L.plan()
    assert [p[0] for p in plan] == ["nodeA", "nodeB"] and L.master_addr == "nodeA"
    a, b = open(plan[0][1]).read(), open(plan[1][1]).read()
    assert "--node-rank 0" in a and "--node-rank 1" in b and "--nnodes 2" in b
    assert "export NCCL_DEBUG=INFO" in b and "export NCCL_DEBUG=WARN" in a and "export EXTRA=1" in a
    assert U.ssh_argv("nodeB", "bash x.sh", 2222, background=True)[:5] == ["ssh", "-f", "-n", "-p", "2222"]


def test_select_best(tmp_path):
    import importlib.util

    spec = importlib.util.spec_from_file_location("select_best", os.path.join(ROOT, "experiments/example/select_best.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rep = {"branch_results": {"8": {"horizon_steps": [8, 16], "per_ratio": {
        "10.0": {"k": 1, "scores": {"abs_g@T4": {"distortion": {"8": 0.5, "16": 0.4}},
                                    "update@T8@fold": {"distortion": {"8": 0.1, "16": 0.3}}}}}},
        "9": {"state_absent": True}}}
    assert mod.best_arm(rep)[:3] == (0.3, "update@T8@fold", 10.0)
    assert mod.overrides_for("update@T8@fold@dl0.5", 10.0) == {
        "sga_score": "update", "sga_selection_ratio_percent": 10.0, "sga_cycle_period": 8,
        "sga_optimizer_residual_mean": True, "sga_optimizer_full_sync_inactive_lr_scale": 0.5}


def test_env_and_setup_scripts_check_the_checkout():
    """``env.sh --check`` accepts the checkout it lives in and refuses a shadowing copy of the package;
    ``setup.sh`` reports against ``manifest.yaml`` (reference counterparts: ``env.sh:1-137``, ``setup.sh:1-70``)."""
    import os
    import subprocess
    import tempfile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ok = subprocess.run(["bash", "-c", f"source {root}/env.sh --check"], capture_output=True, text=True,
                        env={k: v for k, v in os.environ.items() if k != "PYTHONPATH"})
    assert ok.returncode == 0 and "env.sh: ok" in ok.stdout, ok.stdout + ok.stderr
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "sga_b200"))
        open(os.path.join(d, "sga_b200", "__init__.py"), "w").close()
        # python puts the working directory first on its path: a stray copy there shadows the checkout
        bad = subprocess.run(["bash", "-c", f"cd {d} && export PYTHONPATH={d} && source {root}/env.sh --check"],
                             capture_output=True, text=True)
        assert bad.returncode != 0 and "resolves to" in bad.stderr, bad.stdout + bad.stderr


def test_yaml_in_the_reference_vocabulary_launches(tmp_path):
    """A yaml written for the reference (its training stack's flag names: nested precision / logging /
    checkpoint / optimizer / lr_scheduler / tokenizer sections, architecture by flags) goes through the
    launcher unchanged, and the flags it produces train."""
    import torch

    from sga_b200.runtime.trainer import Trainer, build_parser

    (tmp_path / "ref_style.yaml").write_text(f"""
experiment:
  exp_name: ref-style
  exp_dir: {tmp_path}/exp
  task: {{type: train, backend: megatron, entrypoint: ./sga/train_gpt.py}}
  runner: {{type: ssh, nproc_per_node: 1}}
sga:
  sga_enabled: true
  sga_score: abs_m
  sga_selection_method: histogram
  sga_selection_histogram_mode: balanced
  sga_selection_ratio_percent: 10
  sga_cycle_period: 4
  sga_backend: torch_pipelined_index
train:
  system:
    rerun_mode: disabled
    tensor_model_parallel_size: 1
    pipeline_model_parallel_size: 1
    disable_bias_linear: true
    use_flash_attn: true
    use_distributed_optimizer: false
    data_parallel_sharding_strategy: no_shard
    precision: {{bf16: true, attention_softmax_in_fp32: true, accumulate_allreduce_grads_in_fp32: true}}
    logging: {{timing_log_level: 2, log_interval: 1, log_throughput: true, log_num_zeros_in_grad: true}}
    checkpoint: {{save_interval: 100000}}
  model:
    transformer_impl: transformer_engine
    num_layers: 1
    hidden_size: 64
    ffn_hidden_size: 128
    num_attention_heads: 4
    seq_length: 32
    group_query_attention: true
    num_query_groups: 2
    max_position_embeddings: 32
    norm_epsilon: 1e-5
    swiglu: true
    normalization: RMSNorm
    position_embedding_type: rope
    rotary_base: 500000
    untie_embeddings_and_output_weights: true
    attention_dropout: 0.0
    hidden_dropout: 0.0
    clip_grad: 1.0
    train_iters: 20
    exit_interval: 10
    eval_iters: 0
    eval_interval: 1000
    micro_batch_size: 1
    global_batch_size: 2
    seed: 1234
    optimizer:
      weight_decay: 1e-2
      adam_beta1: 0.9
      adam_beta2: 0.95
      lr_scheduler: {{lr: 1.0e-3, min_lr: 1.0e-4, lr_warmup_fraction: 0.1, lr_decay_style: cosine}}
  data:
    split: 1
    tokenizer: {{tokenizer_type: HuggingFaceTokenizer, tokenizer_model: /nowhere, padded_vocab_size: 320,
                make_vocab_size_divisible_by: 64}}
""")
    cfg = load_config(str(tmp_path / "ref_style.yaml"), [])
    validate_task(cfg)
    be = B.TrainBackend(cfg)
    flags = be.train_args
    for tok in ("--hidden-size", "--lr-warmup-fraction", "--lr-decay-style", "--padded-vocab-size", "--bf16",
                "--sga-cycle-period", "--exit-interval"):
        assert tok in flags, tok
    assert "--use-distributed-optimizer" not in flags, "a false switch is not emitted"
    args = build_parser().parse_args(flags + ["--device", "cpu", "--model", "test_tiny"])
    tr = Trainer(args, quiet=True)
    assert (tr.cfg.hidden, tr.cfg.n_heads, tr.cfg.n_kv_heads, tr.cfg.vocab, tr.cfg.seq_len) == (64, 4, 2, 320, 32)
    assert not tr.cfg.tied_embeddings
    for s in range(3):
        assert torch.isfinite(tr.train_step(tr.host_batch(s)))
    assert tr.optimizer.param_groups[0]["lr"] == pytest.approx(1e-3)  # warm-up of 2 steps is over
    tr.close()
    bad = build_parser().parse_args(flags + ["--device", "cpu", "--model", "test_tiny", "--normalization", "LayerNorm"])
    with pytest.raises(ValueError, match="RMSNorm only"):
        Trainer(bad, quiet=True)


def test_audit_tool(tmp_path, capsys):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import audit_trainer_args as audit

    out = str(tmp_path / "flags.json")
    assert audit.main(["check", os.path.join(ROOT, "examples/llama3/train_1b_adamw.yaml"), out]) == 0
    table = json.load(open(out))
    assert table["--lr-decay-style"]["choices"] == ["constant", "linear", "cosine"]
    assert table["--swiglu"]["group"] == "accepted for yaml compatibility"
    (tmp_path / "bad.yaml").write_text("experiment: {exp_name: x, exp_dir: /tmp/x, task: {type: train}}\n"
                                       "train: {model: {no_such_flag: 1}}\n")
    assert audit.main(["check", str(tmp_path / "bad.yaml")]) == 1
    text = capsys.readouterr().out
    assert "REFUSED" in text and "--no-such-flag" in text


def test_find_latest_stdout_log_and_tailer_follow_new_attempts(tmp_path):
    import time

    from sga_b200.launcher.utils import LogTailer, find_latest_stdout_log

    assert find_latest_stdout_log(str(tmp_path / "missing")) is None
    assert find_latest_stdout_log(str(tmp_path)) is None
    base = tmp_path / "host_0_a"
    for run, attempt, rank in (("2024_01", 0, 0), ("2024_02", 0, 0), ("2024_02", 1, 0), ("2024_02", 1, 3)):
        d = base / run / "rid" / f"attempt_{attempt}" / str(rank)
        d.mkdir(parents=True, exist_ok=True)
        (d / "stdout.log").write_text(f"{run} {attempt} {rank}\n")
    (base / "2024_02" / "rid" / "attempt_1" / "7").mkdir()  # a rank directory without a log yet
    want = str(base / "2024_02" / "rid" / "attempt_1" / "3" / "stdout.log")
    assert find_latest_stdout_log(str(tmp_path)) == want
    got = []
    t = LogTailer(lambda: find_latest_stdout_log(str(tmp_path)), poll_s=0.02, out=got.append).start()
    time.sleep(0.2)
    d = base / "2024_03" / "rid" / "attempt_0" / "0"
    d.mkdir(parents=True)
    (d / "stdout.log").write_text("fresh attempt\n")
    time.sleep(0.3)
    t.stop()
    assert got[0] == "2024_02 1 3" and got[-1] == "fresh attempt"

