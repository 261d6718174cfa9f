"""Multi-GPU tests: launches the workers under torchrun on the GPUs of this box: 2 ranks by
default, ``SGA_TEST_RANKS`` of them (2, 4 or 8) when set and that many GPUs are visible. NVLS is
switched off in NCCL for these child processes and the framework's own kernels use plain peer
loads and stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
RANKS = int(os.environ.get("SGA_TEST_RANKS", "2"))


def _run(nproc, timeout=600, worker="dist_gpu_worker.py", port=29741):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, worker)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.timeout(900)
def test_peer_kernels_and_trainer_multi_gpu():
    if torch.cuda.device_count() < RANKS:
        pytest.skip(f"needs at least {RANKS} GPUs")
    res = _run(RANKS)
    assert res.returncode == 0 and "DIST_GPU_OK" in res.stdout, res.stdout[-3000:] + "\n" + res.stderr[-6000:]


@pytest.mark.timeout(900)
def test_tensor_parallel_fused_kernels_and_model_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    res = _run(2, worker="tp_gpu_worker.py", port=29743)
    assert res.returncode == 0 and "TP_GPU_OK" in res.stdout, res.stdout[-3000:] + "\n" + res.stderr[-6000:]


@pytest.mark.timeout(900)
def test_pipeline_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    res = _run(2, worker="pp_gpu_worker.py", port=29745)
    assert res.returncode == 0 and "PP_GPU_OK" in res.stdout, res.stdout[-3000:] + "\n" + res.stderr[-6000:]


@pytest.mark.timeout(900)
def test_fused_replay_two_shards_on_gpus(tmp_path):
    """Two replay shards on two GPUs (NCCL collectives between the device-side selection passes)
    against one shard: discrete quantities exact, sums inside the reordering band."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    from sga_b200.replay import core as RC
    from sga_b200.replay import fused as RF
    from sga_b200.replay.synth import make_synthetic_trace

    trace = make_synthetic_trace(str(tmp_path / "trace"), sizes=(400000, 300000, 170000), steps=12, g_dtype="bf16",
                                 seed=3)
    cfgs = [RC.CycleConfig(score=s, ratio_percent=r, cycle_len=t) for s in ("abs_g", "update") for r in (1.0, 5.0)
            for t in (1, 4)]
    kw = dict(score_names=["abs_g", "update"], ratios=[1.0, 5.0], semantics="topk")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    one = RF.run_fused_branch(trace, 0, cfgs, 12, [6, 12], world=1, device="cuda", **kw)
    two = RF.run_fused_branch(trace, 0, cfgs, 12, [6, 12], world=2, device="cuda", **kw)
    for c in cfgs:
        for h in (6, 12):
            assert two["results"][c][h] == pytest.approx(one["results"][c][h], rel=1e-6), (c, h)
    for key, m in one["front"].items():
        assert two["front"][key]["recall_at_k"] == m["recall_at_k"]

