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
