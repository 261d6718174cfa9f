"""The reference-vs-ours sync + optimizer benchmark runs end to end on one GPU at a small
geometry and both arms follow the same full / sparse calendar."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.timeout(600)
def test_both_arms_small_geometry():
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "sga")):
        pytest.skip("no copy of the reference package under baseline/_ref")
    out = {}
    for impl in ("reference", "ours"):
        res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "ref_sync_bench.py"), "--impl", impl,
                              "--elems", "6291456", "--bucket", "2097152", "--param", "524288", "--steps", "8",
                              "--warmup", "5"], capture_output=True, text=True, timeout=500,
                             env=dict(os.environ, MASTER_PORT="29537"))
        assert res.returncode == 0, res.stderr[-3000:]
        line = [ln for ln in res.stdout.splitlines() if ln.startswith('{"impl"')][-1]
        out[impl] = json.loads(line)
        assert "unavailable" not in out[impl], out[impl]
    assert out["reference"]["phases"] == out["ours"]["phases"]
    assert out["ours"]["phases"].count("full") == 2
    for impl in out:
        assert out[impl]["ms_per_step_cycle"] > 0


@pytest.mark.timeout(600)
def test_check_mode_same_weights_same_result():
    """Both arms from the same weights, clip off (its coefficient is the one quantity whose last bits
    differ between the arms): weights equal to fp32 rounding, residual buffers bit-identical, ending on
    a sparse step so that the residual holds a whole cycle's unselected mass."""
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "sga")):
        pytest.skip("no copy of the reference package under baseline/_ref")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "ref_sync_bench.py"), "--impl", "both", "--check",
                          "--clip", "0", "--elems", "6291456", "--bucket", "2097152", "--param", "524288", "--steps",
                          "9", "--warmup", "2"], capture_output=True, text=True, timeout=500,
                         env=dict(os.environ, MASTER_PORT="29538"))
    assert res.returncode == 0, res.stderr[-3000:]
    chk = json.loads([ln for ln in res.stdout.splitlines() if ln.startswith('{"check"')][-1])
    assert chk["residual_lanes_differing"] == 0 and chk["weight_lanes_off_by_1e-6"] == 0, chk
    assert chk["max_abs_dw"] < 1e-6 < chk["max_weight_movement"], chk
