"""Device side of the replay's boundary reselection (``csrc/replay_select.cu``) against the PyTorch
forms it replaces: the fp64 registry score stored as fp32, bit for bit, and the exact top-k with
index-ordered ties."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _group(n, R, scores, ks_ratio=5.0, optimizer="adamw"):
    from sga_b200.replay import core as RC
    from sga_b200.replay import fused as RF

    torch.manual_seed(n + R)
    cfgs = [RC.CycleConfig(score=s, ratio_percent=ks_ratio, cycle_len=4, optimizer=optimizer) for s in scores]
    hp = RC.Hyper(wd=None, beta1=0.9, beta2=0.95, eps=1e-8, clip=1.0)
    wd = torch.where(torch.rand(n) < 0.8, torch.tensor(0.1), torch.tensor(0.0))
    w0, m0 = torch.randn(n) * 0.02, torch.randn(n) * 1e-4
    v0 = torch.rand(n) * 1e-7
    g = RF.FusedGroup(cfgs[:R], n, n, DEV, RF.Comms(0, 1, None, DEV), hp, wd, w0, m0, v0, 3, 12, [12], {}, True)
    g.RES.copy_(torch.randn(R, n) * 1e-3)
    g.SEL.copy_((torch.rand(R, n) < 0.1).to(torch.uint8))
    return g, RC, RF


@pytest.mark.parametrize("optimizer", ["adamw", "adams"])
@pytest.mark.parametrize("g_dtype", [torch.float32, torch.bfloat16])
def test_score_kernel_equals_registry_score_bitwise(optimizer, g_dtype):
    from sga_b200 import kernels  # noqa: F401  (declares the launchers' argument types)
    from sga_b200.csrc import lib
    from sga_b200.plugins.scores import EMIT_CODES

    n, scores = 100003, ["abs_g", "abs_m", "update", "coi"]
    grp, RC, RF = _group(n, 4, scores, optimizer=optimizer)
    graw = (torch.randn(n, device=DEV) * 1e-3).to(g_dtype)
    count, coef_dense = 9, RC.f32(0.731)
    for boundary, fold in ((True, False), (True, True), (False, False)):
        plan = grp._plan(4 if boundary else 5, count, 3e-4)
        for p in plan:
            p["fold"] = bool(fold and boundary)
            p["coef"] = RC.f32(0.5531)
        grp._upload(plan)
        g32 = RC._div(graw.float(), coef_dense)
        for r, name in enumerate(scores):
            out = torch.empty(n, device=DEV)
            rc = lib().sga_replay_score(graw.data_ptr(), int(g_dtype == torch.bfloat16), coef_dense, grp.W[r].data_ptr(),
                                        grp.M[r].data_ptr(), grp.V[r].data_ptr(), grp.RES[r].data_ptr(),
                                        grp.SEL[r].data_ptr(), grp.wd.data_ptr(),
                                        grp._cfg_dev.data_ptr() + r * ctypes.sizeof(RF._CfgStruct), EMIT_CODES[name],
                                        0.9, 0.95, 1e-8, float(plan[r]["bc1"]), float(plan[r]["bc2"]), n,
                                        out.data_ptr(), torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            q = grp._q_pre(plan[r], g32, r) * plan[r]["coef"]
            ref = RC.replay_score(name, grp.W[r], grp.M[r], grp.V[r], q, grp._hp_dev(), count, optimizer)
            assert torch.equal(out, ref), f"{name} boundary={boundary} fold={fold}"


def test_device_topk_equals_flat_select_with_ties():
    n = 300007
    grp, RC, _RF = _group(n, 3, ["abs_g", "abs_g", "abs_g"])
    torch.manual_seed(5)
    a = torch.randn(n, device=DEV)
    b = torch.randn(n, device=DEV) * 1e-4
    b[::37] = -0.25                      # a tie layer at the top: the cut falls inside it
    c = torch.zeros(n, device=DEV)       # everything ties
    c[1000:1100] = 1.0
    ks = [n // 20, 5000, 250]
    masks = grp._device_topk([a, b, c], ks)
    for x, k, m in zip((a, b, c), ks, masks):
        ref = RC.select_topk_flat(x, k)
        assert int(m.sum()) == k
        assert torch.equal(m.bool(), ref.bool())
