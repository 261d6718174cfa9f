"""Offline replay: exact selection, the from-spec cycle oracle, the fused
engine (one shard bit-exact against the oracle, two gloo shards inside the
pure-reordering band), cache identity, CLI report."""
import json
import math
import os

import pytest
import torch

from sga_b200.replay import core as RC
from sga_b200.replay import fused as RF
from sga_b200.replay.synth import make_synthetic_trace

SIZES = (4000, 3000, 1700)   # parameters straddle the shard boundaries


@pytest.fixture(scope="module")
def trace(tmp_path_factory):
    d = tmp_path_factory.mktemp("trace")
    return make_synthetic_trace(str(d), sizes=SIZES, steps=12, g_dtype="fp32", seed=3)


def _inputs(trace):
    info = RC.discover_trace(trace)
    meta, payload = RC.load_state(info, 0)
    w0, m0, v0, g0 = (RC.flatten(payload[k], info) for k in ("w", "m", "v", "g"))
    steps = info.window(0, 12)
    logged, norms, lrs = [], [], []
    for t in steps:
        gm, gp = RC.load_g(info, t)
        logged.append(RC.flatten(gp, info))
        norms.append(gm["grad_norm"])
        lrs.append(gm["lr"][0])
    wd = RC.group_vector(info, [g["weight_decay"] for g in meta["param_groups"]])
    hp = RC.Hyper(wd=wd, beta1=0.9, beta2=0.95, eps=1e-8, clip=meta["clip_grad"])
    return info, w0, m0, v0, g0, logged, norms, lrs, hp


def test_discover_and_flatten(trace):
    info = RC.discover_trace(trace)
    assert info.numel == sum(SIZES) and info.branch_points == [0] and info.g_steps == list(range(12))
    assert info.window(0, 100) == list(range(12)) and info.window(5, 3) == [5, 6, 7]
    _, p = RC.load_g(info, 3)
    full = RC.flatten(p, info)
    assert torch.equal(RC.flatten(p, info, lo=3990, hi=7010), full[3990:7010])
    os.rename(os.path.join(trace, "step_000007_g.pt"), os.path.join(trace, "hidden.pt"))
    try:
        assert RC.discover_trace(trace).window(0, 100) == list(range(7)), "a gap ends the window"
    finally:
        os.rename(os.path.join(trace, "hidden.pt"), os.path.join(trace, "step_000007_g.pt"))


def test_select_topk_flat_exact_with_index_ordered_ties():
    x = torch.tensor([0.5, -2.0, 0.5, 3.0, 0.5, -0.5, 0.1])
    assert RC.select_topk_flat(x, 3).tolist() == [True, True, False, True, False, False, False]
    assert int(RC.select_topk_flat(x, 5).sum()) == 5
    g = torch.Generator().manual_seed(0)
    y = torch.randint(-4, 5, (5000,), generator=g).float()
    for k in (1, 77, 2500, 5000):
        assert int(RC.select_topk_flat(y, k).sum()) == k


def test_shard_select_equals_flat_select():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(30000, generator=g)
    x[::17] = 1.25
    for k in (1, 300, 1764, 1765, 9000):
        assert torch.equal(RF.shard_select(x, k, RF.Comms()), RC.select_topk_flat(x, k))


def test_ranking_metrics_sanity():
    g = torch.Generator().manual_seed(2)
    lab = torch.rand(2000, generator=g)
    perfect = RC.ranking_metrics(lab.clone(), lab, 200)
    assert perfect["recall_at_k"] == 1.0 and abs(perfect["ndcg_at_k"] - 1.0) < 1e-12
    noise = RC.ranking_metrics(torch.rand(2000, generator=g), lab, 200)
    assert noise["recall_at_k"] < 0.3 and noise["ndcg_at_k"] < perfect["ndcg_at_k"]
    assert 0.0 < perfect["missed_label_mass"] < 1.0


def test_boundary_reselect_is_load_bearing(trace):
    info, w0, m0, v0, g0, logged, norms, lrs, hp = _inputs(trace)
    cfg = RC.CycleConfig("abs_g", 5.0, 4)
    a, _ = RC.reference_cycle(w0, m0, v0, logged, norms, lrs, hp, 0, cfg, g0, horizons={12})
    b, _ = RC.reference_cycle(w0, m0, v0, logged, norms, lrs, hp, 0, cfg, g0, horizons={12}, reselect=False)
    assert not torch.equal(a[12], b[12])


CONFIGS = [RC.CycleConfig(s, r, T, o, f, d) for (s, r, T, o, f, d) in [
    ("abs_g", 1.0, 1, "adamw", False, 1.0), ("abs_g", 5.0, 4, "adamw", False, 1.0),
    ("update", 5.0, 4, "adamw", True, 1.0), ("abs_m", 10.0, 3, "adamw", False, 0.5),
    ("coi", 5.0, 16, "adamw", False, 1.0), ("abs_g", 5.0, 4, "adams", False, 1.0)]]


def test_fused_one_shard_equals_per_config_oracle_bitwise(trace):
    info, w0, m0, v0, g0, logged, norms, lrs, hp = _inputs(trace)
    horizons = [6, 12]
    for opt in ("adamw", "adams"):
        cfgs = [c for c in CONFIGS if c.optimizer == opt]
        frag = RF.run_fused_branch(trace, 0, cfgs, 12, horizons, world=1, device="cpu", score_names=["abs_g"],
                                   ratios=[5.0], keep_state=True)
        Wf, Sf = frag["final_state"]
        dense = RC.dense_replay(w0, m0, v0, logged, lrs, hp, 0, opt, set(horizons))
        for r, c in enumerate(cfgs):
            snaps, _ = RC.reference_cycle(w0, m0, v0, logged, norms, lrs, hp, 0, c, g0, horizons=set(horizons))
            assert torch.equal(Wf[r], snaps[12]), f"{c}: weights differ from the per-configuration replay"
            for h in horizons:
                want = RC.distortion(snaps[h], dense[h], w0)
                assert frag["results"][c][h] == pytest.approx(want, rel=1e-12)
        assert frag["window_len"] == 12 and frag["horizon_steps"] == horizons
    m = frag["front"][("abs_g", 5.0, opt)]
    assert m["k"] == RC.k_for(sum(SIZES), 5.0) and 0.0 <= m["recall_at_k"] <= 1.0


@pytest.mark.timeout(600)
def test_fused_two_shards_stay_in_the_reordering_band(trace):
    cfgs = [c for c in CONFIGS if c.optimizer == "adamw"]
    one = RF.run_fused_branch(trace, 0, cfgs, 12, [6, 12], world=1, device="cpu", score_names=["abs_g", "update"],
                              ratios=[5.0])
    two = RF.run_fused_branch(trace, 0, cfgs, 12, [6, 12], world=2, device="cpu", score_names=["abs_g", "update"],
                              ratios=[5.0])
    for c in cfgs:
        for h in (6, 12):
            assert two["results"][c][h] == pytest.approx(one["results"][c][h], rel=1e-6)
    for key, m in one["front"].items():
        assert two["front"][key]["k"] == m["k"]
        assert two["front"][key]["recall_at_k"] == m["recall_at_k"], "discrete quantities are exact"
        assert two["front"][key]["ndcg_at_k"] == pytest.approx(m["ndcg_at_k"], rel=1e-6)


def test_grouping_and_kill_switches(trace, monkeypatch):
    mk = lambda n, opt="adamw": [RC.CycleConfig("abs_g", float(i + 1), 4, opt) for i in range(n)]  # noqa: E731
    assert [len(g) for g in RF.group_configs(mk(10), 4, 0, 1000)] == [4, 4, 2]
    assert [len(g) for g in RF.group_configs(mk(5), 12, 17 * 2 * 1e6 / (1 << 20), 1000000)] == [2, 2, 1]
    mixed = RF.group_configs(mk(3) + mk(3, "adams"), 12, 0, 1000)
    assert [len(g) for g in mixed] == [3, 3] and all(len({c.optimizer for c in g}) == 1 for g in mixed)
    a = RF.run_fused_branch(trace, 0, CONFIGS[:3], 12, [12], max_configs=1)
    b = RF.run_fused_branch(trace, 0, CONFIGS[:3], 12, [12], max_configs=12)
    assert all(a["results"][c][12] == b["results"][c][12] for c in CONFIGS[:3]), "grouping must not change results"
    monkeypatch.setenv("REPLAY_FUSED_KERNEL", "maybe")
    with pytest.raises(ValueError, match="REPLAY_FUSED_KERNEL"):
        RF._switch(RF.ENV_KERNEL, ("on", "off"), "on")


def test_prefetch_failure_is_latched(trace, monkeypatch):
    info = RC.discover_trace(trace)

    class Boom(RF.GPrefetcher):
        def _load(self, t):
            if t == 2:
                raise OSError("pread failed")
            return super()._load(t)

    pf = Boom(info, [0, 1, 2, 3], 0, info.numel, torch.float32, pin=False)
    pf.get()
    pf.get()
    with pytest.raises(RuntimeError, match="prefetch failed"):
        pf.get()


def test_dense_cache_identity(tmp_path):
    ident = RC.cache_ident("/x", 0, 8, [8], "fp32", "bf16", "fused-1-0", "adamw")
    assert RC.load_cache(str(tmp_path), ident) is None
    path = RC.save_cache(str(tmp_path), ident, {"snap_d": {8: torch.ones(3)}})
    assert os.path.basename(path).startswith("dense_") and RC.load_cache(str(tmp_path), ident)["snap_d"][8].sum() == 3
    other = dict(ident, window=9)
    assert RC.load_cache(str(tmp_path), other) is None
    blob = torch.load(path, weights_only=False)
    blob["ident"] = other
    torch.save(blob, path)
    with pytest.raises(ValueError, match="ident mismatch"):
        RC.load_cache(str(tmp_path), ident)


@pytest.mark.gpu
def test_fused_gpu_kernels_match_per_config_and_cpu(trace):
    cfgs = [c for c in CONFIGS if c.optimizer == "adamw"]
    fused = RF.run_fused_branch(trace, 0, cfgs, 12, [6, 12], device="cuda:0", keep_state=True)
    cpu = RF.run_fused_branch(trace, 0, cfgs, 12, [6, 12], device="cpu")
    Wf = fused["final_state"][0]
    for r, c in enumerate(cfgs):
        single = RF.run_fused_branch(trace, 0, [c], 12, [6, 12], device="cuda:0", keep_state=True)
        assert torch.equal(single["final_state"][0][0], Wf[r]), "R configs at once == one at a time, bit for bit"
        for h in (6, 12):
            assert fused["results"][c][h] == pytest.approx(cpu["results"][c][h], rel=1e-4, abs=1e-6)


@pytest.mark.gpu
def test_fused_gpu_front_block_on_a_bare_cuda_device_with_and_without_the_rank_lane(trace, monkeypatch):
    """device="cuda" carries no index: the ranking worker thread has to be given the creator's device
    by number. Both arms of the background switch give the same front block as the CPU run."""
    cfgs = CONFIGS[:2]
    kw = dict(score_names=["abs_g", "update"], ratios=[5.0])
    cpu = RF.run_fused_branch(trace, 0, cfgs, 12, [12], device="cpu", **kw)
    got = {}
    for arm in ("on", "off"):
        monkeypatch.setenv(RF.ENV_FRONT_RANK_BG, arm)
        got[arm] = RF.run_fused_branch(trace, 0, cfgs, 12, [12], device="cuda", **kw)
        assert got[arm]["profile"][0]["arms"]["front_rank_bg"] == arm
    assert got["on"]["front"] == got["off"]["front"] and got["on"]["results"] == got["off"]["results"]
    for key, m in cpu["front"].items():   # device and host arithmetic may differ in the last bit of a score
        assert got["on"]["front"][key]["recall_at_k"] == pytest.approx(m["recall_at_k"], abs=3.0 / m["k"])
        assert got["on"]["front"][key]["ndcg_at_k"] == pytest.approx(m["ndcg_at_k"], rel=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("g_dtype", [torch.float32, torch.bfloat16])
def test_replay_vector_kernels_equal_scalar_kernels(g_dtype):
    """The four-elements-per-thread kernels (row length a multiple of 4) against the scalar ones (any
    row length) on the common prefix of the same data: state bit for bit, fp64 sums to rounding."""
    import ctypes

    from sga_b200.csrc import lib
    from sga_b200.replay.fused import _CfgStruct

    L, dev, R, n = lib(), "cuda", 7, 4096 * 5
    gen = torch.Generator().manual_seed(4)
    base = {k: torch.randn(R, n + 3, generator=gen) * 1e-3 for k in ("W", "M", "V", "RES")}
    base["V"].abs_()
    sel = (torch.rand(R, n + 3, generator=gen) < 0.1).to(torch.uint8)
    g = (torch.randn(n + 3, generator=gen) * 1e-3).to(g_dtype)
    wd = torch.rand(n + 3, generator=gen) * 0.1
    wden = torch.randn(n + 3, generator=gen) * 1e-3
    arr = (_CfgStruct * R)()
    for r in range(R):
        a = arr[r]
        a.boundary, a.fold, a.dual, a.adams, a.horizon = int(r % 3 == 0), int(r % 2 == 0), int(r == 3), int(r == 5), int(r != 1)
        a.fold_div, a.coef, a.lr, a.lr_inactive, a.bc1, a.bc2 = 4.0, 0.9 - 0.05 * r, 3e-4, 1e-4, 0.5, 0.4
    cfg = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev)
    nb = L.sga_replay_blocks()
    st = torch.cuda.current_stream().cuda_stream
    outs = {}
    for rows in (n, n + 3):  # vector path, scalar path
        t = {k: v[:, :rows].contiguous().to(dev) for k, v in base.items()}
        s_, g_, wd_, wden_ = sel[:, :rows].contiguous().to(dev), g[:rows].contiguous().to(dev), \
            wd[:rows].contiguous().to(dev), wden[:rows].contiguous().to(dev)
        part = torch.zeros(R * nb, dtype=torch.float64, device=dev)
        o1, o3 = torch.zeros(R, dtype=torch.float64, device=dev), torch.zeros(R, dtype=torch.float64, device=dev)
        assert L.sga_replay_pass1(g_.data_ptr(), int(g_dtype == torch.bfloat16), 1.25, t["RES"].data_ptr(), s_.data_ptr(),
                                  cfg.data_ptr(), R, rows, part.data_ptr(), o1.data_ptr(), st) == 0
        assert L.sga_replay_pass3(g_.data_ptr(), int(g_dtype == torch.bfloat16), 1.25, t["W"].data_ptr(),
                                  t["M"].data_ptr(), t["V"].data_ptr(), t["RES"].data_ptr(), s_.data_ptr(),
                                  wd_.data_ptr(), wden_.data_ptr(), cfg.data_ptr(), R, rows, 0.9, 0.1, 0.95, 0.05, 1e-8,
                                  part.data_ptr(), o3.data_ptr(), st) == 0
        torch.cuda.synchronize()
        outs[rows] = (t, o1.cpu(), o3.cpu())
    (tv, v1, v3), (ts, s1, s3) = outs[n], outs[n + 3]
    for k in ("W", "M", "V", "RES"):
        assert torch.equal(tv[k], ts[k][:, :n]), k
    # the scalar run covers three more elements per row: remove their share from its sums on the host
    tail = slice(n, n + 3)
    gq = g.float() / torch.tensor(1.25)
    for r in range(R):
        res = base["RES"][r, tail] / torch.tensor(4.0) if (arr[r].boundary and arr[r].fold) else base["RES"][r, tail]
        q = gq[tail] + res if arr[r].boundary else torch.where(sel[r, tail] > 0, gq[tail], torch.zeros(3))
        assert float(s1[r] - (q.double() ** 2).sum()) == pytest.approx(float(v1[r]), rel=1e-12)
        extra = ((ts["W"][r, tail].cpu().double() - wden[tail].double()) ** 2).sum() if arr[r].horizon else 0.0
        assert float(s3[r] - extra) == pytest.approx(float(v3[r]), rel=1e-12, abs=1e-300)


def test_cli_matches_reference_golden_values(tmp_path):
    """Golden values: the reference's own ``python -m sga.replay`` (its torch-eager arm) on this exact
    synthetic trace (``make_synthetic_trace(sizes=(40000, 30000, 17000), steps=6)``, seed 0), for both
    selection semantics. Distortions and the ranking metrics must agree to the printed digits; the
    default semantics of single-node cycle replay is balanced-histogram, as in ``sga/replay.py:1703``."""
    import json

    from sga_b200.replay import cli
    from sga_b200.replay.synth import make_synthetic_trace

    trace = make_synthetic_trace(str(tmp_path / "t"), sizes=(40000, 30000, 17000), steps=6)
    golden = {
        "balanced-histogram": {("1.0", "abs_g@T4"): 0.50748199, ("1.0", "abs_m@T4"): 0.50587264,
                               ("5.0", "abs_g@T4"): 0.49913694, ("5.0", "abs_m@T4"): 0.49359006},
        "topk": {("1.0", "abs_g@T4"): 0.50759871, ("1.0", "abs_m@T4"): 0.5056148,
                 ("5.0", "abs_g@T4"): 0.49945374, ("5.0", "abs_m@T4"): 0.49333816},
    }
    ndcg = {("1.0", "abs_g"): 0.56205288, ("1.0", "abs_m"): 0.15672116, ("5.0", "abs_g"): 0.49448113,
            ("5.0", "abs_m"): 0.22009503}
    recall = {("1.0", "abs_g"): 0.02414, ("5.0", "abs_g"): 0.24069, ("1.0", "abs_m"): 0.00805,
              ("5.0", "abs_m"): 0.04782}
    for sem, want in golden.items():
        out = str(tmp_path / f"{sem}.json")
        argv = ["--trace-dir", trace, "--branch-point", "0", "--ratios", "1,5", "--replay-mode", "cycle",
                "--cycle-lens", "1,4", "--score-names", "abs_g,abs_m", "--window", "6", "--device", "cpu", "--out", out]
        if sem == "topk":  # balanced-histogram is the default and must not need the flag
            argv += ["--selection-semantics", "topk"]
        assert cli.main(argv) == 0
        per_ratio = json.load(open(out))["branch_results"]["0"]["per_ratio"]
        for (r, key), val in want.items():
            got = per_ratio[r]["scores"][key]["distortion"]["6"]
            assert abs(got - val) < 2e-8, (sem, r, key, got, val)
            assert per_ratio[r]["scores"][key.replace("T4", "T1")]["distortion"]["6"] < 1e-6
        for (r, sc), val in ndcg.items():  # ranking diagnostics stay on exact top-k under either semantics
            m = per_ratio[r]["scores"][f"{sc}@T4"]
            assert abs(m["ndcg_at_k"] - val) < 2e-8 and abs(m["recall_at_k"] - recall[(r, sc)]) < 1e-5, (sem, r, sc, m)


def test_front_block_arms_and_profile_switches(trace, monkeypatch, capsys):
    """The A/B switches of the replay: unknown values raise; the host arms of the front block, the
    whole-file read arm and the profile print leave the report unchanged."""
    cfgs = CONFIGS[:2]
    base = RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g", "update"], ratios=[5.0])
    for name in (RF.ENV_SELECT, RF.ENV_FRONT_SORT, RF.ENV_P1_READ, RF.ENV_S0_PROFILE):
        monkeypatch.setenv(name, "bogus")
        with pytest.raises(ValueError, match=name):
            RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g"], ratios=[5.0])
        monkeypatch.delenv(name)
    monkeypatch.setenv(RF.ENV_SELECT, "cpu")
    monkeypatch.setenv(RF.ENV_FRONT_SORT, "cpu")
    monkeypatch.setenv(RF.ENV_P1_READ, "load")
    monkeypatch.setenv(RF.ENV_S0_PROFILE, "1")
    other = RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g", "update"], ratios=[5.0])
    assert other["front"] == base["front"] and other["results"] == base["results"]
    arms = other["profile"][0]["arms"]
    assert arms["front_sel"] == "cpu" and arms["front_sort"] == "cpu" and arms["g_read"] == "load"
    out = capsys.readouterr().out
    assert "[fused] S0PROFILE group 0: configs=2" in out and "host_syncs=" in out and "S0PROFILE phases" in out


# ---------------------------------------------------------------- pread arm, background front ranking
def test_pt_index_reads_slices_without_loading(tmp_path):
    from sga_b200.replay.ptfile import PtIndex

    torch.manual_seed(0)
    base = torch.randn(50)
    blob = {"meta": {"step": 3, "lr": [1e-3], "nested": {"a": (1, 2.5, "x")}},
            "payload": {"a": torch.randn(7, 5), "b": torch.randn(11).to(torch.bfloat16), "view": base[10:30],
                        "scalar": torch.tensor(2.0)}}
    path = str(tmp_path / "step.pt")
    torch.save(blob, path)
    idx = PtIndex(path)
    assert idx.tree["meta"] == blob["meta"]
    fd = os.open(path, os.O_RDONLY)
    try:
        for name, t in blob["payload"].items():
            stub = idx.tree["payload"][name]
            assert stub.dtype == t.dtype and stub.numel() == t.numel()
            flat = t.reshape(-1)
            for first, count in ((0, t.numel()), (t.numel() // 3, t.numel() - t.numel() // 3), (0, 0)):
                got = idx.read_slice(fd, stub, first, count)
                assert got.dtype == t.dtype and torch.equal(got, flat[first:first + count])
        with pytest.raises(ValueError, match="outside"):
            idx.read_slice(fd, idx.tree["payload"]["a"], 30, 10)
        # a storage record shorter than its tensor claims must fail before any read
        stub = idx.tree["payload"]["a"]
        idx.records[stub.key] = (idx.records[stub.key][0], 16)
        with pytest.raises(ValueError, match="too short"):
            idx.read_slice(fd, stub, 0, 4)
    finally:
        os.close(fd)
    with pytest.raises(ValueError, match="not a torch.save archive"):
        import zipfile
        bad = str(tmp_path / "bad.pt")
        with zipfile.ZipFile(bad, "w") as z:
            z.writestr("readme.txt", "no pickle here")
        PtIndex(bad)


@pytest.mark.parametrize("g_dtype", ["fp32", "bf16"])
def test_pread_arm_equals_mmap_arm(tmp_path, monkeypatch, g_dtype):
    d = make_synthetic_trace(str(tmp_path / "t"), sizes=SIZES, steps=5, g_dtype=g_dtype, seed=11)
    info = RC.discover_trace(d)
    steps = info.window(0, 5)
    for lo, hi in ((0, info.numel), (3500, 7200), (4000, 4001)):   # whole vector, a shard across parameters, one element
        for dtype in (torch.float32, torch.bfloat16):
            outs = {}
            for arm in ("mmap", "pread"):
                monkeypatch.setenv(RF.ENV_P1_READ, arm)
                cache = {}
                pf = RF.GPrefetcher(info, steps, lo, hi, dtype, pin=False, index_cache=cache)
                outs[arm] = [pf.get() for _ in steps]
                if arm == "pread":
                    assert len(cache) == len(steps) and pf.mode == "pread"
            for (ta, ma, fa), (tb, mb, fb) in zip(outs["mmap"], outs["pread"]):
                assert ta == tb and ma == mb and fa.dtype == fb.dtype and torch.equal(fa, fb)


def test_pread_arm_failure_is_latched_and_report_is_unchanged(trace, monkeypatch):
    info = RC.discover_trace(trace)
    monkeypatch.setenv(RF.ENV_P1_READ, "pread")
    pf = RF.GPrefetcher(info, [0, 1, 99], 0, info.numel, torch.float32, pin=False)   # step 99 does not exist
    pf.get()
    pf.get()
    with pytest.raises(RuntimeError, match="prefetch failed"):
        pf.get()
    cfgs = CONFIGS[:2]
    got = RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g"], ratios=[5.0])
    assert got["profile"][0]["arms"]["g_read"] == "pread"
    monkeypatch.delenv(RF.ENV_P1_READ)
    base = RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g"], ratios=[5.0])
    assert got["front"] == base["front"] and got["results"] == base["results"]


def test_front_rank_lane_background_equals_inline_and_keeps_failures(trace, monkeypatch):
    cfgs = CONFIGS[:2]
    monkeypatch.setenv(RF.ENV_FRONT_RANK_BG, "bogus")
    with pytest.raises(ValueError, match=RF.ENV_FRONT_RANK_BG):
        RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g"], ratios=[5.0])
    reports = {}
    for arm in ("on", "off"):
        monkeypatch.setenv(RF.ENV_FRONT_RANK_BG, arm)
        reports[arm] = RF.run_fused_branch(trace, 0, cfgs, 12, [12], score_names=["abs_g", "update"], ratios=[2.0, 5.0])
        assert reports[arm]["profile"][0]["arms"]["front_rank_bg"] == arm
    assert reports["on"]["front"] == reports["off"]["front"] and len(reports["on"]["front"]) == 4
    assert reports["on"]["results"] == reports["off"]["results"]

    # the lane by itself: order of submission, a worker failure surfaces in submit or finish, never as a hang
    lane = RF.RankLane(True, torch.device("cpu"), depth=1)
    s = torch.tensor([3.0, 1.0, 2.0])
    for i in range(5):
        lane.submit(("cell", i), s, s.clone(), s.clone(), 3, 0.5, [3.0, 0.0, 6.0, 0.0, 6.0], False)
    res = lane.finish()
    assert list(res) == [("cell", i) for i in range(5)] and res[("cell", 0)]["ndcg_at_k"] == pytest.approx(1.0)
    bad = RF.RankLane(True, torch.device("cpu"), depth=1)
    with pytest.raises(RuntimeError, match="front ranking failed"):
        for i in range(8):   # the first item kills the worker; a later submit or the finish must report it
            bad.submit(("cell", i), "not a tensor", s, s, 3, 0.5, [0.0] * 5, False)
        bad.finish()
