"""CPU unit tests of the plugin axes: score formulas against fp64 hand oracles,
histogram selection against ``torch.kthvalue`` on adversarial inputs, the
adaptive controller's life cycle, the optimizer reference, support forms."""
import math

import pytest
import torch

from sga_b200 import config as C
from sga_b200 import kernels_torch as KT
from sga_b200.plugins import (plugin_class, register_backend_plugin, resolve_emission, resolve_layout)
from sga_b200.plugins.optimizer.reference import grad_correct_torch
from sga_b200.plugins.scores import compute_score, get_score_spec, register_score, score_names, ScoreSpec
from sga_b200.plugins.selection import threshold as AD
from sga_b200.plugins.selection import _histogram as H
from sga_b200.plugins.selection._exact import select_masks_exact_kthvalue
from sga_b200.support import (BucketSupport, IndexPool, Support, block_desc_from_mask, block_idx_from_mask,
                              compact_mask_u8)

HP = dict(beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)


def _state(n=257, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g) * 0.02, torch.randn(n, generator=g) * 1e-3,
            (torch.randn(n, generator=g) * 1e-3).abs(), torch.randn(n, generator=g) * 1e-2)


# ------------------------------------------------------------------ scores
@pytest.mark.parametrize("opt", ["adamw", "adams"])
def test_scores_match_fp64_oracle(opt):
    w, m, v, g = _state()
    step = 5
    bc1, bc2 = (1 - 0.9 ** step, 1 - 0.95 ** step) if opt == "adamw" else (1.0, 1.0)
    W, M, V, G = (t.double() for t in (w, m, v, g))
    m1 = 0.9 * M + 0.1 * G
    v1 = (0.95 * V if opt == "adamw" else 0.95 * M * M) + 0.05 * G * G
    ug = (m1 / bc1) / ((v1 / bc2).sqrt() + 1e-8)
    v0 = 0.95 * V if opt == "adamw" else 0.95 * M * M
    u0 = (0.9 * M / bc1) / ((v0 / bc2).sqrt() + 1e-8)
    oracle = {"update": 0.1 * W + ug, "abs_g": G.abs(), "abs_m": M.abs(), "coi": (ug - u0).abs()}
    for name, want in oracle.items():
        got = compute_score(name, w, m, v, g, bc1=bc1, bc2=bc2, optimizer=opt, **HP)
        assert got.dtype == torch.float32
        # coi is a difference of two O(1) terms: hold it to the operands' scale
        atol = 4e-6 * float(ug.abs().max()) if name == "coi" else 1e-9
        assert torch.allclose(got.double(), want, rtol=2e-5, atol=atol), name
    wd_free = compute_score("update", w, m, v, g, bc1=bc1, bc2=bc2, optimizer=opt, update_includes_wd=False, **HP)
    assert torch.allclose(wd_free.double(), ug, rtol=2e-5, atol=1e-9)


def test_score_registry():
    assert score_names() == ["abs_g", "abs_m", "coi", "update"]
    with pytest.raises(ValueError, match="Unknown SGA score"):
        get_score_spec("nope")
    with pytest.raises(ValueError, match="duplicate"):
        register_score("abs_g", ScoreSpec(lambda *a, **k: None, "x"))
    with pytest.raises(ValueError, match="Unknown SGA optimizer"):
        compute_score("update", *_state(), bc1=1.0, bc2=1.0, optimizer="sgd", **HP)


# ------------------------------------------------------- optimizer reference
def test_grad_correct_sparse_knobs_equal_standalone_sequence():
    w, m, v, g = _state(1000, 1)
    mask = (torch.rand(1000, generator=torch.Generator().manual_seed(2)) < 0.3).to(torch.uint8)
    a = [t.clone() for t in (w, g, m, v)]
    grad_correct_torch(a[0], a[1], a[2], a[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, mask, None, coeff=0.37,
                       clear=True, fold=True, interval=4.0)
    b = [t.clone() for t in (w, g, m, v)]
    b[1][mask > 0] *= 0.37                                   # standalone masked scale
    resid = b[1].clone()
    grad_correct_torch(b[0], b[1], b[2], b[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, mask, None)
    resid[mask > 0] = 0.0                                    # standalone clear
    resid = resid / torch.tensor(4.0)                        # standalone fold
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    assert torch.equal(a[1], resid)


def test_grad_correct_full_step_emits_score_and_dual_lr():
    w, m, v, g = _state(500, 3)
    mask = (torch.arange(500) % 3 == 0).to(torch.uint8)
    a = [t.clone() for t in (w, g, m, v)]
    grad_correct_torch(a[0], a[1], a[2], a[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, mask, "update",
                       inactive_lr_scale=0.25)
    b = [t.clone() for t in (w, g, m, v)]
    grad_correct_torch(b[0], b[1], b[2], b[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, None, "update")
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3]), "commit is mask-blind"
    on = mask > 0
    assert torch.equal(a[0][on], b[0][on])
    d_a, d_b = (w - a[0])[~on], (w - b[0])[~on]
    assert torch.allclose(d_a, 0.25 * d_b, rtol=1e-3, atol=8e-9)  # differences of fp32 weights near 0.02
    # masked-out lanes of a sparse step still advance m and v with g = 0
    c = [t.clone() for t in (w, g, m, v)]
    grad_correct_torch(c[0], c[1], c[2], c[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, mask, None)
    assert torch.equal(c[2][~on], m[~on] * 0.9 + torch.zeros(1) * (1.0 - 0.9))
    assert torch.equal(c[1][~on], g[~on]), "the residual stays in the grad buffer"


def test_dual_lr_boundary_clips_every_lane():
    """The boundary commit under a split lr consumes the whole merged buffer, so a deferred clip
    coefficient scales the gradient at inactive lanes as well (a sparse step scales only active ones)."""
    w, m, v, g = _state(300, 5)
    mask = (torch.arange(300) % 4 == 0).to(torch.uint8)
    a = [t.clone() for t in (w, g, m, v)]
    grad_correct_torch(a[0], a[1], a[2], a[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, mask, "abs_g", coeff=0.37,
                       inactive_lr_scale=0.5)
    b = [t.clone() for t in (w, g * 0.37, m, v)]
    grad_correct_torch(b[0], b[1], b[2], b[3], 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5, 0.4, mask, "abs_g",
                       inactive_lr_scale=0.5)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_adams_has_no_bias_correction_and_rebuilds_v():
    w, m, v, g = _state(64, 4)
    a = [t.clone() for t in (w, g, m, v)]
    grad_correct_torch(a[0], a[1], a[2], a[3], 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.123, 0.456, None, None, optimizer="adams")
    v1 = (m * m) * 0.95 + (g * (1.0 - 0.95)) * g
    assert torch.equal(a[3], v1)
    m1 = m * 0.9 + g * (1.0 - 0.9)
    assert torch.equal(a[0], w - 1e-3 * (0.0 * w + m1 / (torch.sqrt(v1) + 1e-8)))


# ----------------------------------------------------------------- selection
def _adversarial(kind, n, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "normal":
        return torch.randn(n, generator=g) * 1e-3
    if kind == "heavy":
        x = torch.randn(n, generator=g) * 1e-3
        x[torch.rand(n, generator=g) < 0.01] *= 20
        return x
    if kind == "ties":
        return torch.randint(-3, 4, (n,), generator=g).float() * 0.125
    if kind == "denormal":
        x = torch.randn(n, generator=g) * 1e-41
        x[::7] = 0.0
        return x
    if kind == "one_bin":
        return 1.0 + torch.rand(n, generator=g) * 1e-3
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["normal", "heavy", "ties", "denormal", "one_bin"])
@pytest.mark.parametrize("ratio", [0.001, 0.1, 0.6])
def test_histogram_exact_equals_kthvalue(kind, ratio):
    views = [_adversarial(kind, n, i) for i, n in enumerate((4000, 3001, 1700))]
    n = sum(v.numel() for v in views)
    k = max(1, round(n * ratio))
    thr, masks = H.select_masks_histogram(views, k, None, mode="exact")
    flat = torch.cat(views).abs()
    want = torch.kthvalue(flat, n - k + 1).values.item()
    assert thr == want, "bit-exact k-th value"
    ref_thr, ref_masks = select_masks_exact_kthvalue([v.clone() for v in views], k, None)
    assert ref_thr == thr
    for a, b in zip(masks, ref_masks):
        assert torch.equal(a, b)
    assert sum(int(m.sum()) for m in masks) >= k  # all ties at the threshold are selected


@pytest.mark.parametrize("mode,tol", [("balanced", 0.005), ("fast", 0.03)])
def test_approximate_tiers_within_tolerance(mode, tol):
    views = [_adversarial("heavy", n, i) for i, n in enumerate((40000, 30011, 17003))]
    n = sum(v.numel() for v in views)
    for ratio in (0.05, 0.2, 0.4):
        k = round(n * ratio)
        thr, masks = H.select_masks_histogram(views, k, None, mode=mode)
        got = sum(int(m.sum()) for m in masks) / n
        assert abs(got - ratio) <= tol + (0.06 * ratio if mode == "fast" else 0), (mode, ratio, got)
        shift = H.HIST_MODES[mode][0]
        b = (torch.tensor([thr]).view(torch.int32) & 0x7FFFFFFF) >> shift
        assert H.bin_edge_float(int(b), shift) == thr, "threshold is a bin's lower edge"


def test_balanced_samples_each_view_from_its_own_start():
    a, b = torch.arange(1, 20, dtype=torch.float32), torch.arange(100, 111, dtype=torch.float32)
    h = H.build_histogram([a, b], 16, H.HIST_BINS, 8)
    ref = KT.hist_top(a, 16, 8, H.HIST_BINS) + KT.hist_top(b, 16, 8, H.HIST_BINS)
    assert torch.equal(h, ref) and int(h.sum()) == H.sampled_count(19, 8) + H.sampled_count(11, 8)


def test_block_selection():
    g = torch.Generator().manual_seed(5)
    views = [torch.randn(1000, generator=g), torch.randn(515, generator=g)]
    sel = H.HistogramSelect("exact", block_size=16, block_reduce="max")
    thr, masks = sel.select(views, 160, None)
    for m, v in zip(masks, views):
        assert m.numel() == v.numel()
        nb = v.numel() // 16
        full = m[:nb * 16].view(nb, 16)
        assert bool(((full.sum(1) == 0) | (full.sum(1) == 16)).all()), "blocks are selected whole"
    nblocks = sum(int(m[::16].sum()) for m in masks)
    assert abs(nblocks - 10) <= 1
    with pytest.raises(ValueError):
        H.HistogramSelect("exact", block_size=3)
    with pytest.raises(ValueError):
        H.HistogramSelect("nope")


def test_adaptive_controller_lifecycle():
    views = [_adversarial("normal", 50000, 9)]
    n = 50000
    ad = AD.AdaptiveThresholdSelect(10.0, 2, "balanced")
    assert ad.warmup_sync_target(0, 4) == 1 and ad.warmup_sync_target(100, 4) == 0
    assert AD.AdaptiveThresholdSelect(10.0, None, "fast").warmup_sync_target(0, 4) is None
    assert AD.AdaptiveThresholdSelect(10.0, 5, "fast").warmup_sync_target(0, 4) == 4
    thr0, m0 = ad.select(views, n // 10, None, None)
    assert ad.warmup_passed == 1 and ad.tau == thr0
    ad.select(views, n // 10, None, None)
    assert ad.warmup_passed == 2
    tau = ad.tau
    used, masks = ad.select(views, n // 10, None, None)      # persistent tau from here on
    assert used == tau and torch.equal(masks[0], (views[0].abs() >= tau).to(torch.uint8))
    # outside the dead band the threshold moves by (measured/target)^0.5, clamped
    assert AD.step_threshold(1.0, 0.105, 0.10) == 1.0
    assert math.isclose(AD.step_threshold(1.0, 0.20, 0.10), 1.15)
    assert math.isclose(AD.step_threshold(1.0, 0.02, 0.10), 0.9)
    assert math.isclose(AD.step_threshold(2.0, 0.12, 0.10), 2.0 * math.sqrt(1.2))
    # collapse: a zero measured ratio re-bootstraps, clamped to the smallest positive edge
    ad.tau = 1e9
    thr, _ = ad.select(views, n // 10, None, None)
    assert 0 < thr < 1.0
    # a warm-up select that misses the band resets the consecutive count (fast over-selects here)
    miss = AD.AdaptiveThresholdSelect(10.0, 2, "fast")
    miss.warmup_passed = 1
    _, mm = miss.select(views, n // 10, None, None)
    measured = int(mm[0].sum()) / n
    assert miss.warmup_passed == (2 if abs(measured - 0.10) <= 0.01 else 0)
    zero = [torch.zeros(1000)]
    ad2 = AD.AdaptiveThresholdSelect(10.0, 1, "fast")
    t, _ = ad2.select(zero, 100, None, None)
    assert t == AD.smallest_threshold("fast") > 0.0


def test_topk_plugin_k_and_rank_gate():
    C.set_args(C.make_args(sga_enabled=True, sga_score="abs_g", sga_selection_method="histogram",
                           sga_selection_histogram_mode="exact", sga_selection_ratio_percent=1.0,
                           sga_backend="torch_pipelined_index"))
    sel = plugin_class("selection", "topk")()
    assert sel.k_for(1000) == 10 and sel.k_for(10) == 1 and sel.block_size == 1 and sel.tau is None

    class Ctx:
        grad_views = [_adversarial("normal", 5000, 1)]
        comm_group = None
        warmup_target = None

    masks = sel.select(Ctx())
    assert int(masks[0].sum()) == 50 and sel.last_threshold > 0


# ------------------------------------------------------------------ registry
def test_registries():
    assert resolve_emission(None, "compact") == "compact" and resolve_emission("writeback", "compact") == "writeback"
    assert resolve_layout("auto", 1) == "er" and resolve_layout("auto", 8) == "bb" and resolve_layout("eb", 8) == "eb"
    with pytest.raises(ValueError, match="Unknown SGA optimizer"):
        plugin_class("optimizer", "lion")
    with pytest.raises(ValueError, match="Duplicate"):
        register_backend_plugin("torch_pipelined_mask", object)
    assert plugin_class("optimizer", "adams").optimizer_name == "adams"


# ------------------------------------------------------------------- support
def _oracle_block_desc(mask, spans, x):
    out = []
    for s, e in spans:
        for h in range(s, e, x):
            run = min(x, e - h)
            if mask[h:h + run].any():
                out.append(h | (run if run < x else 0))
    return out


def test_support_forms():
    mask = torch.zeros(100, dtype=torch.uint8)
    mask[[3, 4, 50, 51, 52, 99]] = 1
    pool = IndexPool("cpu")
    idx = compact_mask_u8(mask, pool)
    assert idx.tolist() == [3, 4, 50, 51, 52, 99] and idx.dtype == torch.int32
    sup = BucketSupport(mask, idx_pool=pool)
    assert sup.count == 100 and sup.num_selected() == 6 and sup.split == 2
    assert sup.dir_table.tolist() == [0, 6]
    assert torch.equal(sup.block_idx, sup.idx)
    with pytest.raises(ValueError):
        _ = sup.block_desc
    assert Support([sup, BucketSupport(torch.ones(10, dtype=torch.uint8))]).total_selected == 16
    # block forms: blocks tile each span from its start and never cross spans
    spans = [(0, 40), (40, 100)]
    m = torch.zeros(100, dtype=torch.uint8)
    m[8:16] = 1
    m[36:40] = 1      # short tail block of span 0 (starts at 32)
    m[40:48] = 1
    m[96:100] = 1     # tail of span 1 (blocks from 40: ..., 96)
    m[32:36] = 1
    assert block_idx_from_mask(m, spans, 8).tolist() == [8, 32, 40, 96]
    m2 = m.clone()
    m2[20] = 1        # ANY rule: a single set element lists its block
    assert 16 in block_idx_from_mask(m2, spans, 8).tolist()
    desc = block_desc_from_mask(m, [(0, 40), (40, 100)], 8)
    assert desc.tolist() == _oracle_block_desc(m, spans, 8) == [8, 32, 40, 96 | 4]
    with pytest.raises(AssertionError, match="partially selected"):
        block_desc_from_mask(m2, spans, 8)
    with pytest.raises(AssertionError, match="aligned"):
        block_desc_from_mask(m, [(0, 36), (36, 100)], 8)
    with pytest.raises(AssertionError):
        block_desc_from_mask(m, spans, 2)
    bs = BucketSupport(m, block_size=8, block_spans=spans)
    assert bs.block_idx.tolist() == [8, 32, 40, 96] and bs.block_split == 3
    with pytest.raises(ValueError, match="block_spans"):
        _ = BucketSupport(m, block_size=8).block_idx


def test_descriptor_round_trip():
    from sga_b200.backends.nccl_pipelined_index import expand_descriptors

    spans = [(0, 40), (40, 100)]
    m = torch.zeros(100, dtype=torch.uint8)
    m[8:16] = 1
    m[32:40] = 1
    m[96:100] = 1
    idx = expand_descriptors(block_desc_from_mask(m, spans, 8), 8)
    assert idx.tolist() == torch.nonzero(m).view(-1).tolist()


def test_index_pool_grows_and_never_shrinks():
    p = IndexPool("cpu")
    a = p.get(10)
    assert a.numel() == 4 * 1024 * 1024
    assert p.get(5) is a
    b = p.get(4 * 1024 * 1024 + 1)
    assert b.numel() == 8 * 1024 * 1024 and p.get(3) is b
