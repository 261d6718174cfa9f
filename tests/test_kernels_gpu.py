"""Single-GPU A/B tests: every native kernel against a plain PyTorch reference.

Optimizer tails are compared bit for bit with the fp32 PyTorch reference of the
same operation order; selection kernels must be exact; bf16 model ops are held
to bf16 rounding tolerances against fp32 references. Sizes include awkward
ones (1, 1023, 1025, non multiples of the vector width).
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _k():
    from sga_b200 import kernels

    return kernels


def _kt():
    from sga_b200 import kernels_torch

    return kernels_torch


# ---------------------------------------------------------------- GEMM
@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("shape", [(256, 512, 256), (384, 768, 192), (200, 328, 136), (128, 256, 64),
                                   (1024, 1280, 320)])
def test_gemm_layouts(a_mn, b_mn, shape, pair):
    """Single-CTA (128 x 256) and CTA-pair (256 x 256) tcgen05 kernels; the pair
    kernel takes over from M >= 256."""
    K = _k()
    M, N, Kd = shape
    torch.manual_seed(1)
    Al = torch.randn(M, Kd, device=DEV) * 0.5
    Bl = torch.randn(N, Kd, device=DEV) * 0.5
    A = (Al.t().contiguous() if a_mn else Al).to(torch.bfloat16)
    B = (Bl.t().contiguous() if b_mn else Bl).to(torch.bfloat16)
    ref = (A.t() if a_mn else A).float() @ (B.t() if b_mn else B).float().t()
    out = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_bf16(A, B, out, a_mn=bool(a_mn), b_mn=bool(b_mn), pair=pair)
    assert int(K.gemm_err_word(DEV).item()) == 0
    assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item()
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    K.gemm_bf16(A, B, acc, a_mn=bool(a_mn), b_mn=bool(b_mn), epi=K.EPI_F32_ACC, pair=pair)
    assert (acc - (ref + 1.0)).abs().max().item() <= 2e-3 * ref.abs().max().item()
    res = torch.randn(M, N, device=DEV).to(torch.bfloat16)
    out2 = torch.zeros_like(out)
    K.gemm_bf16(A, B, out2, a_mn=bool(a_mn), b_mn=bool(b_mn), epi=K.EPI_BF16_ADD, residual=res, pair=pair)
    assert (out2.float() - (ref + res.float())).abs().max().item() <= 0.03 * ref.abs().max().item()


# ----------------------------------------------------------- optimizer
def _adam_case(n, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn(n, generator=g) * 0.02
    grad = torch.randn(n, generator=g) * 1e-3
    m = torch.randn(n, generator=g) * 1e-4
    v = (torch.randn(n, generator=g) * 1e-4).abs()
    mask = (torch.rand(n, generator=g) < 0.3).to(torch.uint8)
    return w, grad, m, v, mask


VARIANTS = [
    dict(emit="update"), dict(emit="abs_g"), dict(emit="abs_m"), dict(emit="coi"),
    dict(emit=None, use_mask=True, clear=True),
    dict(emit=None, use_mask=True, clear=True, coeff=0.37),
    dict(emit=None, use_mask=True, clear=True, fold=True, interval=4.0),
    dict(emit=None, use_mask=False, clear=True),
    dict(emit="update", use_mask=True, lr_scale=0.25),
    dict(emit="update", use_mask=True, lr_scale=0.25, coeff=0.37),
]


@pytest.mark.parametrize("opt", ["adamw", "adams"])
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("n", [1, 1023, 4096 + 5, 70001])
def test_adam_step_bitwise(opt, variant, n):
    K = _k()
    from sga_b200.plugins.optimizer.reference import grad_correct_torch
    from sga_b200.plugins.scores import EMIT_CODES

    w, grad, m, v, mask = _adam_case(n)
    lr, b1, b2, eps, wd, step = 3e-4, 0.9, 0.95, 1e-8, 0.1, 7
    use_mask = variant.get("use_mask", False)
    rw, rg, rm, rv = (t.clone().to(DEV) for t in (w, grad, m, v))  # same ops, evaluated by PyTorch on the device
    grad_correct_torch(rw, rg, rm, rv, lr, b1, b2, eps, wd, 1 - b1 ** step, 1 - b2 ** step,
                       mask.to(DEV) if use_mask else None, variant.get("emit"), coeff=variant.get("coeff", 1.0),
                       clear=variant.get("clear", False), fold=variant.get("fold", False),
                       interval=variant.get("interval", 1.0), inactive_lr_scale=variant.get("lr_scale", 1.0),
                       optimizer=opt)
    dw, dg, dm, dv = (t.to(DEV) for t in (w, grad, m, v))
    model = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    table = K.SegmentTable([0], [0], n, DEV)
    coeff = torch.tensor([variant["coeff"]], dtype=torch.float32, device=DEV) if "coeff" in variant else None
    K.adam_step(dw, dg, dm, dv, table, [lr], [wd], beta1=b1, beta2=b2, eps=eps, step=step, model=model,
                mask=mask.to(DEV) if use_mask else None, coeff=coeff, emit=EMIT_CODES[variant.get("emit")],
                clear=variant.get("clear", False), fold=variant.get("fold", False),
                interval=variant.get("interval", 1.0), lr_scale=variant.get("lr_scale", 1.0), adams=(opt == "adams"))
    torch.cuda.synchronize()
    assert torch.equal(dm, rm), "m differs"
    assert torch.equal(dv, rv), "v differs"
    assert torch.equal(dw, rw), "w differs"
    assert torch.equal(dg, rg), "grad buffer differs"
    assert torch.equal(model, rw.to(torch.bfloat16))


def test_adam_step_segments_groups():
    K = _k()
    from sga_b200.plugins.optimizer.reference import grad_correct_torch

    sizes, groups = [4096, 64, 8192 + 64, 128], [0, 1, 0, 1]
    n = sum(sizes)
    starts = [0]
    for s in sizes[:-1]:
        starts.append(starts[-1] + s)
    w, grad, m, v, _ = _adam_case(n, seed=3)
    lrs, wds = [1e-3, 2e-3], [0.1, 0.0]
    rw, rg, rm, rv = (t.clone().to(DEV) for t in (w, grad, m, v))
    for s, sz, gi in zip(starts, sizes, groups):
        sl = slice(s, s + sz)
        grad_correct_torch(rw[sl], rg[sl], rm[sl], rv[sl], lrs[gi], 0.9, 0.95, 1e-8, wds[gi], 1 - 0.9 ** 2,
                           1 - 0.95 ** 2, None, "update")
    dw, dg, dm, dv = (t.to(DEV) for t in (w, grad, m, v))
    K.adam_step(dw, dg, dm, dv, K.SegmentTable(starts, groups, n, DEV), lrs, wds, beta1=0.9, beta2=0.95, eps=1e-8,
                step=2, emit=0)
    assert torch.equal(dw, rw) and torch.equal(dg, rg)


def test_sumsq_and_clip():
    K = _k()
    x = torch.randn(100003, device=DEV)
    mask = (torch.rand(100003, device=DEV) < 0.5).to(torch.uint8)
    out = torch.zeros(1, device=DEV)
    K.sumsq(x, out)
    assert abs(out.item() - (x.double() ** 2).sum().item()) <= 1e-4 * out.item()
    first = out.item()
    K.sumsq(x, out)
    assert out.item() == first, "sum of squares must be deterministic"
    K.sumsq(x, out, mask=mask)
    ref = ((x * mask).double() ** 2).sum().item()
    assert abs(out.item() - ref) <= 1e-4 * ref
    coeff = torch.zeros(1, device=DEV)
    norm = torch.zeros(1, device=DEV)
    K.clip_coeff(out, 1.0, 1.0, coeff, norm)
    assert abs(norm.item() - math.sqrt(ref)) < 1e-2
    assert abs(coeff.item() - 1.0 / (math.sqrt(ref) + 1e-6)) < 1e-5


# ------------------------------------------------------------ selection
@pytest.mark.parametrize("n", [1, 1000, 1 << 16, (1 << 20) + 77])
@pytest.mark.parametrize("mode", [(16, 1, 32769), (16, 8, 32769), (19, 8, 4097)])
def test_hist_top(n, mode):
    K, KT = _k(), _kt()
    shift, stride, nb = mode
    x = (torch.randn(n, device=DEV) * 1e-3) * (1 + 20 * (torch.rand(n, device=DEV) < 0.01))
    h = K.hist_top(x, shift, stride, nb)
    ref = KT.hist_top(x.cpu(), shift, stride, nb)
    assert torch.equal(h.cpu(), ref)


def test_exact_threshold_two_digit():
    K, KT = _k(), _kt()
    n, k = (1 << 18) + 3, 2621
    x = torch.randn(n, device=DEV) * 1e-3
    h = K.hist_top(x, 16, 1, 32769)
    cum = torch.cumsum(h.flip(0), 0)  # suffix counts from the top bin
    b = 32768 - int(torch.searchsorted(cum, torch.tensor(k, device=DEV)).item())
    above = int(h[b + 1:].sum().item())
    h2 = K.hist_low16(x, b)
    assert int(h2.sum().item()) == int(h[b].item())
    cum2 = torch.cumsum(h2.flip(0), 0)
    lb = 65535 - int(torch.searchsorted(cum2, torch.tensor(k - above, device=DEV)).item())
    key = (b << 16) | lb
    ref_key = torch.kthvalue(KT.abs_bit_key(x.cpu()), n - k + 1).values.item()
    assert key == ref_key


@pytest.mark.parametrize("n", [5, 4096, 4097, 300001])
def test_mask_compact_stats(n):
    K, KT = _k(), _kt()
    x = torch.randn(n, device=DEV)
    mask = torch.empty(n, dtype=torch.uint8, device=DEV)
    cnt = torch.zeros(1, dtype=torch.int64, device=DEV)
    K.mask_ge(x, mask, thr=1.0, count=cnt)
    ref = (x.abs() >= 1.0)
    assert torch.equal(mask.bool(), ref) and cnt.item() == int(ref.sum())
    mask2 = torch.empty_like(mask)
    K.mask_ge(x, mask2, bin_=0x3F80, shift=16)
    assert torch.equal(mask2.bool(), KT.abs_bit_key(x, 16) >= 0x3F80)
    st = K.mask_stats(mask)
    assert torch.equal(st.cpu(), KT.mask_stats(mask.cpu()))
    for off in (1, 7, 15):  # views that start off the 16-byte grid of the vector loads
        if n > off + 1:
            assert torch.equal(K.mask_stats(mask[off:]).cpu(), KT.mask_stats(mask[off:].cpu())), off
    idx = torch.full((n,), -1, dtype=torch.int32, device=DEV)
    total = torch.zeros(1, dtype=torch.int64, device=DEV)
    K.compact_mask(mask, idx, total)
    ref_idx = KT.compact_mask_idx(mask)
    assert total.item() == ref_idx.numel()
    assert torch.equal(idx[:ref_idx.numel()], ref_idx)
    tb = K.dir_table(idx, ref_idx.numel(), n)
    assert torch.equal(tb.cpu(), KT.dir_table(ref_idx.cpu(), ref_idx.numel(), n))


def test_pack_scatter_blocks():
    K, KT = _k(), _kt()
    n = 50000
    g = torch.randn(n, device=DEV)
    mask = (torch.rand(n, device=DEV) < 0.1).to(torch.uint8)
    idx = KT.compact_mask_idx(mask)
    vals = torch.empty(idx.numel(), device=DEV)
    g1, g2 = g.clone(), g.clone()
    K.pack_selected(g1, idx, vals, factor=0.5, zero=True)
    rv = torch.empty_like(vals)
    KT.pack_selected(g2, idx, rv, factor=0.5, zero=True)
    assert torch.equal(vals, rv) and torch.equal(g1, g2)
    K.scatter_selected(g1, idx, vals)
    KT.scatter_selected(g2, idx, rv)
    assert torch.equal(g1, g2)
    # block forms
    x = 16
    bmask = (torch.rand((n + x - 1) // x, device=DEV) < 0.2).to(torch.uint8)
    emask = K.expand_blocks(bmask, x, n)
    assert torch.equal(emask, KT.expand_blocks(bmask, x, n))
    heads = (KT.compact_mask_idx(bmask) * x).to(torch.int32)
    bv = torch.empty(heads.numel() * x, device=DEV)
    rbv = torch.empty_like(bv)
    g1, g2 = g.clone(), g.clone()
    K.gather_selected_blocks(g1, emask, heads, x, bv, factor=0.25)
    KT.gather_selected_blocks(g2, emask, heads, x, rbv, factor=0.25)
    assert torch.equal(bv, rbv) and torch.equal(g1, g2)
    K.scatter_selected_blocks(g1, emask, heads, x, bv)
    KT.scatter_selected_blocks(g2, emask, heads, x, rbv)
    assert torch.equal(g1, g2)
    br = K.block_reduce(g, x, True)
    assert torch.equal(br, KT.block_reduce(g, x, True))
    brm = K.block_reduce(g, x, False)
    assert torch.allclose(brm, KT.block_reduce(g, x, False), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("x", [4, 8, 64, 3])
def test_block_forms_on_device_match_cpu(x):
    """Block heads and packed descriptors derived on the device against the per-span PyTorch path."""
    from sga_b200.support import block_desc_from_mask, block_idx_from_mask

    torch.manual_seed(x)
    al = x if x & (x - 1) == 0 else 1
    spans, off = [], 0
    for ln in (1000, 4096, 7, 333, 65536 + 5, 12):
        spans.append((off, off + ln))
        off = (off + ln + al - 1) // al * al + (al * 3)  # gaps between spans, starts aligned to the block size
    n = off
    mask = (torch.rand(n) < 0.05).to(torch.uint8)
    for s, e in zip([0] + [b for _a, b in spans], [a for a, _b in spans] + [n]):
        mask[s:e] = 0  # nothing selected in the gaps
    ref = block_idx_from_mask(mask, spans, x)
    got = block_idx_from_mask(mask.to(DEV), spans, x)
    assert torch.equal(got.cpu(), ref)
    if x >= 4 and x & (x - 1) == 0:
        whole = torch.zeros(n, dtype=torch.uint8)
        for h in ref.tolist()[::3]:
            sp = next((a, b) for a, b in spans if a <= h < b)
            whole[h:min(h + x, sp[1])] = 1
        rd = block_desc_from_mask(whole, spans, x)
        gd = block_desc_from_mask(whole.to(DEV), spans, x)
        assert torch.equal(gd.cpu(), rd) and rd.numel() > 0
        with pytest.raises(AssertionError, match="partially selected"):
            block_desc_from_mask(mask.to(DEV), spans, x)


# ---------------------------------------------- fused peer kernels, 1 rank
def _channel():
    from sga_b200.parallel.p2p import PeerChannel
    from sga_b200.parallel.symm import SymmPool

    pool = SymmPool(device=DEV)
    return pool, PeerChannel(pool)


def _check_index_sync(acc0, k, score=None, score_abs=None, scale=0.5, reps=2, max_ctas=0):
    """One rank: selection, payload, residual write-back, staging buffer and norm of the fused
    rank-local chain against the PyTorch oracle (``score_abs``: |score| per coordinate)."""
    import numpy as np

    from sga_b200.parallel import p2p

    KT = _kt()
    n = acc0.numel()
    pool, ch = _channel()
    try:
        sa = acc0.abs() if score_abs is None else score_abs
        ref_mask = KT.topk_rank_local(sa, k)
        ref_idx = KT.compact_mask_idx(ref_mask)
        ksel = ref_idx.numel()
        slots = p2p.IndexSyncSlots(pool, k, n)
        comm = torch.zeros(n, device=DEV)
        sq = torch.zeros(1, device=DEV)
        scratch = p2p.IndexSyncScratch(DEV, n)
        acc = acc0.clone()
        for rep in range(reps):  # the second launch checks what the first left in the scratch
            acc.copy_(acc0)
            comm.zero_()
            p2p.bucket_index_sync_(ch, scratch, acc, k, slots=slots, comm=comm, scale=scale, sumsq_out=sq,
                                   score=score, max_ctas=max_ctas)
            ch.check()
            assert int(scratch.result[3].item()) == ksel
            pairs = slots.pairs(0, ksel)
            order = torch.argsort(pairs[:, 0])
            assert torch.equal(pairs[order, 0], ref_idx), "selected indices differ from exact top-k"
            vals = pairs[order, 1].contiguous().view(torch.float32)
            assert torch.equal(vals, acc0[ref_idx.long()])
            exp_acc = torch.where(ref_mask.bool(), torch.zeros_like(acc0), acc0)
            assert torch.equal(acc, exp_acc), "residual write-back differs"
            exp_comm = torch.where(ref_mask.bool(), acc0 * scale, torch.zeros_like(acc0))
            assert torch.equal(comm, exp_comm)
            assert abs(sq.item() - (exp_comm.double() ** 2).sum().item()) <= 1e-4 * max(sq.item(), 1e-30)
        # select-only mode writes the bit mask and leaves the bucket alone
        acc.copy_(acc0)
        bits = torch.full(((n + 31) // 32,), -1, dtype=torch.int32, device=DEV)
        p2p.bucket_index_sync_(ch, scratch, acc, k, bits=bits, select_only=True, score=score, max_ctas=max_ctas)
        ch.check()
        un = np.unpackbits(bits.cpu().numpy().view("uint8"), bitorder="little")[:n]
        assert np.array_equal(un, ref_mask.cpu().numpy())
        assert torch.equal(acc, acc0)
        return scratch
    finally:
        pool.close()


@pytest.mark.parametrize("n,k", [(4096, 41), (100000, 1000), ((1 << 20) + 13, 10486), (5000, 5000), (777, 1),
                                 (3 * (1 << 20) + 77, 31458)])
def test_bucket_index_sync_single_rank(n, k):
    torch.manual_seed(n)
    acc = torch.randn(n, device=DEV) * 1e-3
    acc[::97] = 0.5  # many exact ties at the top: the tie cut by index decides
    _check_index_sync(acc, k)


@pytest.mark.parametrize("max_ctas", [1, 5])
def test_bucket_index_sync_few_ctas(max_ctas):
    """A grid far smaller than the bucket: every warp walks many segments, every CTA many ranges."""
    n = 5 * (1 << 20) + 3
    torch.manual_seed(max_ctas)
    acc = torch.randn(n, device=DEV) * 1e-3
    acc[::1013] = -0.75
    _check_index_sync(acc, 60000, max_ctas=max_ctas)


def test_bucket_index_sync_degenerate_inputs():
    n = (1 << 21) + 5
    torch.manual_seed(3)
    # all zeros: nothing is selected
    _check_index_sync(torch.zeros(n, device=DEV), 2000, reps=1)
    # fewer non-zero coordinates than k: exactly those
    acc = torch.zeros(n, device=DEV)
    acc[torch.randperm(n, device=DEV)[:700]] = torch.randn(700, device=DEV)
    _check_index_sync(acc, 2000, reps=1)
    # one magnitude everywhere: the k lowest indices
    _check_index_sync(torch.full((n,), -0.125, device=DEV), 3000, reps=1)
    # the hashed 1/64 sample sees only large values (they sit exactly where it looks) and puts the
    # bound among them, but there are fewer of them than k: the second filter pass over every
    # non-zero element must take over
    acc = torch.randn(n, device=DEV) * 1e-6
    g = torch.arange((n // 4 + 63) // 64, device=DEV, dtype=torch.int64)
    h = ((g * 2654435761) & 0xFFFFFFFF) >> 26
    base = ((g << 6) + h) * 4
    base = base[base + 4 <= n]
    for j in range(4):
        acc[base + j] = 1.0 + torch.rand(base.numel(), device=DEV)
    scratch = _check_index_sync(acc, 100000, reps=1)
    assert int(scratch.state[1].item()) == 1, "the fallback pass did not run"


@pytest.mark.parametrize("name", ["update", "abs_m", "coi"])
@pytest.mark.parametrize("adams", [False, True])
def test_bucket_index_sync_scores(name, adams):
    from sga_b200.parallel import p2p
    from sga_b200.plugins.scores import compute_score

    n = (1 << 21) + 40
    torch.manual_seed(11)
    acc = torch.randn(n, device=DEV) * 1e-3
    w = torch.randn(n, device=DEV) * 0.02
    m = torch.randn(n, device=DEV) * 1e-4
    v = torch.rand(n, device=DEV) * 1e-7
    starts = [0, 400000, 400004, 1500000, n]
    wds = [0.1, 0.0, 0.1, 0.0]
    beta1, beta2, eps, step = 0.9, 0.95, 1e-8, 7
    inp = p2p.ScoreInputs(name, w=w, m=m, v=v, beta1=beta1, beta2=beta2, eps=eps, step=step, adams=adams,
                          span_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                          span_wd=torch.tensor(wds, dtype=torch.float32, device=DEV))
    sa = torch.empty_like(acc)
    for (s, e), wd in zip(zip(starts[:-1], starts[1:]), wds):
        sa[s:e] = compute_score(name, w[s:e], m[s:e], v[s:e], acc[s:e], beta1=beta1, beta2=beta2, eps=eps,
                                weight_decay=wd, bc1=inp.bc1, bc2=inp.bc2,
                                optimizer="adams" if adams else "adamw").abs()
    _check_index_sync(acc, 20000, score=inp, score_abs=sa, reps=1)


def test_p2p_allreduce_and_mask_union_single_rank():
    from sga_b200.parallel import p2p

    KT = _kt()
    pool, ch = _channel()
    try:
        n = 100003
        buf = pool.alloc(4 * n)
        v = buf.view(torch.float32, 0, n)
        x = torch.randn(n, device=DEV)
        v.copy_(x)
        sq = torch.zeros(1, device=DEV)
        p2p.allreduce_(ch, buf, 0, n, scale=0.5, sumsq_out=sq)
        ch.check()
        assert torch.equal(v, x * 0.5)
        assert abs(sq.item() - ((x * 0.5).double() ** 2).sum().item()) <= 1e-4 * sq.item()
        # pack -> reduce -> scatter round trip
        grad = torch.randn(4 * n, device=DEV)
        g0 = grad.clone()
        mask = (torch.rand(4 * n, device=DEV) < 0.2).to(torch.uint8)
        idx = KT.compact_mask_idx(mask)[:n]
        p2p.allreduce_(ch, buf, 0, idx.numel(), scale=1.0, grad=grad, idx=idx, factor=0.25, pack=True,
                       zero_after_pack=True, scatter=True)
        ch.check()
        exp = g0.clone()
        exp[idx.long()] = g0[idx.long()] * 0.25
        assert torch.equal(grad, exp)
        # descriptor wire form: whole runs of x elements (the last run of a span shorter), 16 bytes at a time
        from sga_b200.backends.nccl_pipelined_index import expand_descriptors
        from sga_b200.support import block_desc_from_mask

        for xb in (4, 16, 64):
            spans = [(0, 50000 + 3), (50048, 200000 + 1), (200064, 4 * n - 7)]
            whole = torch.zeros(4 * n, dtype=torch.uint8, device=DEV)
            for s0, e0 in spans:
                heads = torch.arange(s0, e0, xb, device=DEV)
                pick = heads[torch.rand(heads.numel(), device=DEV) < 0.02]
                pick = torch.cat([pick, heads[-1:]])  # always the span's last (short) run
                for h in pick.tolist()[:400]:
                    whole[h:min(h + xb, e0)] = 1
            desc = block_desc_from_mask(whole, spans, xb)
            assert desc.numel() * xb <= n
            grad.copy_(g0)
            p2p.allreduce_(ch, buf, 0, desc.numel() * xb, scale=1.0, grad=grad, idx=desc, factor=0.5, pack=True,
                           scatter=True, block_x=xb, sumsq_out=sq)
            ch.check()
            eidx = expand_descriptors(desc, xb).long()
            assert torch.equal(eidx, torch.nonzero(whole).view(-1))
            exp = g0.clone()
            exp[eidx] = g0[eidx] * 0.5
            assert torch.equal(grad, exp), f"descriptor form, x={xb}"
            assert abs(sq.item() - (exp[eidx].double() ** 2).sum().item()) <= 1e-4 * sq.item()
        # mask union (one rank: union == own mask, values scaled in place)
        gb = pool.alloc(4 * n)
        bb = pool.alloc(4 * ((n + 31) // 32))
        ub = pool.alloc(4 * ((n + 31) // 32))
        g = gb.view(torch.float32, 0, n)
        import numpy as np

        for density in (0.05, 0.6, 1.0):   # sparse words, words with most bits set, every coordinate
            g.copy_(x)
            m = (torch.rand(n, device=DEV) < density)
            packed = np.packbits(m.cpu().numpy().astype("uint8"), bitorder="little")
            packed = np.concatenate([packed, np.zeros((-len(packed)) % 4, dtype="uint8")]).view("int32")
            bb.view(torch.int32, 0, packed.size).copy_(torch.from_numpy(packed.copy()))
            mu8 = torch.empty(n, dtype=torch.uint8, device=DEV)
            cnt = torch.zeros(1, dtype=torch.int64, device=DEV)
            p2p.mask_union_reduce_(ch, gb, 0, bb, 0, ub, 0, n, scale=0.5, mask_u8=mu8, sumsq_out=sq, count_out=cnt)
            ch.check()
            assert torch.equal(mu8.bool(), m), density
            assert torch.equal(g, torch.where(m, x * 0.5, x)), density
            assert cnt.item() == int(m.sum()), density
            want = (torch.where(m, x * 0.5, torch.zeros_like(x)).double() ** 2).sum().item()
            assert abs(sq.item() - want) <= 1e-4 * max(want, 1e-12), density
    finally:
        pool.close()


def test_peer_wait_times_out_cleanly():
    """A flag that nothing sets: the bounded wait expires, the kernel returns,
    the status word says so and the context stays usable."""
    from sga_b200.parallel import p2p

    pool, ch = _channel()
    try:
        ch.wait_cycles = 2_000_000  # about a millisecond
        n = 4096
        buf = pool.alloc(4 * n)
        ch.seq = 5
        d = ch.next_desc()
        d.seq = 1 << 20  # wait for a sequence number nobody will ever publish
        import ctypes

        from sga_b200.csrc import lib

        # signal uses d.seq too, so waiting on our own signal would succeed; make W=2 with a
        # second "rank" whose flag word is our own memory that nobody writes
        d.W = 2
        d.flags[1] = ch.ctrl.peer_ptrs[0] + 128
        bufs = buf.ptr_array(0)
        bufs[1] = bufs[0]
        ns = ch.norm_slots()
        ns[1] = ns[0]
        rc = lib().sga_p2p_allreduce(ctypes.byref(d), bufs, n, 1.0, None, None, 1.0, 0, 0, 0, 0, 0, ns,
                                     ch.cta_partials.data_ptr(), None, 0, 0, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        with pytest.raises(p2p.PeerTimeout):
            ch.check()
        x = torch.ones(8, device=DEV)
        assert (x + 1).sum().item() == 16.0
    finally:
        pool.close()


# ------------------------------------------------------------ model ops
def test_rmsnorm_fwd_bwd():
    from sga_b200.ops import functional as F

    for T, H in [(64, 2048), (37, 1024), (50, 128), (16, 4096)]:
        x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
        dy = torch.randn(T, H, device=DEV).to(torch.bfloat16)
        y, rstd = F.rmsnorm_fwd(x, w, 1e-5)
        xf = x.float().requires_grad_()
        wf = w.float().requires_grad_()
        ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        assert (y.float() - ref).abs().max().item() < 0.05
        ref.backward(dy.float())
        dw = torch.zeros(H, device=DEV)
        dx = F.rmsnorm_bwd(x, w, dy, rstd, dw_out=dw)
        assert (dx.float() - xf.grad).abs().max().item() < 0.06
        assert (dw - wf.grad).abs().max().item() < 0.02 * wf.grad.abs().max().item() + 0.05


def test_rope_swiglu_ce_embed():
    from sga_b200.ops import functional as F

    T, S, nh, hd = 64, 32, 4, 64
    x = torch.randn(T, nh * hd, device=DEV).to(torch.bfloat16)
    cs, sn = F.rope_tables(S, hd, 500000.0, DEV)
    x0 = x.clone()
    F.rope_(x, cs, sn, S, nh, hd, 0, +1.0)
    xf = x0.float().view(T, nh, hd)
    pos = torch.arange(T, device=DEV) % S
    c, s = cs[pos][:, None, :], sn[pos][:, None, :]
    a, b = xf[..., :hd // 2], xf[..., hd // 2:]
    ref = torch.cat([a * c - b * s, b * c + a * s], -1).view(T, nh * hd)
    assert (x.float() - ref).abs().max().item() < 0.03
    F.rope_(x, cs, sn, S, nh, hd, 0, -1.0)
    assert (x.float() - x0.float()).abs().max().item() < 0.06
    # swiglu
    Fd = 256
    gu = torch.randn(T, 2 * Fd, device=DEV).to(torch.bfloat16)
    out = F.swiglu_fwd(gu)
    guf = gu.float().requires_grad_()
    ref = torch.nn.functional.silu(guf[:, :Fd]) * guf[:, Fd:]
    assert (out.float() - ref).abs().max().item() < 0.05
    do = torch.randn(T, Fd, device=DEV).to(torch.bfloat16)
    ref.backward(do.float())
    din = F.swiglu_bwd(gu, do)
    assert (din.float() - guf.grad).abs().max().item() < 0.08
    # cross entropy (+ in-place gradient)
    V = 1000 * 8
    z = (torch.randn(T, V, device=DEV) * 2).to(torch.bfloat16)
    tgt = torch.randint(0, V, (T,), device=DEV)
    zf = z.float().requires_grad_()
    ref_loss = torch.nn.functional.cross_entropy(zf, tgt, reduction="none")
    ref_loss.mean().backward()
    loss = F.cross_entropy_(z, tgt, grad_scale=1.0 / T)
    assert (loss - ref_loss).abs().max().item() < 2e-2
    assert (z.float() - zf.grad).abs().max().item() < 2e-3
    # embedding
    W = torch.randn(500, 256, device=DEV).to(torch.bfloat16)
    ids = torch.randint(0, 500, (T,), device=DEV)
    e = F.embed_fwd(ids, W)
    assert torch.equal(e, W[ids])
    mg = torch.zeros(500, 256, device=DEV)
    de = torch.randn(T, 256, device=DEV).to(torch.bfloat16)
    F.embed_bwd(ids, de, mg)
    ref = torch.zeros_like(mg).index_add_(0, ids, de.float())
    assert (mg - ref).abs().max().item() < 1e-4


def test_dense_adamw_ag_single_rank():
    from sga_b200.parallel import p2p
    from sga_b200.plugins.optimizer.reference import grad_correct_torch

    K = _k()
    pool, ch = _channel()
    try:
        n = 3 * 4096 + 64
        w, grad, m, v, _ = _adam_case(n, seed=5)
        rw, rg, rm, rv = (t.clone().to(DEV) for t in (w, grad, m, v))
        grad_correct_torch(rw, rg * 0.5, rm, rv, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** 3, 1 - 0.95 ** 3, None, None)
        dw, dg, dm, dv = (t.to(DEV) for t in (w, grad, m, v))
        model = pool.alloc(2 * n)
        bstart = torch.tensor([0, 8192], dtype=torch.int64, device=DEV)
        blen = torch.tensor([8192, n - 8192], dtype=torch.int64, device=DEV)
        coeff = torch.tensor([0.5], device=DEV)
        p2p.dense_adamw_ag_(ch, dw, dg, dm, dv, model, bstart, blen, K.SegmentTable([0], [0], n, DEV), [1e-3], [0.1],
                            beta1=0.9, beta2=0.95, eps=1e-8, step=3, coeff=coeff)
        ch.check()
        assert torch.equal(dw, rw) and torch.equal(dm, rm) and torch.equal(dv, rv)
        assert torch.equal(model.view(torch.bfloat16, 0, n), rw.to(torch.bfloat16))
    finally:
        pool.close()
