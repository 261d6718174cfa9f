"""Tensor parallelism combined with pipeline stages, on CPU (gloo, 4 ranks as
2 tensor-parallel x 2 stages): the sharded, staged model reproduces the unsplit
model's losses and gradients over several micro-batches in flight, and the
trainer follows the single-rank trainer's trajectory, dense and with SGA."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sga_b200.models.gpt import GPT, get_config
from sga_b200.parallel.pp import Pipeline
from sga_b200.parallel.tp import TPContext


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _shard_of(full: torch.Tensor, spec) -> torch.Tensor:
    if spec.tp_pieces is None:
        return full
    dim = spec.tp_pieces[0][0]
    return torch.cat([full.narrow(dim, lo, hi - lo) for _, lo, hi in spec.tp_pieces], dim)


def _worker(rank, world, port, n_micro, vocab_parallel, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp_size, pp_size = 2, 2
        tp_rank, pp_rank = rank % tp_size, rank // tp_size
        groups = [dist.new_group(ranks=[p * tp_size + t for t in range(tp_size)]) for p in range(pp_size)]
        cfg = get_config("test_tiny_qk", num_layers=3)
        tp = TPContext(group=groups[pp_rank], device="cpu")
        assert tp.rank == tp_rank and tp.world == tp_size
        stage = GPT(cfg, device="cpu", seed=9, tp=tp, pp_size=pp_size, pp_rank=pp_rank, vocab_parallel=vocab_parallel)
        full = GPT(cfg, device="cpu", seed=9)
        for slot in stage.arena.slots:
            assert torch.equal(slot.main, _shard_of(full.arena.by_name[slot.name].main, slot.spec)), slot.name
        g = torch.Generator().manual_seed(5)
        toks = torch.randint(0, cfg.vocab, (2 * n_micro, cfg.seq_len + 1), generator=g)
        mbs = [(toks[2 * i:2 * i + 2, :-1], toks[2 * i:2 * i + 2, 1:]) for i in range(n_micro)]
        pipe = Pipeline(stage, pp_rank=pp_rank, pp_size=pp_size, prev_rank=rank - tp_size if pp_rank > 0 else None,
                        next_rank=rank + tp_size if pp_rank < pp_size - 1 else None)
        finals = []
        losses = pipe.run(mbs, loss_scale=1.0 / n_micro, on_param_done_last=lambda s: finals.append(s.name))
        ref_losses = [full.forward_backward(t, y, loss_scale=1.0 / n_micro) for t, y in mbs]
        assert sorted(finals) == sorted(s.name for s in stage.arena.slots)
        if pp_rank == pp_size - 1:
            assert len(losses) == n_micro
            for a, b in zip(losses, ref_losses):
                assert abs(float(a) - float(b)) < 2e-3 * max(1.0, abs(float(b)))
        else:
            assert losses == []
        # sharded gradients equal the full model's shard; replicated ones hold the sum over the group
        for slot in stage.arena.slots:
            ref = _shard_of(full.arena.by_name[slot.name].grad, slot.spec)
            err = float((slot.grad - ref).abs().max())
            assert err <= 0.06 * float(ref.abs().max()) + 1e-6, (slot.name, err)
        # the first stage holds two micro-batches between forward and backward: it must own two sets of gather buffers
        keys = [k[0] for k in tp.slots if isinstance(k[0], tuple) and k[0][0] == "h1"]
        inflight = {k[2] for k in keys}
        assert inflight == ({0, 1} if (pp_rank == 0 and n_micro > 1) else {0}), (pp_rank, inflight)
        if rank == 0:
            torch.save({"ok": True}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_micro,vocab_parallel", [(1, False), (4, False), (4, True)])
def test_tp2_pp2_matches_unsplit_model(tmp_path, n_micro, vocab_parallel):
    out = str(tmp_path / "r.pt")
    mp.spawn(_worker, args=(4, _free_port(), n_micro, vocab_parallel, out), nprocs=4, join=True)
    assert torch.load(out)["ok"]


def _trainer_worker(rank, world, port, tp_size, pp_size, sga, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from sga_b200.runtime.trainer import Trainer, default_args

    kw = dict(model="test_tiny_qk", micro_batch_size=2, global_batch_size=8, device="cpu", lr=1e-3, clip_grad=1.0,
              tensor_model_parallel_size=tp_size, pipeline_model_parallel_size=pp_size, log_interval=0,
              untie_embeddings_and_output_weights=True)
    if sga:
        kw.update(sga_enabled=True, sga_score="abs_g", sga_selection_method="exact", sga_selection_ratio_percent=5.0,
                  sga_backend="torch_pipelined_index", sga_selection_locality="rank_local", sga_cycle_period=3)
    tr = Trainer(default_args(**kw), quiet=True)
    assert (tr.tp_rank, tr.pp_rank, tr.dp_rank) == (rank % tp_size, rank // (tp_size * tr.dp_world),
                                                    (rank // tp_size) % tr.dp_world)
    ev0 = tr.evaluate(1)
    losses, norms = [], []
    for s in range(4):
        losses.append(float(tr.train_step(tr.host_batch(s))))
        gn = tr.last_grad_norm
        norms.append(float(gn.item()) if hasattr(gn, "item") else float(gn))
    if tr.tp is not None:
        for slot in tr.model.arena.slots:
            if slot.spec.tp_duplicate:
                parts = [torch.empty_like(slot.main) for _ in range(tp_size)]
                dist.all_gather(parts, slot.main.contiguous(), group=tr.tp_group)
                assert all(torch.equal(parts[0], p) for p in parts), slot.name
    if rank == 0:
        torch.save({"losses": losses, "norms": norms, "eval0": ev0}, out)
    tr.close()
    if dist.is_initialized():
        dist.destroy_process_group()


@pytest.mark.parametrize("sga", [False, True])
def test_tp2_pp2_trainer_tracks_single_rank(tmp_path, sga):
    a, b = str(tmp_path / "mp.pt"), str(tmp_path / "one.pt")
    mp.spawn(_trainer_worker, args=(4, _free_port(), 2, 2, sga, a), nprocs=4, join=True)
    mp.spawn(_trainer_worker, args=(1, _free_port(), 1, 1, sga, b), nprocs=1, join=True)
    ra, rb = torch.load(a), torch.load(b)
    # sparse steps select per bucket, and the sharded, staged model has other buckets: close, not equal
    ltol, ntol = (5e-2, 0.25) if sga else (2e-2, 0.05)
    assert abs(ra["eval0"] - rb["eval0"]) < 2e-3 * max(1.0, abs(rb["eval0"])), (ra["eval0"], rb["eval0"])
    assert abs(ra["losses"][0] - rb["losses"][0]) < 2e-2
    for x, y in zip(ra["losses"], rb["losses"]):
        assert abs(x - y) < ltol, (ra, rb)
    for x, y in zip(ra["norms"], rb["norms"]):
        assert abs(x - y) < ntol * max(y, 1e-3), (ra, rb)
