"""Pipeline parallelism on CPU (gloo): two stages reproduce the unsplit
model's loss and gradients micro-batch for micro-batch, and a 2-stage x
2-replica trainer follows the 2-replica trainer's trajectory."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sga_b200.models.gpt import GPT, get_config, param_specs, stage_layers
from sga_b200.parallel.pp import Pipeline


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_stage_layers_partition():
    assert [list(stage_layers(5, 2, r)) for r in range(2)] == [[0, 1, 2], [3, 4]]
    assert [list(stage_layers(4, 4, r)) for r in range(4)] == [[0], [1], [2], [3]]
    cfg = get_config("test_tiny_qk")
    names = [s.name for s in param_specs(cfg)]
    split = [s.name for r in range(2) for s in param_specs(cfg, 1, 0, 2, r)]
    assert sorted(split) == sorted(names)
    with pytest.raises(ValueError, match="untied"):
        param_specs(get_config("test_tiny"), 1, 0, 2, 0)


def _worker(rank, world, port, n_micro, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = get_config("test_tiny_qk", num_layers=3)
        stage = GPT(cfg, device="cpu", seed=9, pp_size=world, pp_rank=rank)
        full = GPT(cfg, device="cpu", seed=9)
        for slot in stage.arena.slots:
            assert torch.equal(slot.main, full.arena.by_name[slot.name].main), slot.name
        g = torch.Generator().manual_seed(5)
        toks = torch.randint(0, cfg.vocab, (2 * n_micro, cfg.seq_len + 1), generator=g)
        mbs = [(toks[2 * i:2 * i + 2, :-1], toks[2 * i:2 * i + 2, 1:]) for i in range(n_micro)]
        pipe = Pipeline(stage, pp_rank=rank, pp_size=world, prev_rank=rank - 1 if rank > 0 else None,
                        next_rank=rank + 1 if rank < world - 1 else None)
        armed, finals = [], []
        losses = pipe.run(mbs, loss_scale=1.0 / n_micro, on_param_done_last=lambda s: finals.append(s.name),
                          before_last_backward=lambda: armed.append(True))
        ref_losses = [full.forward_backward(t, y, loss_scale=1.0 / n_micro) for t, y in mbs]
        assert armed == [True]
        assert sorted(finals) == sorted(s.name for s in stage.arena.slots)
        if rank == world - 1:
            assert len(losses) == n_micro
            for a, b in zip(losses, ref_losses):
                assert abs(float(a) - float(b)) < 1e-3
        else:
            assert losses == []
        for slot in stage.arena.slots:
            ref = full.arena.by_name[slot.name].grad
            err = float((slot.grad - ref).abs().max())
            assert err <= 0.05 * float(ref.abs().max()) + 1e-6, (slot.name, err)
        if rank == 0:
            torch.save({"ok": True, "transfers": pipe.transfers}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_micro", [(2, 1), (2, 4), (3, 2)])
def test_pipeline_matches_unsplit_model(tmp_path, world, n_micro):
    out = str(tmp_path / "r.pt")
    mp.spawn(_worker, args=(world, _free_port(), n_micro, out), nprocs=world, join=True)
    r = torch.load(out)
    assert r["ok"] and r["transfers"] == 2 * n_micro  # first stage: one send and one receive per micro-batch


def _trainer_worker(rank, world, port, pp, sga, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from sga_b200.runtime.trainer import Trainer, default_args

    kw = dict(model="test_tiny_qk", micro_batch_size=2, global_batch_size=8, device="cpu", lr=1e-3, clip_grad=1.0,
              pipeline_model_parallel_size=pp, log_interval=0)
    if sga:
        kw.update(sga_enabled=True, sga_score="abs_g", sga_selection_method="exact", sga_selection_ratio_percent=5.0,
                  sga_backend="torch_pipelined_index", sga_selection_locality="rank_local", sga_cycle_period=3,
                  untie_embeddings_and_output_weights=True)
    tr = Trainer(default_args(**kw), quiet=True)
    ev0 = tr.evaluate(1)   # forward-only schedule over the stages, before any update: same weights in both layouts
    losses, norms = [], []
    for s in range(4):
        losses.append(float(tr.train_step(tr.host_batch(s))))
        gn = tr.last_grad_norm
        norms.append(float(gn.item()) if hasattr(gn, "item") else float(gn))
    if rank == 0:
        torch.save({"losses": losses, "norms": norms, "eval0": ev0}, out)
    tr.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("sga", [False, True])
def test_pp2_dp2_trainer_tracks_dp2(tmp_path, sga):
    a, b = str(tmp_path / "pp.pt"), str(tmp_path / "dp.pt")
    mp.spawn(_trainer_worker, args=(4, _free_port(), 2, sga, a), nprocs=4, join=True)
    mp.spawn(_trainer_worker, args=(2, _free_port(), 1, sga, b), nprocs=2, join=True)
    ra, rb = torch.load(a), torch.load(b)
    ltol, ntol = (5e-2, 0.25) if sga else (2e-2, 0.05)
    assert abs(ra["eval0"] - rb["eval0"]) < 2e-3 * max(1.0, abs(rb["eval0"])), (ra["eval0"], rb["eval0"])
    assert abs(ra["losses"][0] - rb["losses"][0]) < 2e-2
    for x, y in zip(ra["losses"], rb["losses"]):
        assert abs(x - y) < ltol, (ra, rb)
    for x, y in zip(ra["norms"], rb["norms"]):
        assert abs(x - y) < ntol * max(y, 1e-3), (ra, rb)
