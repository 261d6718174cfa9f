"""Tensor parallelism on CPU (gloo, 2 ranks): the sharded model with
sequence-parallel activations reproduces the unsharded model's loss and
gradients, shard by shard, and replicated parameters end with the full
gradient on every rank."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sga_b200.models.gpt import GPT, get_config, param_specs
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


def _worker(rank, world, port, preset, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = get_config(preset)
        tp = TPContext(device="cpu")
        model = GPT(cfg, device="cpu", seed=3, tp=tp)
        full = GPT(cfg, device="cpu", seed=3)
        # same seed -> the shard is cut from the same full tensors
        for slot in model.arena.slots:
            ref = _shard_of(full.arena.by_name[slot.name].main, slot.spec)
            assert torch.equal(slot.main, ref), slot.name
        g = torch.Generator().manual_seed(11)
        B, S = 2, cfg.seq_len
        toks = torch.randint(0, cfg.vocab, (B, S + 1), generator=g)
        loss_tp = model.forward_backward(toks[:, :-1], toks[:, 1:])
        loss_full = full.forward_backward(toks[:, :-1], toks[:, 1:])
        assert abs(float(loss_tp) - float(loss_full)) < 2e-3 * max(1.0, abs(float(loss_full)))
        worst = 0.0
        for slot in model.arena.slots:
            ref = _shard_of(full.arena.by_name[slot.name].grad, slot.spec)
            err = float((slot.grad - ref).abs().max())
            scale = float(ref.abs().max()) + 1e-8
            worst = max(worst, err / scale)
            assert err <= 0.06 * scale + 1e-6, (slot.name, err, scale)
        if rank == 0:
            torch.save({"worst": worst}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("preset", ["test_tiny", "test_tiny_qk"])
def test_tp2_matches_unsharded_model(tmp_path, preset):
    out = str(tmp_path / "r.pt")
    mp.spawn(_worker, args=(2, _free_port(), preset, out), nprocs=2, join=True)
    assert torch.load(out)["worst"] < 0.06


def test_tp_specs_cover_the_full_tensors():
    cfg = get_config("test_tiny")
    full = {s.name: s for s in param_specs(cfg)}
    shards = [param_specs(cfg, 2, r) for r in range(2)]
    for name, fs in full.items():
        parts = [next(s for s in sh if s.name == name) for sh in shards]
        if parts[0].tp_pieces is None:
            assert parts[0].tp_duplicate and parts[0].shape == fs.shape
            continue
        assert parts[0].tp_full_shape == fs.shape
        dim = parts[0].tp_pieces[0][0]
        covered = sorted((lo, hi) for p in parts for _, lo, hi in p.tp_pieces)
        pos = 0
        for lo, hi in covered:
            assert lo == pos
            pos = hi
        assert pos == fs.shape[dim]
