"""The replay's balanced-histogram selection must be bit-faithful to the online engine's plugin selection.

One process: ``replay.fused.shard_select_balanced`` on a flat score vector with per-parameter entries against
``plugins.selection._histogram.select_masks_histogram(mode="balanced", global_allreduce=False)`` on the
per-parameter views, over awkward geometries (odd sizes, one-element parameters, runs of equal values that land
inside the crossing bin) and several k: thresholds equal bit for bit, masks equal.

Sharded (gloo ranks, worlds 2 and 3): the shards' masks, put together in ``shard_bounds`` order, are the
one-shard mask and every rank reports the one-shard threshold: the per-parameter sampling grid, the catalog-wide
counts and the summed histogram rebuild the unsharded selection exactly.

The reference pins the same property in ``tests/test_selection_semantics_switch.py``.
"""
import math
import os
import socket
import struct
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sga_b200.plugins.selection._histogram import select_masks_histogram
from sga_b200.replay import fused as RF

GEOMETRIES = [
    (1, 7, 64, 1000, 3, 4097),          # one-element and odd-sized parameters
    (513, 8, 8, 8, 2049, 31),           # short parameters next to the sampling stride
    (5000,),                            # one parameter
    (9, 1, 1, 1, 1, 777, 12345),
]


def _bits(x: float) -> bytes:
    return struct.pack("<f", x)


def _scores(sizes, seed):
    g = torch.Generator().manual_seed(seed)
    n = sum(sizes)
    x = torch.randn(n, generator=g) * torch.logspace(-3, 1, n)[torch.randperm(n, generator=g)]
    # runs of equal magnitudes (both signs) so that some crossing bins are crowded, and exact zeros
    x[torch.randperm(n, generator=g)[:max(1, n // 10)]] = 0.0371
    x[torch.randperm(n, generator=g)[:max(1, n // 20)]] = -0.0371
    x[torch.randperm(n, generator=g)[:max(1, n // 50)]] = 0.0
    return x


def _info(sizes):
    offs, o = [], 0
    for s in sizes:
        offs.append(o)
        o += s
    return SimpleNamespace(offsets=offs, shapes=[(s,) for s in sizes], numel=o)


@pytest.mark.parametrize("sizes", GEOMETRIES)
def test_replay_balanced_select_equals_the_online_plugin(sizes):
    info = _info(sizes)
    for seed in (0, 1):
        x = _scores(sizes, seed)
        views = [x[o:o + s] for o, s in zip(info.offsets, sizes)]
        for k in sorted({1, max(1, info.numel // 100), max(1, info.numel // 5), info.numel // 2, info.numel}):
            thr_online, masks = select_masks_histogram(views, k, None, mode="balanced", global_allreduce=False)
            want = torch.cat([m.view(-1) for m in masks]).bool()
            sel, thr = RF.shard_select_balanced(x, k, RF.Comms(), RF.shard_entries(info, 0, info.numel),
                                                return_threshold=True)
            assert _bits(thr) == _bits(thr_online), (sizes, seed, k, thr, thr_online)
            assert torch.equal(sel, want), (sizes, seed, k)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _shard_worker(rank, world, port, sizes, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        info = _info(sizes)
        x = _scores(sizes, 4)
        lo, hi = RF.shard_bounds(info.numel, world, rank)
        comms = RF.Comms(rank, world, None, "cpu")
        res = {}
        for k in (1, info.numel // 100, info.numel // 5):
            sel, thr = RF.shard_select_balanced(x[lo:hi].clone(), k, comms, RF.shard_entries(info, lo, hi),
                                                return_threshold=True)
            res[k] = (lo, hi, sel, _bits(thr))
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_balanced_select_rebuilds_the_unsharded_one(tmp_path, world):
    sizes = (1001, 7, 4099, 3, 2500)   # not a multiple of 8, so shard cuts fall inside parameters and off the grid
    info = _info(sizes)
    x = _scores(sizes, 4)
    mp.spawn(_shard_worker, args=(world, _free_port(), sizes, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    for k in (1, info.numel // 100, info.numel // 5):
        one, thr1 = RF.shard_select_balanced(x, k, RF.Comms(), RF.shard_entries(info, 0, info.numel),
                                             return_threshold=True)
        whole = torch.zeros(info.numel, dtype=torch.bool)
        covered = 0
        for p in parts:
            lo, hi, sel, tb = p[k]
            assert lo == covered and sel.numel() == hi - lo
            whole[lo:hi] = sel
            covered = hi
            assert tb == _bits(thr1), (world, k)
        assert covered == info.numel
        assert torch.equal(whole, one), (world, k)
        assert math.isfinite(thr1)
