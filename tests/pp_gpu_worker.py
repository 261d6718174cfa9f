"""Worker for the pipeline-parallel GPU test (torchrun, one rank per GPU, two
stages): the staged model reproduces the unsplit model's gradients through
NCCL point-to-point transfers, and a staged SGA trainer trains. Prints
``PP_GPU_OK`` on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from sga_b200.models.gpt import GPT, get_config  # noqa: E402
from sga_b200.parallel.pp import Pipeline  # noqa: E402
from sga_b200.runtime.trainer import Trainer, default_args  # noqa: E402


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = get_config("llama_tiny", seq_len=256)
    stage = GPT(cfg, device=dev, seed=4, pp_size=world, pp_rank=rank)
    full = GPT(cfg, device=dev, seed=4)
    g = torch.Generator().manual_seed(8)
    n_micro = 3
    toks = torch.randint(0, cfg.vocab, (2 * n_micro, cfg.seq_len + 1), generator=g).to(dev)
    mbs = [(toks[2 * i:2 * i + 2, :-1], toks[2 * i:2 * i + 2, 1:]) for i in range(n_micro)]
    pipe = Pipeline(stage, pp_rank=rank, pp_size=world, prev_rank=rank - 1 if rank > 0 else None,
                    next_rank=rank + 1 if rank < world - 1 else None)
    losses = pipe.run(mbs, loss_scale=1.0 / n_micro)
    ref = [full.forward_backward(t, y, loss_scale=1.0 / n_micro) for t, y in mbs]
    torch.cuda.synchronize()
    if rank == world - 1:
        for a, b in zip(losses, ref):
            assert abs(float(a) - float(b)) < 5e-3 * max(1.0, float(b)), (float(a), float(b))
    for slot in stage.arena.slots:
        r = full.arena.by_name[slot.name].grad
        err = float((slot.grad - r).abs().max())
        assert err <= 0.08 * float(r.abs().max()) + 1e-6, (slot.name, err)
    del stage, full
    dist.barrier()
    tr = Trainer(default_args(model="llama_tiny", seq_length=256, micro_batch_size=2, global_batch_size=8, lr=1e-3,
                              pipeline_model_parallel_size=2, log_interval=0, sga_enabled=True, sga_score="abs_g",
                              sga_selection_method="exact", sga_selection_ratio_percent=5.0,
                              sga_backend="torch_pipelined_index", sga_selection_locality="rank_local",
                              sga_cycle_period=3, sga_bucket_elems=1 << 20,
                              untie_embeddings_and_output_weights=True), quiet=True)
    ls = [float(tr.train_step(tr.host_batch(0)).item()) for _ in range(6)]
    tr.check()
    assert ls[-1] < ls[0] and all(x == x for x in ls), ls
    tr.close()
    dist.barrier()
    if rank == 0:
        print("pp trainer losses", [round(x, 4) for x in ls])
        print("PP_GPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
