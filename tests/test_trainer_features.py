"""Trainer features around the step: token-file data source, learning-rate schedule, validation pass."""
import struct

import numpy as np
import pytest
import torch

from sga_b200.runtime.data import TokenFile, indexed_dataset_dtype
from sga_b200.runtime.trainer import Trainer, default_args


def _write_pair(prefix, tokens, code=8, dtype=np.uint16):
    np.asarray(tokens, dtype=dtype).tofile(str(prefix) + ".bin")
    with open(str(prefix) + ".idx", "wb") as fh:  # header of the indexed-dataset index: magic, version, dtype code
        fh.write(b"MMIDIDX\x00\x00" + struct.pack("<Q", 1) + struct.pack("<B", code) + struct.pack("<QQ", 1, 1))


def test_index_header_and_windows(tmp_path):
    n, seq = 1000, 16
    toks = np.arange(n) % 500
    _write_pair(tmp_path / "corpus", toks)
    assert indexed_dataset_dtype(str(tmp_path / "corpus.idx")) == np.uint16
    ds = TokenFile(str(tmp_path / "corpus"), vocab=512, seq_len=seq, seed=7, global_batch=8)
    assert ds.num_samples == (n - 1) // seq
    b = ds.batch(0, 0, 8)
    assert b.shape == (8, seq + 1) and b.dtype == torch.int64
    starts = set()
    for row in b:
        d = (row[1:] - row[:-1]) % 500
        assert bool((d == 1).all()), "a window is a contiguous run of the stream"
        starts.add(int(row[0]))
    assert len(starts) == 8, "distinct windows within a batch"
    # the order depends on the seed only: two ranks' halves are the one-rank batch, and a resume repeats it
    again = TokenFile(str(tmp_path / "corpus.bin"), vocab=512, seq_len=seq, seed=7, global_batch=8)
    assert torch.equal(torch.cat([again.batch(0, 0, 4), again.batch(0, 4, 4)]), b)
    assert not torch.equal(TokenFile(str(tmp_path / "corpus"), 512, seq, 8, 8).batch(0, 0, 8), b)
    # an epoch visits every window once; the next epoch reshuffles
    per_epoch = ds.num_samples
    seen = [int(ds.batch(s, 0, 1)[0, 0]) for s in range(0, per_epoch * 8, 8)]
    first = torch.cat([ds.batch(s, 0, 8) for s in range((per_epoch + 7) // 8)])[:per_epoch, 0]
    assert len(set(first.tolist())) == per_epoch and len(seen) == per_epoch


def test_flat_file_dtype_and_vocab_check(tmp_path):
    np.arange(300, dtype=np.int32).tofile(str(tmp_path / "flat.bin"))
    ds = TokenFile(str(tmp_path / "flat.bin"), vocab=1000, seq_len=8, seed=1, global_batch=2)
    assert int(ds.batch(0, 0, 2).max()) < 300
    with pytest.raises(ValueError, match="outside"):
        TokenFile(str(tmp_path / "flat.bin"), vocab=100, seq_len=8, seed=1, global_batch=2).batch(0, 0, 37)
    with pytest.raises(ValueError, match="fewer than one sequence"):
        TokenFile(str(tmp_path / "flat.bin"), vocab=1000, seq_len=4096, seed=1, global_batch=2)
    with pytest.raises(FileNotFoundError):
        TokenFile(str(tmp_path / "absent"), vocab=10, seq_len=8, seed=1, global_batch=2)
    (tmp_path / "bad.idx").write_bytes(b"not an index")
    with pytest.raises(ValueError, match="bad magic"):
        indexed_dataset_dtype(str(tmp_path / "bad.idx"))


def test_trainer_reads_the_corpus(tmp_path):
    tr0 = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=4, train_iters=2, device="cpu",
                               log_interval=0), quiet=True)
    vocab, seq = tr0.cfg.vocab, tr0.cfg.seq_len
    tr0.close()
    g = torch.Generator().manual_seed(0)
    _write_pair(tmp_path / "c", torch.randint(0, vocab, (seq * 40 + 1,), generator=g).numpy(), code=4, dtype=np.int32)
    tr = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=4, train_iters=2, device="cpu",
                              log_interval=0, data_path=str(tmp_path / "c")), quiet=True)
    b = tr.host_batch(0)
    assert b.shape == (4, seq + 1) and int(b.max()) < vocab
    loss = tr.train_step(b)
    assert torch.isfinite(loss)
    tr.close()


def test_learning_rate_schedule():
    from sga_b200.runtime.trainer import scheduled_lr

    a = default_args(lr=1e-3, min_lr=1e-4, lr_decay_style="cosine", lr_warmup_iters=10, train_iters=110)
    assert scheduled_lr(a, 0) == 0.0 and scheduled_lr(a, 5) == pytest.approx(5e-4) and scheduled_lr(a, 10) == 1e-3
    assert scheduled_lr(a, 60) == pytest.approx(1e-4 + 0.5 * 9e-4) and scheduled_lr(a, 110) == pytest.approx(1e-4)
    assert scheduled_lr(a, 500) == 1e-4
    lin = default_args(lr=1e-3, min_lr=0.0, lr_decay_style="linear", lr_warmup_iters=0, lr_decay_iters=100, train_iters=200)
    assert scheduled_lr(lin, 25) == pytest.approx(7.5e-4) and scheduled_lr(lin, 150) == 0.0
    assert scheduled_lr(default_args(lr=3e-4), 12345) == 3e-4
    # the trainer applies it before every step, and the trace / checkpoint see the scheduled value
    tr = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=2, train_iters=8, device="cpu",
                              log_interval=0, lr=1e-3, lr_warmup_iters=4), quiet=True)
    seen = []
    for s in range(6):
        tr.train_step(tr.host_batch(s))
        seen.append(tr.optimizer.param_groups[0]["lr"])
    assert seen == pytest.approx([0.0, 2.5e-4, 5e-4, 7.5e-4, 1e-3, 1e-3])
    tr.close()


def test_validation_pass_leaves_training_state_alone(capsys):
    tr = Trainer(default_args(model="test_tiny", micro_batch_size=2, global_batch_size=4, train_iters=4, device="cpu",
                              log_interval=0), quiet=True)
    tr.train_step(tr.host_batch(0))
    w, g, m = (t.clone() for t in (tr.model.arena.main_param, tr.model.arena.main_grad, tr.model.arena.exp_avg))
    v1 = tr.evaluate(2)
    assert v1 == tr.evaluate(2) and 0.0 < v1 < 20.0
    assert all(torch.equal(a, b) for a, b in ((w, tr.model.arena.main_param), (g, tr.model.arena.main_grad),
                                              (m, tr.model.arena.exp_avg)))
    tr.close()
    from sga_b200 import train_gpt

    assert train_gpt.main(["--model", "test_tiny", "--micro-batch-size", "2", "--global-batch-size", "2",
                           "--train-iters", "4", "--device", "cpu", "--log-interval", "0", "--eval-interval", "2",
                           "--eval-iters", "1"]) == 0
    out = capsys.readouterr().out
    assert out.count("validation loss at iteration") == 2


def test_warmup_fraction_and_exit_interval(tmp_path, capsys):
    from sga_b200 import train_gpt
    from sga_b200.runtime.trainer import scheduled_lr

    a = default_args(lr=1e-3, lr_decay_style="linear", lr_warmup_fraction=0.1, train_iters=100)
    assert scheduled_lr(a, 5) == pytest.approx(5e-4) and scheduled_lr(a, 10) == 1e-3
    with pytest.raises(ValueError, match="not both"):
        scheduled_lr(default_args(lr=1e-3, lr_warmup_fraction=0.1, lr_warmup_iters=3, train_iters=100), 1)
    argv = ["--model", "test_tiny", "--micro-batch-size", "2", "--global-batch-size", "2", "--train-iters", "6",
            "--device", "cpu", "--log-interval", "0", "--save", str(tmp_path), "--exit-interval", "4"]
    assert train_gpt.main(argv) == 0
    assert "exiting at iteration 4" in capsys.readouterr().out
    assert open(tmp_path / "latest_checkpointed_iteration.txt").read().strip() == "4"
    assert train_gpt.main(argv + ["--load", str(tmp_path)]) == 0   # resumes at 4, runs to 6
    assert open(tmp_path / "latest_checkpointed_iteration.txt").read().strip() == "6"


def test_architecture_flags_override_the_preset():
    tr = Trainer(default_args(model="test_tiny", num_layers=1, hidden_size=64, ffn_hidden_size=128,
                              num_attention_heads=4, num_query_groups=2, padded_vocab_size=320, rotary_base=1e6,
                              norm_epsilon=1e-6, qk_layernorm=True, micro_batch_size=2, global_batch_size=2,
                              train_iters=2, device="cpu", log_interval=0), quiet=True)
    c = tr.cfg
    assert (c.hidden, c.ffn, c.n_heads, c.n_kv_heads, c.head_dim, c.vocab) == (64, 128, 4, 2, 16, 320)
    assert c.rope_theta == 1e6 and c.norm_eps == 1e-6 and c.qk_norm and c.num_layers == 1
    assert torch.isfinite(tr.train_step(tr.host_batch(0)))
    tr.close()
    with pytest.raises(ValueError, match="multiple of"):
        Trainer(default_args(model="test_tiny", num_attention_heads=4, num_query_groups=3, device="cpu"), quiet=True)


@pytest.mark.parametrize("sga", [
    dict(sga_score="abs_m", sga_selection_method="histogram", sga_selection_histogram_mode="balanced",
         sga_backend="torch_pipelined_index", sga_cycle_period=4),
    dict(sga_score="update", sga_selection_method="adaptive", sga_backend="torch_pipelined_mask", sga_cycle_period=3,
         sga_optimizer_residual_mean=True),
    dict(sga_score="abs_g", sga_selection_method="exact", sga_backend="torch_pipelined_index",
         sga_selection_locality="rank_local", sga_cycle_period=0),
])
def test_saved_sga_state_resumes_bit_for_bit(tmp_path, monkeypatch, sga):
    """With --save-sga-state a run stopped in the middle of a cycle and resumed ends with the weights, moments
    and residual of the uninterrupted run, bit for bit; without it the resumed engine cold-starts and differs."""
    from sga_b200 import train_gpt

    monkeypatch.setenv("SGA_ALLOW_FROZEN_SELECTION", "1")
    flags = ["--model", "test_tiny", "--micro-batch-size", "2", "--global-batch-size", "2", "--device", "cpu",
             "--log-interval", "0", "--sga-enabled", "true", "--sga-selection-ratio-percent", "10"]
    for k, v in sga.items():
        flags += ["--" + k.replace("_", "-"), str(v).lower() if isinstance(v, bool) else str(v)]
    final, now = {}, {"tag": None}
    stock_close = Trainer.close

    def close(self):
        a = self.model.arena
        final[now["tag"]] = (a.main_param.clone(), a.exp_avg.clone(), a.main_grad.clone())
        return stock_close(self)

    monkeypatch.setattr(Trainer, "close", close)

    def run(tag, argv):
        now["tag"] = tag
        assert train_gpt.main(flags + argv) == 0

    run("whole", ["--train-iters", "11"])
    for tag, extra in (("warm", ["--save-sga-state"]), ("cold", [])):
        d = str(tmp_path / tag)
        run("first_" + tag, ["--train-iters", "6", "--save", d] + extra)
        run(tag, ["--train-iters", "11", "--load", d] + extra)
    assert all(torch.equal(a, b) for a, b in zip(final["whole"], final["warm"]))
    assert not torch.equal(final["whole"][0], final["cold"][0])


def test_tensorboard_scalars(tmp_path):
    pytest.importorskip("tensorboard")
    from sga_b200 import train_gpt

    assert train_gpt.main(["--model", "test_tiny", "--micro-batch-size", "2", "--global-batch-size", "2",
                           "--train-iters", "3", "--device", "cpu", "--log-interval", "1", "--tensorboard-dir",
                           str(tmp_path / "tb"), "--eval-interval", "3", "--eval-iters", "1"]) == 0
    from tensorboard.backend.event_processing.event_accumulator import EventAccumulator

    acc = EventAccumulator(str(tmp_path / "tb"))
    acc.Reload()
    tags = set(acc.Tags()["scalars"])
    assert {"lm loss", "grad-norm", "learning-rate", "lm loss validation"} <= tags
    assert [e.step for e in acc.Scalars("lm loss")] == [1, 2, 3]
