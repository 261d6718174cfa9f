"""Token sources for the trainer.

``SyntheticTokens`` (in ``trainer.py``) draws uniform ids from a seed. ``TokenFile``
serves a pre-tokenised corpus from disk:

* ``PREFIX.bin`` + ``PREFIX.idx``: the indexed-dataset pair written by the
  Megatron-LM preprocessing tools (``--data-path PREFIX`` in the reference's
  yamls, ``examples/llama3/*.yaml`` there). Only the index header is read (the
  token dtype); the ``.bin`` file is the concatenation of every document's
  tokens and is memory-mapped.
* a bare ``FILE.bin`` / any other file: a flat array of token ids of
  ``--data-dtype`` (default ``int32``).

The stream is cut into windows of ``seq_len + 1`` tokens that start every
``seq_len`` tokens (the last token of a window is the first of the next, so
every token is predicted once). Sample ``g`` of the run is window
``perm_e[g % N]`` of epoch ``e = g // N``, with ``perm_e`` a permutation seeded
by ``(seed, e)``: the order depends on the seed only, so a global batch is the
same whatever the number of data-parallel ranks, and a resumed run continues
where it stopped.
"""
from __future__ import annotations

import os
import struct

import numpy as np
import torch

_IDX_MAGIC = b"MMIDIDX\x00\x00"
_IDX_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32,
               8: np.uint16}
_NAMED_DTYPES = {"uint16": np.uint16, "int32": np.int32, "uint32": np.uint32, "int64": np.int64}


def indexed_dataset_dtype(idx_path: str):
    """Token dtype recorded in a Megatron indexed-dataset ``.idx`` header."""
    with open(idx_path, "rb") as fh:
        if fh.read(9) != _IDX_MAGIC:
            raise ValueError(f"{idx_path} is not an indexed-dataset index (bad magic)")
        (version,) = struct.unpack("<Q", fh.read(8))
        if version != 1:
            raise ValueError(f"{idx_path}: unsupported index version {version}")
        (code,) = struct.unpack("<B", fh.read(1))
    if code not in _IDX_DTYPES or not np.issubdtype(_IDX_DTYPES[code], np.integer):
        raise ValueError(f"{idx_path}: dtype code {code} is not an integer token type")
    return _IDX_DTYPES[code]


class TokenFile:
    """Windows of a memory-mapped token stream; same ``batch`` contract as ``SyntheticTokens``."""

    def __init__(self, path: str, vocab: int, seq_len: int, seed: int, global_batch: int, dtype: str | None = None,
                 pin: bool = False):
        prefix = path[:-4] if path.endswith((".bin", ".idx")) else path
        bin_path = prefix + ".bin" if os.path.exists(prefix + ".bin") else path
        if not os.path.exists(bin_path):
            raise FileNotFoundError(f"--data-path: neither {prefix}.bin nor {path} exists")
        if dtype is not None:
            np_dtype = _NAMED_DTYPES[dtype]
        elif os.path.exists(prefix + ".idx"):
            np_dtype = indexed_dataset_dtype(prefix + ".idx")
        else:
            np_dtype = np.int32
        self.tokens = np.memmap(bin_path, dtype=np_dtype, mode="r")
        self.vocab, self.seq_len, self.seed, self.global_batch, self.pin = vocab, seq_len, seed, global_batch, pin
        self.num_samples = (len(self.tokens) - 1) // seq_len
        if self.num_samples < 1:
            raise ValueError(f"{bin_path} holds {len(self.tokens)} tokens: fewer than one sequence of {seq_len} + 1")
        self._perm_epoch, self._perm = -1, None

    def _order(self, epoch: int) -> torch.Tensor:
        if epoch != self._perm_epoch:
            g = torch.Generator().manual_seed(self.seed * 1000003 + epoch)
            self._perm, self._perm_epoch = torch.randperm(self.num_samples, generator=g), epoch
        return self._perm

    def batch(self, step: int, first_sample: int, n: int) -> torch.Tensor:
        """``n`` sequences starting at sample ``first_sample`` of the global batch of ``step``."""
        out = torch.empty(n, self.seq_len + 1, dtype=torch.int64, pin_memory=self.pin)
        base = step * self.global_batch + first_sample
        for i in range(n):
            epoch, at = divmod(base + i, self.num_samples)
            start = int(self._order(epoch)[at]) * self.seq_len
            window = np.asarray(self.tokens[start:start + self.seq_len + 1]).astype(np.int64)
            out[i] = torch.from_numpy(window)
        if int(out.max()) >= self.vocab or int(out.min()) < 0:
            raise ValueError(f"token id outside [0, {self.vocab}) in the data at step {step}: wrong --data-dtype, or a "
                             "corpus tokenised for another vocabulary")
        return out
