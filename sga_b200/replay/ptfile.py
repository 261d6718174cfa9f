"""Positional reads out of ``torch.save`` archives, without loading them.

A trace step file is a zip archive written by ``torch.save``: one pickle
(``<root>/data.pkl``) that describes every tensor as (storage key, offset,
shape, stride, dtype), and one *stored* (uncompressed) record per storage
(``<root>/data/<key>``). ``PtIndex`` parses the pickle with stand-in tensors,
so no storage is read, and records where each storage's bytes start in the
file. ``read_slice`` then copies any element range of a tensor straight from
the file descriptor into a caller-visible buffer with ``os.preadv``: the
kernel fills the buffer while the interpreter lock is released, nothing is
mapped, and a shard of a sharded replay reads exactly its own bytes.

This is the ``pread`` arm of the replay's gradient reader (the other arms map
the file or load it whole). The reference reads its traces the same way
(``sga/replay_fused.py:999``); the archive walk here is this framework's own.
"""
from __future__ import annotations

import os
import pickle
import struct
import zipfile
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

_STORAGE_DTYPES = {
    "FloatStorage": torch.float32, "DoubleStorage": torch.float64, "HalfStorage": torch.float16,
    "BFloat16Storage": torch.bfloat16, "LongStorage": torch.int64, "IntStorage": torch.int32,
    "ShortStorage": torch.int16, "CharStorage": torch.int8, "ByteStorage": torch.uint8, "BoolStorage": torch.bool,
}


@dataclass(frozen=True)
class TensorStub:
    """What the pickle says about one tensor; holds no data."""
    key: str
    dtype: torch.dtype
    offset: int          # elements into the storage
    shape: Tuple[int, ...]
    stride: Tuple[int, ...]

    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= int(d)
        return n

    def is_contiguous(self) -> bool:
        want = 1
        for d, s in zip(reversed(self.shape), reversed(self.stride)):
            if d != 1 and s != want:
                return False
            want *= int(d)
        return True


class _StorageTag:
    def __init__(self, name):
        self.dtype = _STORAGE_DTYPES[name]


def _rebuild_stub(storage, storage_offset, size, stride, *unused):
    key, dtype = storage
    return TensorStub(key=key, dtype=dtype, offset=int(storage_offset), shape=tuple(int(x) for x in size),
                      stride=tuple(int(x) for x in stride))


class _StubUnpickler(pickle.Unpickler):
    """Rebuilds the pickled object tree with ``TensorStub`` in place of every tensor. Only the
    handful of globals a trace file needs are resolvable; anything else is refused."""

    _PLAIN = {("collections", "OrderedDict"), ("builtins", "dict"), ("builtins", "list"), ("builtins", "tuple"),
              ("builtins", "set"), ("builtins", "int"), ("builtins", "float"), ("builtins", "str"),
              ("builtins", "bool"), ("builtins", "complex"), ("builtins", "bytes")}

    def find_class(self, module, name):
        if module == "torch._utils" and name in ("_rebuild_tensor_v2", "_rebuild_tensor"):
            return _rebuild_stub
        if module == "torch" and name in _STORAGE_DTYPES:
            return _StorageTag(name)
        if module == "torch" and name == "Size":
            return tuple
        if module == "torch" and isinstance(getattr(torch, name, None), torch.dtype):
            return getattr(torch, name)
        if (module, name) in self._PLAIN:
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"global {module}.{name} is not expected in a trace step file")

    def persistent_load(self, pid):
        # ('storage', storage type, key, location, element count)
        if not (isinstance(pid, tuple) and len(pid) >= 3 and pid[0] == "storage"):
            raise pickle.UnpicklingError(f"unknown persistent id {pid!r}")
        tag = pid[1]
        dtype = tag.dtype if isinstance(tag, _StorageTag) else torch.uint8
        return (str(pid[2]), dtype)


class PtIndex:
    """Object tree of one archive (tensors as stubs) and the file range of every storage record."""

    def __init__(self, path: str):
        self.path = path
        self.records: Dict[str, Tuple[int, int]] = {}   # storage key -> (first byte in the file, bytes)
        with zipfile.ZipFile(path) as z:
            pkl = [n for n in z.namelist() if n.endswith("/data.pkl") or n == "data.pkl"]
            if len(pkl) != 1:
                raise ValueError(f"{path}: not a torch.save archive (found {len(pkl)} data.pkl records)")
            root = pkl[0][:-len("data.pkl")]
            with z.open(pkl[0]) as fh:
                self.tree = _StubUnpickler(fh).load()
            with open(path, "rb") as raw:
                for zi in z.infolist():
                    if not zi.filename.startswith(root + "data/"):
                        continue
                    if zi.compress_type != zipfile.ZIP_STORED:
                        raise ValueError(f"{path}: record {zi.filename} is compressed; positional reads need stored records")
                    raw.seek(zi.header_offset)
                    head = raw.read(30)
                    if len(head) != 30 or head[:4] != b"PK\x03\x04":
                        raise ValueError(f"{path}: bad local header for {zi.filename}")
                    name_len, extra_len = struct.unpack("<HH", head[26:30])
                    self.records[zi.filename[len(root) + 5:]] = (zi.header_offset + 30 + name_len + extra_len,
                                                                 zi.file_size)

    def read_slice(self, fd: int, stub: TensorStub, first: int, count: int) -> torch.Tensor:
        """Elements ``[first, first + count)`` of the (contiguous) tensor ``stub`` as a 1-D tensor of its
        stored dtype, read from ``fd`` with positional reads. A slice that does not lie inside the
        tensor, or a tensor that does not lie inside its storage record, raises before any read."""
        if not stub.is_contiguous():
            raise ValueError(f"{self.path}: tensor of storage {stub.key} is not contiguous (stride {stub.stride})")
        if first < 0 or count < 0 or first + count > stub.numel():
            raise ValueError(f"{self.path}: slice [{first}, {first + count}) is outside a tensor of {stub.numel()} elements")
        if stub.key not in self.records:
            raise ValueError(f"{self.path}: no storage record {stub.key}")
        start, nbytes = self.records[stub.key]
        esz = torch.empty(0, dtype=stub.dtype).element_size()
        if (stub.offset + stub.numel()) * esz > nbytes:
            raise ValueError(f"{self.path}: storage record {stub.key} ({nbytes} bytes) is too short for its tensor")
        want = count * esz
        buf = bytearray(want)
        view = memoryview(buf)
        pos, got = start + (stub.offset + first) * esz, 0
        while got < want:
            r = os.preadv(fd, [view[got:]], pos + got)
            if r <= 0:
                raise OSError(f"{self.path}: short read at byte {pos + got} ({got} of {want})")
            got += r
        if want == 0:
            return torch.empty(0, dtype=stub.dtype)
        return torch.frombuffer(buf, dtype=stub.dtype)
