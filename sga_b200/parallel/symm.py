"""Symmetric (peer-mapped) device memory for the in-kernel NVLink transport.

Every rank of a single-node process group allocates the same-sized buffer with
``cudaMalloc``, exports it as a CUDA IPC handle, and opens every peer's handle,
so a kernel on any rank can load from and store to every rank's copy with
plain pointers. Allocation happens once, at attach time; nothing on the
training path allocates. Handles travel over ``torch.distributed``
(``all_gather_object``), which stays the bootstrap plane.

This is the counterpart of the reference's communicator setup
(``sga/backends/torch_pipelined_index.py:180-233`` twin NCCL group + warm-up,
``sga/backends/nccl_pipelined_index.py:256-329`` raw ncclComm bootstrap).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import kernels as _kernels  # noqa: F401  (declares the argument types of every launcher: 64-bit sizes)
from ..csrc import lib

_DT_SIZE = {torch.float32: 4, torch.int32: 4, torch.bfloat16: 2, torch.uint8: 1, torch.int64: 8, torch.float16: 2}


def _tensor_from_ptr(ptr: int, nbytes: int, device) -> torch.Tensor:
    """A uint8 tensor aliasing ``nbytes`` of device memory at ``ptr`` (not owning)."""

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {
        "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
    }
    return torch.as_tensor(h, device=device)


@dataclass
class SymmBuffer:
    """One symmetric allocation: the local tensor plus every rank's base pointer."""

    nbytes: int
    local_ptr: int
    peer_ptrs: list            # base pointer of rank r's copy, as mapped into this process
    raw: torch.Tensor          # uint8 view of the local copy
    world: int
    rank: int
    _opened: list = field(default_factory=list)
    mc_ptr: int = 0            # the buffer through an NVLink multicast mapping (0: not bound to one)
    _keep: object = None       # what owns the memory when it did not come from sga_symm_alloc

    def view(self, dtype, offset_bytes: int = 0, numel: int | None = None) -> torch.Tensor:
        sz = _DT_SIZE[dtype]
        assert offset_bytes % sz == 0
        t = self.raw[offset_bytes:] if numel is None else self.raw[offset_bytes:offset_bytes + numel * sz]
        return t.view(dtype)

    def ptr_array(self, offset_bytes: int = 0):
        """``void*[8]`` of every rank's (base + offset), for a kernel argument."""
        arr = (ctypes.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.peer_ptrs[r] + offset_bytes
        return arr


class SymmPool:
    """Allocator of symmetric buffers over one process group (single node)."""

    def __init__(self, group=None, device=None):
        self.group = group
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        if self.world > 8:
            raise ValueError("the peer-memory transport covers one NVSwitch domain of at most 8 GPUs")
        self.buffers: list[SymmBuffer] = []

    def alloc(self, nbytes: int) -> SymmBuffer:
        nbytes = (int(nbytes) + 255) // 256 * 256
        L = lib()
        with torch.cuda.device(self.device):
            out = ctypes.c_void_p()
            rc = L.sga_symm_alloc(nbytes, ctypes.byref(out))
            if rc != 0:
                free, total = torch.cuda.mem_get_info(self.device)
                raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed (CUDA error {-rc}; "
                                   f"{free >> 20} MiB free of {total >> 20} MiB)")
            local = out.value
            peers = [local]
            opened = []
            if self.world > 1:
                handle = ctypes.create_string_buffer(64)
                if L.sga_ipc_get_handle(local, handle) != 0:
                    raise RuntimeError("cudaIpcGetMemHandle failed")
                gathered = [None] * self.world
                dist.all_gather_object(gathered, bytes(handle.raw), group=self.group)
                peers = []
                for r, hb in enumerate(gathered):
                    if r == self.rank:
                        peers.append(local)
                        continue
                    p = ctypes.c_void_p()
                    rc = L.sga_ipc_open(ctypes.create_string_buffer(hb, 64), ctypes.byref(p))
                    if rc != 0:
                        raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
                    peers.append(p.value)
                    opened.append(p.value)
                dist.barrier(group=self.group)
        buf = SymmBuffer(nbytes, local, peers, _tensor_from_ptr(local, nbytes, self.device), self.world, self.rank,
                         opened)
        self.buffers.append(buf)
        return buf

    def close(self) -> None:
        """Unmap peers and free local copies (between steps, nothing in flight)."""
        L = lib()
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self.buffers:
            for p in b._opened:
                L.sga_ipc_close(p)
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self.buffers:
            L.sga_symm_free(b.local_ptr)
        self.buffers = []


class McastPool(SymmPool):
    """Symmetric buffers that are also bound to an NVLink multicast object, so that a kernel can reduce
    a buffer inside the NVSwitch (``multimem.ld_reduce``) and broadcast through it (``multimem.st``).
    Allocation, the exchange of the handles and the multicast binding are ``torch.distributed``'s
    symmetric memory; this class only adapts its handles to :class:`SymmBuffer`. A buffer whose
    ``mc_ptr`` is 0 (no multicast support on this system) still has its peer pointers and serves the
    peer-load kernels unchanged.

    Gated: nothing takes this pool unless the trainer is started with ``--nvls-dense``. A rank that
    dies while its memory is bound to a multicast object can raise NVLink faults on the other ranks'
    GPUs, so failure tests must not run with it."""

    def __init__(self, group=None, device=None):
        super().__init__(group=group, device=device)
        import torch.distributed._symmetric_memory as symm_mem

        self._symm_mem = symm_mem
        self._handles = []

    def alloc(self, nbytes: int) -> SymmBuffer:
        nbytes = (int(nbytes) + 255) // 256 * 256
        if self.world == 1:
            return super().alloc(nbytes)
        sm = self._symm_mem
        with torch.cuda.device(self.device):
            t = sm.empty(nbytes, dtype=torch.uint8, device=self.device)
            t.zero_()
            torch.cuda.synchronize(self.device)
            group = self.group if self.group is not None else dist.group.WORLD
            hdl = sm.rendezvous(t, group=group)
        peers = [int(p) for p in hdl.buffer_ptrs]
        if len(peers) != self.world or peers[self.rank] != t.data_ptr():
            raise RuntimeError("symmetric-memory rendezvous returned an unexpected pointer table")
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        buf = SymmBuffer(nbytes, t.data_ptr(), peers, t, self.world, self.rank, [], mc_ptr=mc, _keep=(t, hdl))
        self.buffers.append(buf)
        self._handles.append(hdl)
        dist.barrier(group=self.group)
        return buf

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        own = [b for b in self.buffers if b._keep is None]
        self.buffers = own          # buffers of the framework's allocator are released with their tensors
        self._handles = []
        super().close()
