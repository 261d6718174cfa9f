"""``sga_compact_mask_noalloc``: the mask-compaction entry point for hosts that
cannot allocate device memory (everything on the GPU already belongs to their
own arena, or an allocation's implicit synchronisation is not acceptable, or
they are only handed input and output buffers). Its work array is built into
the library, so the caller passes inputs and outputs only.

The test calls the exported C symbol directly, the way such a host would, and
checks it against ``sga_compact_mask`` (which takes a caller-supplied work
array) on two calls in a row. The second mask is shorter and sparser than the
first, so stale contents of the shared work array would show. Collected last
(file name) so a run that stops at the first failure has run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_ELEMS = 65536 * 4096
E_TOO_LARGE = -8


def _lib():
    from sga_b200.csrc import lib

    L = lib()
    fn = L.sga_compact_mask_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    ref = L.sga_compact_mask
    ref.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                    ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    ref.restype = ctypes.c_int
    return fn, ref


def _run_both(fn, ref, mask):
    n = mask.numel()
    stream = torch.cuda.current_stream().cuda_stream
    idx_a = torch.full((n,), -1, dtype=torch.int32, device=DEV)
    idx_b = torch.full((n,), -1, dtype=torch.int32, device=DEV)
    tot_a = torch.zeros(1, dtype=torch.int64, device=DEV)
    tot_b = torch.zeros(1, dtype=torch.int64, device=DEV)
    err_a = torch.zeros(1, dtype=torch.int32, device=DEV)
    err_b = torch.zeros(1, dtype=torch.int32, device=DEV)
    work = torch.empty((n + 4095) // 4096, dtype=torch.int32, device=DEV)  # only the existing entry point needs it
    assert ref(mask.data_ptr(), n, work.data_ptr(), idx_b.data_ptr(), n, tot_b.data_ptr(), err_b.data_ptr(),
               stream) == 0
    assert fn(mask.data_ptr(), n, idx_a.data_ptr(), n, tot_a.data_ptr(), err_a.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(err_a.item()) == 0 and int(err_b.item()) == 0
    assert int(tot_a.item()) == int(tot_b.item()) == int(mask.sum().item())
    assert torch.equal(idx_a, idx_b)  # integer output: exact
    k = int(tot_a.item())
    assert torch.equal(idx_a[:k].long(), torch.nonzero(mask).view(-1))


def test_noalloc_matches_existing_entry_point_twice_in_a_row():
    fn, ref = _lib()
    g = torch.Generator(device="cpu").manual_seed(11)
    first = (torch.rand(3 * 4096 * 50 + 123, generator=g) < 0.30).to(torch.uint8).to(DEV)
    second = (torch.rand(4096 * 7 + 5, generator=g) < 0.02).to(torch.uint8).to(DEV)
    _run_both(fn, ref, first)
    _run_both(fn, ref, second)


def test_noalloc_refuses_masks_beyond_its_limit():
    fn, _ = _lib()
    # nothing is launched or dereferenced on refusal, so no buffers are needed
    rc = fn(None, MAX_ELEMS + 1, None, 0, None, None, None)
    assert rc == E_TOO_LARGE
    x = torch.ones(4, device=DEV)
    assert float(x.sum().item()) == 4.0


def test_noalloc_refuses_a_mask_off_the_16_byte_boundary():
    fn, _ = _lib()
    buf = torch.zeros(4096 + 16, dtype=torch.uint8, device=DEV)
    idx = torch.empty(64, dtype=torch.int32, device=DEV)
    tot = torch.zeros(1, dtype=torch.int64, device=DEV)
    # refused on the host before any launch: a misaligned 16-byte load would fault the context
    rc = fn(buf.data_ptr() + 3, 4096, idx.data_ptr(), 64, tot.data_ptr(), None, None)
    assert rc == -10
    torch.cuda.synchronize()
    assert int(tot.item()) == 0
