"""The ``-DSGA_BOUNDS`` debug library: an index outside the registered window
is counted and its access skipped; the production library reports that it
carries no checks."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounds_build_counts_and_skips_bad_indices():
    from sga_b200.csrc import build as B
    from sga_b200.csrc import lib

    path = os.path.join(os.path.dirname(B.__file__), "libsga_b200_bounds.so")
    if not os.path.exists(path):
        path = B.build(bounds=True)
    dbg = ctypes.CDLL(path)
    for fn in (dbg.sga_bounds_set_limit, dbg.sga_bounds_hits):
        fn.restype = ctypes.c_longlong
    dbg.sga_bounds_set_limit.argtypes = [ctypes.c_longlong]
    dbg.sga_scatter.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                ctypes.c_void_p]
    n = 1000
    # the buffer is larger than the registered window, so the stray index lands in owned memory either way
    dst = torch.zeros(2 * n, device="cuda")
    idx = torch.tensor([3, 17, n + 5, 999], dtype=torch.int32, device="cuda")
    vals = torch.ones(4, device="cuda")
    assert dbg.sga_bounds_set_limit(n) == 0
    st = torch.cuda.current_stream().cuda_stream
    assert dbg.sga_scatter(dst.data_ptr(), idx.data_ptr(), vals.data_ptr(), 4, 0, st) == 0
    torch.cuda.synchronize()
    assert dbg.sga_bounds_hits() == 1
    assert dbg.sga_bounds_hits() == 0  # read-and-clear
    assert float(dst.sum()) == 3.0 and float(dst[n + 5]) == 0.0
    prod = lib()
    prod.sga_bounds_hits.restype = ctypes.c_longlong
    assert prod.sga_bounds_hits() == -1
