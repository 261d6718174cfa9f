"""The gated in-switch (NVLS) dense all-reduce: without a multicast mapping, or for a range that is not a
whole number of 16-byte groups, the wrapper declines before it touches the channel, and the caller's
peer-load kernel runs instead. (The kernel itself needs GPUs bound to an NVLink multicast object.)"""
from sga_b200.parallel import p2p
from sga_b200.runtime.ddp import DDPConfig
from sga_b200.runtime.trainer import build_parser


class _Buf:
    def __init__(self, mc_ptr):
        self.mc_ptr, self.local_ptr = mc_ptr, 1 << 20


class _Channel:
    def next_desc(self):
        raise AssertionError("a declined call must not consume a sequence number of the channel")


def test_wrapper_declines_without_launching():
    ch = _Channel()
    assert p2p.nvls_allreduce_(ch, _Buf(0), 0, 4096) is False            # not bound to a multicast object
    assert p2p.nvls_allreduce_(ch, _Buf(1 << 30), 0, 4098) is False      # not a multiple of four values
    assert p2p.nvls_allreduce_(ch, _Buf(1 << 30), 8, 4096) is False      # the range does not start on 16 bytes
    assert p2p.nvls_allreduce_(ch, object(), 0, 4096) is False           # a buffer of the plain pool


def test_option_is_off_by_default():
    assert DDPConfig().nvls_dense is False
    ns = build_parser().parse_args([])
    assert ns.nvls_dense is False
    assert build_parser().parse_args(["--nvls-dense"]).nvls_dense is True
