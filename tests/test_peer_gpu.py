"""Single-GPU checks of the peer-memory exchange kernels (the two-GPU run is in test_multi_gpu.py)."""
import ctypes as C

import pytest
import torch

from ffa_speedtest_b200 import _lib

pytestmark = pytest.mark.gpu


def test_world_of_one_merges_its_own_partial():
    """world = 1: the push only raises the rank's own flag and the merge returns the partial's rows."""
    rows = 64
    g = torch.zeros((2, 1, rows, 129), dtype=torch.float32, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    out = torch.empty((rows, 128), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    gp, fp = (C.c_void_p * 1)(g.data_ptr()), (C.c_void_p * 1)(flags.data_ptr())
    for step in (1, 2, 3):
        part = torch.randn(rows, 129, device="cuda")
        part[5, 128] = float("-inf")                       # a row whose rank kept nothing
        g[step & 1, 0] = part
        rc = _lib.lib().ffa_peer_exchange_merge(g[step & 1, 0].data_ptr(), rows, 0, 1, gp, fp, step, out.data_ptr(),
                                                _lib.float_code(out.dtype), status.data_ptr(),
                                                _lib.current_stream(out.device))
        assert rc == 0
        torch.cuda.synchronize()
        want = part[:, :128].to(torch.bfloat16)
        want[5] = 0
        assert torch.equal(out, want) and int(status[0]) == 0 and int(flags[0]) == step


def test_a_flag_that_nothing_raises_ends_in_a_status_word_not_a_hang():
    """Rank 1 of a world of two never pushes: the wait-and-merge kernel gives up after its one-second
    limit, sets the status word and writes NaN rows; the context stays usable."""
    rows = 8
    g = torch.zeros((2, 2, rows, 129), dtype=torch.float32, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[0] = 1                                           # this rank's own rows are there, the peer's never come
    out = torch.zeros((rows, 128), dtype=torch.float32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = _lib.lib().ffa_peer_wait_merge(g.data_ptr(), flags.data_ptr(), 2, rows, 1, out.data_ptr(),
                                        _lib.float_code(out.dtype), status.data_ptr(), _lib.current_stream(out.device))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status[0]) == 3 and bool(torch.isnan(out).all())
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0      # the device still answers


def test_bad_arguments_are_refused_before_any_launch():
    L = _lib.lib()
    z = (C.c_void_p * 1)(0)
    assert L.ffa_peer_exchange_merge(0, 8, 0, 1, z, z, 1, 0, 1, 0, 0) != 0
    assert L.ffa_peer_wait_merge(0, 0, 1, 8, 1, 0, 1, 0, 0) != 0
    t = torch.zeros(4096, dtype=torch.float32, device="cuda")
    assert L.ffa_peer_wait_merge(t.data_ptr(), t.data_ptr(), 17, 8, 1, t.data_ptr(), 3, 0, 0) != 0     # too many ranks
    assert L.ffa_peer_wait_merge(t.data_ptr(), t.data_ptr(), 2, 8, 0, t.data_ptr(), 3, 0, 0) != 0      # steps start at 1
