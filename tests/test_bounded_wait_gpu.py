"""A device-side wait that runs out must end by itself: the kernel returns, the error word says who
was missed, and the stream keeps working. Made to happen on the host side of the protocol only: a
two-rank flag barrier whose "peer" flag buffer is local memory that nothing ever writes, with the
wait limit set to 30 ms. No kernel faults, traps or spins without a limit."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def test_peer_barrier_wait_runs_out_and_the_stream_stays_usable(ops, cgb):
    import torch
    capi = cgb.capi
    L = cgb.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert ops.last_device_error() == 0                      # read-and-clear: start from a clean word
    mine = torch.zeros(8, dtype=torch.int64, device="cuda")      # this rank's flag buffer
    silent = torch.zeros(8, dtype=torch.int64, device="cuda")    # stands for rank 1's: nobody publishes into `mine`
    table = (C.c_void_p * 2)(mine.data_ptr(), silent.data_ptr())
    bar = C.c_void_p()
    capi.check(L.cg_b200_peer_barrier_create(C.byref(bar), table, 2, 0), "peer_barrier_create")
    try:
        assert L.cg_b200_peer_barrier_set_timeout(bar, 0) == capi.ERR_INVALID_ARG
        capi.check(L.cg_b200_peer_barrier_set_timeout(bar, 30_000_000), "set_timeout")
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        capi.check(L.cg_b200_peer_barrier(bar, stream), "peer_barrier")
        t1.record()
        torch.cuda.synchronize()
        waited_ms = t0.elapsed_time(t1)
        assert 25.0 <= waited_ms <= 500.0, f"the wait took {waited_ms:.1f} ms for a 30 ms limit"
        assert ops.last_device_error() == 0x501                 # rank 1 never arrived
        assert int(silent[0].item()) == 1                       # this rank did publish its epoch to the "peer"
        # the context and the stream are intact: the next launch runs and is correct
        x = torch.randn(4, 256, device="cuda")
        y = ops.softmax(x)
        torch.cuda.synchronize()
        assert torch.allclose(y.sum(dim=1), torch.ones(4, device="cuda"), atol=1e-5)
        assert ops.last_device_error() == 0
    finally:
        capi.check(L.cg_b200_peer_barrier_destroy(bar), "peer_barrier_destroy")
