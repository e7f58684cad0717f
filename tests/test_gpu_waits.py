"""The bounded device-side waits give up, report and leave the context usable.

Nothing here faults, traps or hangs a GPU: a wait is given a limit of a few milliseconds and a
condition that nothing will ever satisfy (a barrier phase nobody completes; a peer flag nobody
sets), runs out, writes the status words and the kernel returns normally."""

import ctypes as C

import pytest
import torch

from oracle import trimul_oracle as O
from tests._util import forward_kwargs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from miniworld_engine_b200 import _lib
    return _lib, _lib.load(), torch.device("cuda", 0)


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def test_an_expiring_barrier_wait_reports_and_returns(env):
    _lib, lib, dev = env
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.trimul_b200_selftest_expiring_wait(3000, _stream(dev), st.data_ptr()) == _lib.OK
    t1.record()
    torch.cuda.synchronize(dev)
    assert st.tolist() == [_lib.E_DEVICE_TIMEOUT, 10, 0, 1077]        # code, stage, block, detail (+1000: tear-down ran)
    assert 2.5 <= t0.elapsed_time(t1) < 200.0                         # it waited about as long as asked, not a second
    # the context is intact: a block call right after is correct
    from miniworld_engine_b200 import read_status, trimul_forward
    w, z = O.make_weights(128, 0), O.make_input(1, 40, 128, 1)
    y = trimul_forward(z.bfloat16().to(dev), None, outgoing=True, **forward_kwargs(w, torch.bfloat16, dev))
    ref = O.trimul_forward(z.bfloat16(), None, w.to(torch.bfloat16), True)
    assert O.rel_rms(y.float().cpu(), ref.float()) <= 1e-2
    assert read_status(dev)[0] == 0


def test_the_cross_gpu_barrier_gives_up_when_a_rank_never_arrives(env):
    _lib, lib, dev = env
    mine = torch.zeros(2, dtype=torch.int32, device=dev)       # this rank's flag array
    peer = torch.zeros(2, dtype=torch.int32, device=dev)       # stands in for a peer that never runs
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), peer.data_ptr())
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    assert lib.trimul_b200_peer_barrier(0, 2, ptrs, 1, 2000, _stream(dev), st.data_ptr()) == _lib.OK
    torch.cuda.synchronize(dev)
    assert st.tolist() == [_lib.E_DEVICE_TIMEOUT, 9, 1, 1]     # stage 9 = barrier, rank 1 missing, epoch 1
    assert mine.tolist() == [1, 0] and peer.tolist() == [1, 0] # our own arrival was published to both arrays
    # the same barrier completes once the peer's word is there (set here by hand), and stays silent
    st.zero_()
    mine[1] = 2
    assert lib.trimul_b200_peer_barrier(0, 2, ptrs, 2, 2000, _stream(dev), st.data_ptr()) == _lib.OK
    torch.cuda.synchronize(dev)
    assert st.tolist() == [0, 0, 0, 0] and peer.tolist() == [2, 0]
    # a one-rank group never waits
    solo = torch.zeros(1, dtype=torch.int32, device=dev)
    p1 = (C.c_void_p * 1)(solo.data_ptr())
    for epoch in (1, 2, 3):
        assert lib.trimul_b200_peer_barrier(0, 1, p1, epoch, 2000, _stream(dev), st.data_ptr()) == _lib.OK
    torch.cuda.synchronize(dev)
    assert st.tolist() == [0, 0, 0, 0] and solo.tolist() == [3]
