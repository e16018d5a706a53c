"""amct_peer_barrier on one GPU: both ranks' flag arrays live on the same device and the peer's arrival is written by
the host beforehand, so no launch ever waits for another launch.  The time-out case waits for a flag that nothing
sets and must come back with status bit 1 and a usable context."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from amct_b200.backend import ops
    return ops


def test_barrier_passes_when_the_peer_has_arrived():
    mine = torch.zeros(2, dtype=torch.int32, device='cuda')
    peer = torch.zeros(2, dtype=torch.int32, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    for seq in (1, 2, 3):
        mine[1] = seq + (seq == 2)                   # the peer may already be one barrier ahead
        _ops().peer_barrier([mine.data_ptr(), peer.data_ptr()], 0, seq, status)
        torch.cuda.synchronize()
        assert peer.tolist() == [seq, 0]             # rank 0 signalled word [0] of the peer's array
        assert int(status.item()) == 0


def test_barrier_gives_up_and_reports():
    mine = torch.zeros(2, dtype=torch.int32, device='cuda')
    peer = torch.zeros(2, dtype=torch.int32, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    _ops().peer_barrier([mine.data_ptr(), peer.data_ptr()], 0, 1, status)
    t1.record()
    torch.cuda.synchronize()
    assert int(status.item()) & 2
    assert 1500 < t0.elapsed_time(t1) < 4000
    with pytest.raises(Exception):
        _ops().raise_if_timed_out(status)
    assert float(torch.ones(4, device='cuda').sum()) == 4.0          # the context is still usable


def test_single_rank_and_bad_arguments():
    from amct_b200.backend import lib
    flags = torch.zeros(1, dtype=torch.int32, device='cuda')
    _ops().peer_barrier([flags.data_ptr()], 0, 1, None)               # world 1: nothing to wait for, no launch
    with pytest.raises(lib.BackendError):
        _ops().peer_barrier([flags.data_ptr()] * 17, 0, 1, None)
    with pytest.raises(lib.BackendError):
        _ops().peer_barrier([flags.data_ptr(), 0], 0, 1, None)
