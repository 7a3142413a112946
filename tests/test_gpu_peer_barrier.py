"""The cross-GPU barrier's failure path, exercised on one GPU without any fault: a barrier whose
peer never arrives (a flag that nothing sets) must give up after its bounded wait, record
AICI_STATUS_WAIT_TIMEOUT and leave the context usable; one whose peer has arrived passes at once."""
import ctypes
import time

import pytest
import torch

from aici_b200 import _lib

pytestmark = pytest.mark.gpu
WAIT_TIMEOUT = 4


def _barrier(flags, rank):
    ptrs = (ctypes.c_void_p * len(flags))(*[f.data_ptr() for f in flags])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check("aici_peer_barrier", _lib.lib().aici_peer_barrier(ptrs, ctypes.c_int(len(flags)),
                                                                 ctypes.c_int(rank), stream))


def test_barrier_passes_when_the_peer_has_arrived(cuda_device):
    mine = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    peer = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    mine[1] = 3  # "rank 1" already published epochs 1..3 into rank 0's array
    for epoch in (1, 2, 3):
        t0 = time.perf_counter()
        _barrier([mine, peer], 0)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        assert int(peer[0]) == epoch and int(mine[0]) == epoch and int(mine[8]) == epoch
    assert _lib.last_status() == 0


def test_barrier_gives_up_after_its_bounded_wait(cuda_device):
    mine = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    peer = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    t0 = time.perf_counter()
    _barrier([mine, peer], 0)  # nobody will ever write mine[1]
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.2 < waited < 10.0, waited
    assert _lib.last_status() & WAIT_TIMEOUT
    assert _lib.last_status() == 0  # reading clears the word
    # the kernel returned normally: the context works and a later barrier can succeed
    mine[1] = 100
    _barrier([mine, peer], 0)
    torch.cuda.synchronize()
    assert _lib.last_status() == 0
    assert float(torch.ones(8, device=cuda_device).sum()) == 8.0


def test_barrier_rejects_bad_arguments(cuda_device):
    mine = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    with pytest.raises(_lib.AiciError, match="world must be 1..8"):
        _barrier([mine] * 9, 0)
    with pytest.raises(_lib.AiciError, match="rank inside it"):
        _barrier([mine, mine], 2)
