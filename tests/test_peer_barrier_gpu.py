"""The bounded flag barrier of the head-parallel exchange, on one GPU.

With one rank the barrier completes at once.  With a second "rank" that never announces
itself (its flag array is a buffer nothing writes) the wait runs out after the given
time, the status word is set and the kernel returns: the context stays usable.  Nothing
faults or hangs; no second process is involved."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _barrier(lib, flags, rank, epoch, status, timeout_ms):
    from anchor_attention_b200 import _lib
    b = _lib.AAPeerBarrier()
    b.n_peers, b.rank, b.epoch, b.timeout_ms = len(flags), rank, epoch, timeout_ms
    for i, f in enumerate(flags):
        b.flags[i] = f.data_ptr()
    b.status = status.data_ptr()
    return lib.aa_peer_barrier(ctypes.byref(b), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_single_rank_barrier_passes(lib):
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda")]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        assert _barrier(lib, flags, 0, epoch, status, 1000) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(flags[0][0]) == 3


def test_missing_peer_times_out_and_context_survives(lib):
    mine = torch.zeros(8, dtype=torch.int32, device="cuda")
    absent = torch.zeros(8, dtype=torch.int32, device="cuda")      # the peer's array: we announce there, it never does here
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    assert _barrier(lib, [mine, absent], 0, 1, status, 50) == 0
    t1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert 40 <= t0.elapsed_time(t1) < 2000
    assert int(absent[0]) == 1 and int(mine[0]) == 1 and int(mine[1]) == 0
    # the peer "arrives" (its announcement written by hand): the same epoch now passes
    status.zero_()
    mine[1] = 1
    assert _barrier(lib, [mine, absent], 0, 1, status, 50) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # and the context still computes
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_barrier_argument_checks(lib):
    from anchor_attention_b200 import _lib
    b = _lib.AAPeerBarrier()
    assert lib.aa_peer_barrier(None, None) == -1
    b.n_peers, b.rank = 2, 0
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -1            # no status word
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    b.status = status.data_ptr()
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -1            # NULL flag arrays
    b.n_peers = 9
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -2
    b.n_peers, b.rank = 2, 2
    assert lib.aa_peer_barrier(ctypes.byref(b), None) == -2
