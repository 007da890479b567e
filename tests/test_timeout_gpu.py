"""A bounded device wait that runs out: the kernel returns, the host learns which wait gave up, and the next healthy
call works (the reference gives every wait a timeout and raises TimeoutError with a report, ferrite/runtime.py:466-484).
Nothing faults and nothing hangs: the wait's bound is set to ~50 ms for the test and the flag it waits for is simply
never written."""
import ctypes

import pytest
import torch

from ferrite_b200._lib import check, lib

pytestmark = pytest.mark.gpu


def test_a_rank_that_never_arrives_times_out_and_the_next_call_works(cuda):
    from ferrite_b200.tensor import Runtime
    rt = Runtime(0)
    n = 4096
    # "two ranks" on one GPU: this process is rank 0; rank 1 never runs, so nothing writes rank 0's flag word for it
    mine, theirs = torch.full((n,), 1.0, dtype=torch.bfloat16, device=cuda), torch.full((n,), 2.0, dtype=torch.bfloat16, device=cuda)
    flags0, flags1 = torch.zeros(8, dtype=torch.int32, device=cuda), torch.zeros(8, dtype=torch.int32, device=cuda)
    state = torch.zeros(4, dtype=torch.int32, device=cuda)
    state[3] = 100_000_000  # the wait's bound in clock cycles: ~50 ms instead of ~2 s
    out = torch.empty(n, dtype=torch.bfloat16, device=cuda)
    partials = (ctypes.c_void_p * 2)(mine.data_ptr(), theirs.data_ptr())
    flags = (ctypes.c_void_p * 2)(flags0.data_ptr(), flags1.data_ptr())
    call = lambda: check(lib().fb_peer_reduce_add(partials, flags, 0, 2, state.data_ptr(), n, None, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    rt.wait()  # (clears whatever an earlier test left)
    call()
    torch.cuda.synchronize()
    assert int(state[2]) == 202, "the wait for rank 1 gave up and said so"
    with pytest.raises(TimeoutError):
        rt.wait()  # the library's status word carries the same code to Runtime.wait
    rt.wait()      # read once, cleared
    # rank 1 "arrives" (its flag word for every call to come), the record of the time-out is cleared: a healthy call
    state[2] = 0
    flags0[1] = 1 << 20
    call()
    torch.cuda.synchronize()
    assert int(state[2]) == 0 and bool((out.float() == 3.0).all())
    rt.wait()


def test_peer_reduce_check_raises(cuda):
    # PeerReduce.check() turns the recorded code into the TimeoutError a caller sees
    from ferrite_b200.peer import PeerReduce
    peer = PeerReduce.__new__(PeerReduce)
    peer.state = torch.tensor([0, 0, 202, 0], dtype=torch.int32, device=cuda)
    with pytest.raises(TimeoutError, match="rank 1"):
        peer.check()
    peer.check()
