"""A device-side wait that nobody satisfies gives up: the kernel ends, reports status 2 and leaves its outputs alone.

One GPU plays rank 0 of a two-rank group whose "peer" buffers are ordinary local memory that no other rank ever
writes, with the wait limit shortened to about a millisecond (``state[2]``, in units of 1024 clock cycles).  Nothing
here faults or hangs: the wait simply runs out.  The reference reports a stuck collective the same way, as an error the
host reads (singe-nccl/src/communicator/mod.rs:401-480, ``async_error``).
"""
import ctypes

import pytest
import torch

from singe_b200 import kernel_sys as ks

pytestmark = pytest.mark.gpu

ROWS, WIDTH, EPS = 8, 1024, 1e-5


def _pointers(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _setup():
    generator = torch.Generator(device="cuda").manual_seed(3)
    hidden = torch.randn((ROWS, WIDTH), generator=generator, device="cuda").to(torch.bfloat16)
    weight = torch.ones(WIDTH, dtype=torch.bfloat16, device="cuda")
    partial = torch.randn((ROWS, WIDTH), generator=generator, device="cuda").to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return hidden, weight, partial, status


def test_one_shot_all_reduce_gives_up_on_a_peer_that_never_signals():
    lib = ks.lib()
    hidden, weight, partial, status = _setup()
    before = hidden.clone()
    normed = torch.full_like(hidden, 7.0)
    silent_peer = torch.zeros_like(partial)
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    state[2] = 1500  # 1.5 M cycles: about a millisecond
    stream = int(torch.cuda.current_stream().cuda_stream)
    code = lib.singe_allreduce_add_rms_norm_bf16(stream, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(),
                                                 _pointers([partial, silent_peer]), _pointers(flags),
                                                 state.data_ptr(), 0, 2, ROWS, WIDTH, EPS, status.data_ptr())
    assert code == ks.OK
    torch.cuda.synchronize()  # returns: the wait ran out instead of spinning on
    assert int(status.item()) == ks.STATUS_WAIT_TIMEOUT
    assert torch.equal(hidden, before) and bool((normed == 7.0).all())
    # the context is intact: a complete group (one rank) runs normally afterwards
    status.zero_()
    fresh_flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    fresh_state = torch.zeros(4, dtype=torch.int32, device="cuda")
    code = lib.singe_allreduce_add_rms_norm_bf16(stream, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(),
                                                 _pointers([partial]), _pointers([fresh_flags]),
                                                 fresh_state.data_ptr(), 0, 1, ROWS, WIDTH, EPS, status.data_ptr())
    assert code == ks.OK
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    expect = (before.float() + partial.float()).to(torch.bfloat16)
    assert torch.equal(hidden, expect)


def test_two_phase_all_reduce_gives_up_when_the_other_rank_never_pushes():
    lib = ks.lib()
    hidden, weight, partial, status = _setup()
    before = hidden.clone()
    per = ROWS // 2
    packets = lambda rows: torch.zeros((rows, WIDTH // 4, 4), dtype=torch.int32, device="cuda")
    receive = [packets(2 * per) for _ in range(2)]
    gather = [packets(ROWS + per) for _ in range(2)]   # all rows, then the staging area of the owned ones
    normed = torch.full((ROWS, WIDTH), 7.0, dtype=torch.bfloat16, device="cuda")
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    state[2] = 1500
    stream = int(torch.cuda.current_stream().cuda_stream)
    code = lib.singe_allreduce_two_phase_add_rms_norm_bf16(
        stream, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(), partial.data_ptr(), _pointers(receive),
        _pointers(gather), state.data_ptr(), 0, 2, ROWS, WIDTH, EPS, 0, status.data_ptr())
    assert code == ks.OK
    torch.cuda.synchronize()
    assert int(status.item()) == ks.STATUS_WAIT_TIMEOUT
    assert torch.equal(hidden, before) and bool((normed == 7.0).all())
    # rank 0 did push its own partial rows, stamped with the first epoch: the half it owns into its own slot 0,
    # the other half into slot 0 of the silent peer
    assert bool((receive[0][:per, :, 1] == 1).all()) and bool((receive[1][:per, :, 3] == 1).all())
    assert bool((receive[0][per:] == 0).all())   # the silent rank's slot stayed empty
    # a complete group of one rank runs normally afterwards
    status.zero_()
    lone_state = torch.zeros(4, dtype=torch.int32, device="cuda")
    code = lib.singe_allreduce_two_phase_add_rms_norm_bf16(
        stream, hidden.data_ptr(), normed.data_ptr(), weight.data_ptr(), partial.data_ptr(),
        _pointers([packets(ROWS)]), _pointers([packets(2 * ROWS)]), lone_state.data_ptr(), 0, 1, ROWS, WIDTH, EPS, 0,
        status.data_ptr())
    assert code == ks.OK
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    expect = (before.float() + partial.float()).to(torch.bfloat16)
    assert torch.equal(hidden, expect)
    scale = torch.rsqrt(expect.float().pow(2).mean(dim=1, keepdim=True) + EPS)
    assert torch.allclose(normed.float(), (expect.float() * scale), atol=2e-2, rtol=1e-2)
