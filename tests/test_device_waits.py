"""Bounded device-side waits: what happens when one runs out, without faulting or hanging the GPU.

The tcgen05 kernels wait on mbarriers (TMA arrival, MMA commit) with a poll limit, and the sequence-parallel state
passing waits on a flag another GPU sets, with a time limit. A wait that gives up raises the per-device status word,
skips its stores, frees its tensor memory and returns; the host learns of it from ``lq_status_poll`` /
``linquant_b200.check_status``. Here the failures are made without any GPU fault: an mbarrier nobody arrives on (nothing
in flight), and a flag nobody posts."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hold_tmem", [0, 1])
def test_mbarrier_wait_runs_out_and_is_reported(hold_tmem):
    import linquant_b200
    from linquant_b200 import _cabi

    L = _cabi.lib()
    dev = torch.device("cuda", 0)
    status = _cabi.status_word(dev)
    linquant_b200.check_status(dev)  # clean before
    trace = torch.zeros(4, dtype=torch.int32, device=dev)
    fn = L.lq_selftest_wait_timeout
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    _cabi.check(fn(status.data_ptr(), trace.data_ptr(), hold_tmem, stream), "selftest")
    t1.record()
    torch.cuda.synchronize()
    print(f"\nbounded mbarrier wait gave up after {t0.elapsed_time(t1):.2f} ms")
    assert trace.tolist() == [1, 2, 3 if hold_tmem else 0, 4], trace.tolist()
    assert int(status.item()) == 1
    with pytest.raises(_cabi.LinQuantError, match="wait"):
        linquant_b200.check_status(dev)
    linquant_b200.check_status(dev)  # the poll cleared the word
    # the tensor memory was released and the context is healthy: a tcgen05 kernel runs right after
    from linquant_b200.kernels.mamba2.chunk_state import _quant_chunk_state_fwd_xfp_static_int8 as cs
    from tests.test_zz_no_alloc import _inputs

    st = cs(*_inputs(3))
    torch.cuda.synchronize()
    assert int(st.abs().max()) > 0
    linquant_b200.check_status(dev)


def test_status_poll_returns_timeout_code_through_the_c_abi():
    from linquant_b200 import _cabi

    L = _cabi.lib()
    word = torch.ones(1, dtype=torch.int32, device="cuda")
    L.lq_status_poll.argtypes = [C.c_void_p, C.c_void_p]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.lq_status_poll(word.data_ptr(), stream) == 6  # LQ_ERR_TIMEOUT
    torch.cuda.synchronize()
    assert int(word.item()) == 0 and L.lq_status_poll(word.data_ptr(), stream) == 0


def test_flag_wait_of_the_state_passing_runs_out_when_nobody_posts():
    """The consumer end of the sequence-parallel hand-off with a producer that never posts: after wait_ns the kernel
    raises the status word and returns with nothing stored."""
    import linquant_b200
    from linquant_b200 import _cabi, seqpar
    from linquant_b200.kernels.mamba2.state_passing import _fixedpoint_state_passing_fwd as sp

    B, NC, H, D = 1, 4, 2, 4096
    g = torch.Generator().manual_seed(1)
    states = torch.randint(-127, 128, (B, NC, H, D), generator=g, dtype=torch.int8).cuda()
    dA = -torch.rand(B, H, NC, generator=g).cuda()
    link = seqpar.SsdLink(B, H, D, "cuda", local=True, wait_ns=2_000_000)  # a last-rank end: waits, posts nothing
    link.next_call()
    linquant_b200.check_status("cuda")
    out, fin = sp(states, dA, link=link)
    torch.cuda.synchronize()
    assert int(_cabi.status_word("cuda").item()) == 2
    with pytest.raises(_cabi.LinQuantError):
        linquant_b200.check_status("cuda")
    # posting the flags (what the producer's kernel would have done) lets the same call through
    flags = link.buf[link.carry_bytes:].view(torch.int32)
    flags.fill_(link.epoch)
    out2, fin2 = sp(states, dA, link=link)
    ref, fref = sp(states, dA)
    torch.cuda.synchronize()
    assert torch.equal(out2, ref) and torch.equal(fin2, fref)  # the carry buffer is still all zero
    linquant_b200.check_status("cuda")
