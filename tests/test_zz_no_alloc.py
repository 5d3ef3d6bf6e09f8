"""The allocation-free chunk-state entry point against the regular one.

Some hosts of this library may not allocate device memory at call time (their pools are fixed at start-up), so
``lq_ssd_chunk_state_value_static`` keeps its scratch in an array inside the library. This file checks, through the
C ABI, that it returns exactly what ``lq_ssd_chunk_state_value`` returns, twice in a row on different inputs (the
array keeps the first call's contents), and that it refuses a problem larger than the array. It is collected last."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, B=2, L=512, H=4, P=64, G=1, N=128, chunk=256):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H, P, generator=g).half().cuda()
    qB = torch.randint(-127, 128, (B, L, G, N), generator=g, dtype=torch.int8).cuda()
    dt = (torch.rand(B, H, L // chunk, chunk, generator=g) * 0.2).cuda()
    dA = (-dt * 2.0).cumsum(-1).contiguous()
    alpha = torch.full((H, P), 0.02).cuda()
    out_scale = torch.full((H, P), 0.5).cuda()
    bscale = torch.full((G,), 0.03).cuda()
    return x, qB, dt, dA, alpha, bscale, out_scale


def test_no_alloc_entry_matches_regular_entry_twice():
    from linquant_b200.kernels.mamba2.chunk_state import (_quant_chunk_state_fwd_xfp_static_int8,
                                                          chunk_state_value_no_alloc)

    keep = []  # nothing is freed between the two measurements below
    for seed in (11, 12):  # second call reuses the array that still holds the first call's bytes
        x, qB, dt, dA, alpha, bscale, out_scale = _inputs(seed)
        want = _quant_chunk_state_fwd_xfp_static_int8(x, qB, dt, dA, alpha, bscale, out_scale)
        out = torch.full_like(want, 77)
        keep.append((x, qB, dt, dA, alpha, bscale, out_scale, want, out))
        torch.cuda.synchronize()
        held, free = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        got = chunk_state_value_no_alloc(x, qB, dt, dA, alpha, bscale, out_scale, out)
        torch.cuda.synchronize()
        if seed == 12:  # the first call may load the kernel images; from the second on nothing may be allocated
            assert torch.cuda.memory_allocated() == held, "the wrapper allocated through torch"
            assert torch.cuda.mem_get_info()[0] == free, "free device memory changed across the call"
        assert torch.equal(got, want), f"seed {seed}: {(got != want).sum().item()} state codes differ"
        assert int(want.abs().max()) > 0


def test_no_alloc_entry_rejects_oversized_problem():
    import ctypes as C

    from linquant_b200 import _cabi
    from linquant_b200.kernels.mamba2 import _ssd

    cap = _cabi.lib().lq_ssd_static_scratch_bytes
    cap.restype = C.c_size_t
    assert cap() == 8 << 20
    p = _ssd.SsdProblem()
    p.B, p.L, p.H, p.P, p.G, p.N, p.chunk = 16, 16384, 4, 64, 1, 128, 256  # 32 MiB of scratch would be needed
    dummy = torch.zeros(64, dtype=torch.float16, device="cuda")
    p.x, p.x_dtype, p.x_stride_b, p.x_stride_t, p.x_stride_h = dummy.data_ptr(), 0, 16384 * 256, 256, 64
    fn = _cabi.lib().lq_ssd_chunk_state_value_static
    fn.argtypes = [C.POINTER(_ssd.SsdProblem), C.c_void_p]
    status = fn(C.byref(p), None)
    assert status == 7 and b"8388608" in _cabi.lib().lq_last_error_string()


def test_no_alloc_entry_capacity_boundary():
    """B*L*G*N equal to the array size is accepted and computes the same states as the regular entry; the next valid
    length (one more chunk) is refused with LQ_ERR_WORKSPACE, and a bad extent with LQ_ERR_SHAPE, before any launch."""
    import ctypes as C

    from linquant_b200 import _cabi
    from linquant_b200.kernels.mamba2 import _ssd
    from linquant_b200.kernels.mamba2.chunk_state import (_quant_chunk_state_fwd_xfp_static_int8,
                                                          chunk_state_value_no_alloc)

    B, L, H, P, G, N, chunk = 1, 65536, 1, 64, 1, 128, 256  # 65536 * 128 = 8 MiB exactly
    x, qB, dt, dA, alpha, bscale, out_scale = _inputs(21, B=B, L=L, H=H, P=P, G=G, N=N, chunk=chunk)
    want = _quant_chunk_state_fwd_xfp_static_int8(x, qB, dt, dA, alpha, bscale, out_scale)
    got = chunk_state_value_no_alloc(x, qB, dt, dA, alpha, bscale, out_scale, torch.empty_like(want))
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    fn = _cabi.lib().lq_ssd_chunk_state_value_static
    fn.argtypes = [C.POINTER(_ssd.SsdProblem), C.c_void_p]
    p = _ssd.SsdProblem()
    p.B, p.L, p.H, p.P, p.G, p.N, p.chunk, p.x_dtype = B, L + chunk, H, P, G, N, chunk, 0
    p.x = x.data_ptr()
    p.x_stride_b, p.x_stride_t, p.x_stride_h = (L + chunk) * H * P, H * P, P
    assert fn(C.byref(p), None) == 7 and b"8421376" in _cabi.lib().lq_last_error_string()
    p.L = 0
    assert fn(C.byref(p), None) == 2  # a non-positive extent is a shape error, not a capacity error
    p.L, p.B = L, 2**30  # a product that would wrap 32-bit arithmetic is still refused as too large
    assert fn(C.byref(p), None) == 7


def test_no_alloc_wrapper_refuses_inputs_it_would_have_to_copy():
    from linquant_b200.kernels.mamba2.chunk_state import chunk_state_value_no_alloc

    x, qB, dt, dA, alpha, bscale, out_scale = _inputs(13)
    out = torch.empty(2, 2, 4, 64, 128, dtype=torch.int8, device="cuda")
    with pytest.raises(AssertionError):
        chunk_state_value_no_alloc(x.transpose(2, 3).contiguous().transpose(2, 3), qB, dt, dA, alpha, bscale, out_scale, out)
    with pytest.raises(AssertionError):
        chunk_state_value_no_alloc(x, qB, dt, dA, alpha[:, :1].expand(4, 64), bscale, out_scale, out)
