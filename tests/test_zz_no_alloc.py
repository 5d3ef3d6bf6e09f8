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

    for seed in (11, 12):  # second call reuses the array that still holds the first call's bytes
        x, qB, dt, dA, alpha, bscale, out_scale = _inputs(seed)
        want = _quant_chunk_state_fwd_xfp_static_int8(x, qB, dt, dA, alpha, bscale, out_scale)
        out = torch.full_like(want, 77)
        got = chunk_state_value_no_alloc(x, qB, dt, dA, alpha, bscale, out_scale, out)
        torch.cuda.synchronize()
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
    fn = _cabi.lib().lq_ssd_chunk_state_value_static
    fn.argtypes = [C.POINTER(_ssd.SsdProblem), C.c_void_p]
    status = fn(C.byref(p), None)
    assert status == 7 and b"8388608" in _cabi.lib().lq_last_error_string()
