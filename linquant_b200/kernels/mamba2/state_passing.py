"""All-INT8 fixed-point state passing, Q0.7 gate (``linquant/kernels/mamba2/state_passing.py:96-121``)."""

import torch

from . import _ssd


def _fixedpoint_state_passing_fwd(states_i8, dA_chunk_cumsum, gate_shift=7, initial_carry=None, return_carry=False,
                                  link=None):
    """states_i8 (B, nchunks, H, dim) int8, dA_chunk_cumsum (B, H, nchunks) -> (out_i8, final_states_i8);
    out_i8[:, c] is the state entering chunk c.

    Extensions over the reference signature (which always starts from a zero state, state_passing.py:54-60):
    ``initial_carry`` (B, H, dim) int32 is the unclamped carry entering the first chunk; ``return_carry=True`` appends
    the unclamped int32 carry after the last chunk to the result. Feeding one call's carry to the next reproduces the
    single call over the concatenated chunks bit for bit (cached prefill, sequence split over GPUs). ``link`` is the
    sequence-parallel hand-off (``linquant_b200.seqpar.SsdLink``): where the carry comes from and goes to, and the
    flags that order the two GPUs' kernels."""
    _ssd.require_cuda(states_i8, "_fixedpoint_state_passing_fwd")
    if gate_shift != 7:
        raise NotImplementedError("the fixed-point gate is Q0.7 (gate_shift=7)")
    B, nc, H, dim = states_i8.shape
    dev = states_i8.device
    states_i8 = states_i8.contiguous()
    a = dA_chunk_cumsum
    # The kernel reads dA[b, h, c, chunk-1] of a dense [B,H,NC,chunk] buffer. The usual argument is exactly that
    # column of the chunk cumsum (dA_cumsum[..., -1]): then the cumsum's own storage is handed over untouched.
    C_ = a.stride(2) if a.dim() == 3 and nc > 1 else 0
    if (a.dtype == torch.float32 and a.shape == (B, H, nc) and C_ in (64, 128, 192, 256) and a.stride(1) == nc * C_
            and a.stride(0) == H * nc * C_ and a.storage_offset() >= C_ - 1):
        call = _ssd.Call(dev).dims(B=B, L=nc * C_, H=H, P=1, G=1, N=dim, chunk=C_)
        call.keep.append(a)
        call.p.dA = a.data_ptr() - (C_ - 1) * 4
    else:
        call = _ssd.Call(dev).dims(B=B, L=nc * 64, H=H, P=1, G=1, N=dim, chunk=64)
        dA = torch.zeros(B, H, nc, 64, device=dev, dtype=torch.float32)
        dA[..., -1] = a.to(torch.float32)
        call.put("dA", dA)
    call.put("states", states_i8)
    out = call.put("passed", torch.empty_like(states_i8, memory_format=torch.contiguous_format))
    final = call.put("final_state", torch.empty(B, H, dim, device=dev, dtype=torch.int8))
    carry = None
    if initial_carry is not None:
        assert initial_carry.shape == (B, H, dim) and initial_carry.dtype == torch.int32
        call.put("carry_in", initial_carry.contiguous())
    if return_carry:
        carry = call.put("carry_out", torch.empty(B, H, dim, device=dev, dtype=torch.int32))
    if link is not None:
        link.apply(call, B, H, dim)
    call.launch("lq_ssd_state_passing")
    return (out, final, carry) if return_carry else (out, final)
