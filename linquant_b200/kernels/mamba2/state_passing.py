"""All-INT8 fixed-point state passing, Q0.7 gate (``linquant/kernels/mamba2/state_passing.py:96-121``)."""

import torch

from . import _ssd


def _fixedpoint_state_passing_fwd(states_i8, dA_chunk_cumsum, gate_shift=7):
    """states_i8 (B, nchunks, H, dim) int8, dA_chunk_cumsum (B, H, nchunks) -> (out_i8, final_states_i8);
    out_i8[:, c] is the state entering chunk c."""
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
    call.launch("lq_ssd_state_passing")
    return out, final
