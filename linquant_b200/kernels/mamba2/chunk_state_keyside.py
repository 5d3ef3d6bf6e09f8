"""Key-side INT8 chunk state (``linquant/kernels/mamba2/chunk_state_keyside.py:342-424``)."""

import torch

from . import _ssd


def _bgs_strides(t):
    """(batch, chunk, head, dstate) element strides of b_gate_scale, zero on size-1 dims."""
    assert t.dim() == 4, f"b_gate_scale must be 4D (B,C,H,N), got {t.dim()}D"
    return tuple(t.stride(i) if t.size(i) > 1 else 0 for i in range(4))


def _chunk_state_keyside_fwd(x_fp, x_scale_hp, b_fp, dt, dA_cumsum, out_qscale, b_gate_scale):
    """x_fp [B,L,H,P], b_fp [B,L,G,N] (same dtype), x_scale_hp / out_qscale (H,P), b_gate_scale 4-D broadcastable to
    (B,NC,H,N) -> states int8 [B,NC,H,P,N]."""
    _ssd.require_cuda(x_fp, "_chunk_state_keyside_fwd")
    _, _, nc, chunk = dt.shape
    _, _, G, N = b_fp.shape
    B, L, H, P = x_fp.shape
    dev = x_fp.device
    call = _ssd.Call(dev).dims(B=B, L=L, H=H, P=P, G=G, N=N, chunk=chunk)
    call.x(x_fp)
    call.put("b_fp", b_fp.to(x_fp.dtype).contiguous())
    call.f32("dt", dt)
    call.f32("dA", dA_cumsum)
    call.f32("x_scale_hp", x_scale_hp, (H, P))
    call.f32("state_scale", out_qscale, (H, P))
    bgs = b_gate_scale if b_gate_scale.dtype == torch.float32 else b_gate_scale.float()
    call.put("b_gate_scale", bgs)
    for i, s in enumerate(_bgs_strides(bgs)):
        call.p.bgs_stride[i] = s
    states = call.put("states", torch.empty(B, nc, H, P, N, device=dev, dtype=torch.int8))
    call.launch("lq_ssd_chunk_state_key")
    return states
