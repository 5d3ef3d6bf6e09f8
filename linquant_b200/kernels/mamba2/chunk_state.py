"""Value-side INT8 chunk state (``linquant/kernels/mamba2/chunk_state.py:258-349``)."""

import torch

from . import _ssd


def _quant_chunk_state_fwd_xfp_static_int8(x_fp, q_B, dt, dA_cumsum, alpha_hp, bscale_g, out_qscale):
    """x_fp [B,L,H,P] f16/bf16 (may be a strided view), q_B [B,L,G,N] int8, dt/dA_cumsum [B,H,NC,C] fp32,
    alpha_hp / out_qscale (H,P) fp32 (stride-0 views allowed), bscale_g (G,) -> states int8 [B,NC,H,P,N]."""
    _ssd.require_cuda(x_fp, "_quant_chunk_state_fwd_xfp_static_int8")
    _, _, nc, chunk = dt.shape
    _, _, G, N = q_B.shape
    B, L, H, P = x_fp.shape
    dev = x_fp.device
    call = _ssd.Call(dev).dims(B=B, L=L, H=H, P=P, G=G, N=N, chunk=chunk)
    call.x(x_fp)
    call.put("q_B", q_B.contiguous())
    call.put("q_BT", torch.empty(B, nc, G, N, chunk, device=dev, dtype=torch.int8))
    call.f32("dt", dt)
    call.f32("dA", dA_cumsum)
    call.f32("alpha_hp", alpha_hp, (H, P))
    call.f32("state_scale", out_qscale, (H, P))
    call.f32("bscale_g", bscale_g)
    states = call.put("states", torch.empty(B, nc, H, P, N, device=dev, dtype=torch.int8))
    call.launch("lq_ssd_chunk_state_value")
    return states
