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


def chunk_state_value_no_alloc(x_fp, q_B, dt, dA_cumsum, alpha_hp, bscale_g, out_qscale, out, status=None):
    """Value-side chunk state for callers that must not allocate device memory while the model runs (for example a
    serving process whose memory pools were fixed at start-up). It is the same computation as
    ``_quant_chunk_state_fwd_xfp_static_int8`` but goes through ``lq_ssd_chunk_state_value_static``: the transposed
    copy of ``q_B`` lives in an 8 MiB array inside the library, so ``B*L*G*N`` must stay within 8 MiB (a larger
    problem raises), and the caller passes the ``out`` tensor (B,NC,H,P,N) int8 itself. Every tensor must already be
    in the form the kernel reads: x with a unit stride along headdim, q_B dense int8, dt, dA_cumsum and the three
    scale tensors dense fp32 on the device ((H,P) for the two per-channel scales). Anything else is an assertion
    error, never a copy: this wrapper allocates no device memory. ``status`` is an optional int32 device tensor of one
    element, allocated by the caller beforehand, that the kernel raises if a bounded barrier wait runs out; without it
    that condition goes unreported. Calls on one device share the array, so do not overlap them on two streams."""
    _ssd.require_cuda(x_fp, "chunk_state_value_no_alloc")
    _, _, nc, chunk = dt.shape
    _, _, G, N = q_B.shape
    B, L, H, P = x_fp.shape
    for name, t, dtype in (("q_B", q_B, torch.int8), ("dt", dt, torch.float32), ("dA_cumsum", dA_cumsum, torch.float32),
                           ("alpha_hp", alpha_hp, torch.float32), ("bscale_g", bscale_g, torch.float32),
                           ("out_qscale", out_qscale, torch.float32), ("out", out, torch.int8)):
        assert t.is_cuda and t.dtype == dtype and t.is_contiguous(), f"{name} must be a dense {dtype} CUDA tensor"
    assert alpha_hp.shape == (H, P) and out_qscale.shape == (H, P) and out.shape == (B, nc, H, P, N)
    assert status is None or (status.is_cuda and status.dtype == torch.int32 and status.numel() == 1)
    call = _ssd.Call(x_fp.device, status=status)
    call.dims(B=B, L=L, H=H, P=P, G=G, N=N, chunk=chunk)
    call.x(x_fp, copy_ok=False)
    for name, t in (("q_B", q_B), ("dt", dt), ("dA", dA_cumsum), ("alpha_hp", alpha_hp), ("state_scale", out_qscale),
                    ("bscale_g", bscale_g), ("states", out)):
        call.put(name, t)
    call.p.q_BT = None
    call.launch("lq_ssd_chunk_state_value_static")
    return out
