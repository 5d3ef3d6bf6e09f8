"""INT8 chunk scan (``linquant/kernels/mamba2/chunk_scan_v2.py:259-366``)."""

import os

import torch

from . import _ssd


SCAN_KERNELS = {None: 0, "auto": 0, "warp_mma": 1, "tcgen05": 2}


def _quant_chunk_scan_fwd(cb_i8, x_fp, dt, dA_cumsum, q_C, C_scale, states, q_D, D_scale, state_dequant_scale, cb_scale,
                          kernel=None):
    """cb_i8 (B,NC,G,C,C) int8 on cb_scale (G,); x_fp (B,L,H,P); q_C (B,L,G,N) int8 on C_scale (G,); states
    (B,NC,H,P,N) int8 entering each chunk on state_dequant_scale (H,P); q_D (H,) or (H,P) with scalar D_scale, or None.
    ``kernel`` (not in the reference signature): None / "auto" = the library's choice, "warp_mma", or "tcgen05"
    (d_state 128 with chunk 128 or 256). Returns out (B,L,H,P) fp16."""
    _ssd.require_cuda(x_fp, "_quant_chunk_scan_fwd")
    _, _, nc, chunk = dt.shape
    _, _, G, N = q_C.shape
    B, L, H, P = x_fp.shape
    dev = x_fp.device
    if kernel is None:  # LQ_SCAN_KERNEL names one of the kernels for a whole process (measurements, bisecting)
        kernel = os.environ.get("LQ_SCAN_KERNEL") or None
        if kernel == "tcgen05" and not (N == 128 and chunk % 128 == 0):
            kernel = None
    call = _ssd.Call(dev).dims(B=B, L=L, H=H, P=P, G=G, N=N, chunk=chunk, scan_kernel=SCAN_KERNELS[kernel])
    call.x(x_fp)
    call.put("cb", cb_i8.contiguous())
    call.f32("dt", dt)
    call.f32("dA", dA_cumsum)
    call.put("q_C", q_C.contiguous())
    call.f32("C_scale", C_scale, (G,))
    call.put("passed", states.contiguous())
    call.f32("state_scale", state_dequant_scale, (H, P))
    call.f32("cb_scale", cb_scale, (G,))
    if q_D is not None:
        D = q_D.to(torch.float32) * (D_scale.to(torch.float32) if torch.is_tensor(D_scale) else float(D_scale))
        call.put("D", D.contiguous())
        call.p.D_has_hdim = int(q_D.dim() == 2)
    else:
        call.p.D = None
    out = call.put("out", torch.empty(B, L, H, P, device=dev, dtype=torch.float16))
    call.launch("lq_ssd_chunk_scan")
    return out
