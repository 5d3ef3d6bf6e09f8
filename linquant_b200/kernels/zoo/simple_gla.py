"""INT8 chunk_simple_gla (linear attention with no or scalar decay) on sm_100a.

Same call as ``linquant/kernels/zoo/simple_gla.py:175-212``; the device work is the C-ABI entry
``lq_simple_gla_fwd`` (fused prologue -> tiled state pass -> output kernel)."""

from __future__ import annotations

import torch

from . import _common
from ... import _cabi


def chunk_simple_gla_int8(q, k, v, g, scales, *, eta=1.0, scale=None, chunk_size=64, output_final_state=False,
                          unrot=None, bits=8, out_dtype=None, rot=None, dqk=None, initial_state=None, _debug=None):
    """q,k [B,T,H,K], v [B,T,H,V] (fp16/bf16), g [B,T,H] fp32 log-decay or None.
    scales: dict with 'q' (H,) [calibrated on q*scale], 'k' (H,), 'kw' (H,K), 'vw' (H,V), 'vl' (H,V), 'state' (H,V),
    fp32 on q's device. T must be a multiple of chunk_size.
    unrot: optional (V,V) R_V^T for canonical storage when v was rotated by R_V (the output comes out canonical).
    Extensions over the reference signature (all optional): ``rot`` fuses the persistent signed-Hadamard R_QK into
    the prologue (a (K,) sign vector or the (K,K) matrix of ``hadamard_rotation``); ``dqk`` (H,K) fuses the
    diagonal rescale q*D, k/D ahead of it; ``initial_state`` (B,H,K,V) fp32 is the carry entering the first chunk
    (zero when omitted), which is what a sequence split over several calls or GPUs hands from one segment to the next.
    Returns (o [B,T,H,V] in v.dtype or out_dtype, final fp32 state [B,H,K,V] or None)."""
    if not q.is_cuda:
        raise _cabi.LinQuantError("chunk_simple_gla_int8 runs on CUDA tensors only (no CPU path)")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, T, H, K = q.shape
    V = v.shape[-1]
    assert T % chunk_size == 0, f"T={T} must be a multiple of the chunk size {chunk_size}"
    scale = K**-0.5 if scale is None else scale
    o = torch.empty(v.shape, dtype=out_dtype or v.dtype, device=v.device)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    keep = []
    P = _common.make_problem(q, k, v, g, None, scales, decay=_cabi.DECAY_NONE if g is None else _cabi.DECAY_SCALAR,
                             eta=eta, sigma=1.0, tau=1.0, scale=scale, chunk_size=chunk_size, bits=bits, out=o,
                             final_state=ht, rot_signs=_common.signs_of(rot, K, q.device), dqk=dqk, keep=keep,
                             initial_state=initial_state, unrot=unrot)
    _common.run("lq_simple_gla_fwd", P, False, q, _debug)
    return o, ht
