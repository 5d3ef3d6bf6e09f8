"""INT8 chunk_gla (linear attention with diagonal, per-channel decay) on sm_100a.

Same call as ``linquant/kernels/zoo/gla.py:235-279``; the device work is the C-ABI entry ``lq_gla_fwd``
(row pass -> A matrix in 16-token secondary chunks -> tiled state pass -> output kernel)."""

from __future__ import annotations

import torch

from . import _common
from ... import _cabi

BC = 16  # secondary chunk


def chunk_gla_int8(q, k, v, g, scales, *, eta=0.0, scale=None, chunk_size=64, output_final_state=False, unrot=None,
                   rot=None, bits=8, out_dtype=None, initial_state=None, _debug=None):
    """q,k [B,T,H,K], v [B,T,H,V] (fp16/bf16), g [B,T,H,K] fp32 per-channel log-decay.
    scales: 'q' (H,) [on q*scale, tied read/local], 'k' (H,), 'kw' (H,K), 'vw' (H,V), 'vl' (H,V), 'state' (H,V).
    unrot: optional (V,V) R_V^T (canonical storage, v arrives rotated).
    rot: optional signed-Hadamard R_QK ((K,K) matrix or (K,) signs) applied to the anchored local operands only.
    Returns (o [B,T,H,V] in v.dtype or out_dtype, final fp32 state [B,H,K,V] or None)."""
    if not q.is_cuda:
        raise _cabi.LinQuantError("chunk_gla_int8 runs on CUDA tensors only (no CPU path)")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, T, H, K = q.shape
    V = v.shape[-1]
    assert T % chunk_size == 0 and K <= 128 and chunk_size % BC == 0
    scale = K**-0.5 if scale is None else scale
    o = torch.empty(v.shape, dtype=out_dtype or v.dtype, device=v.device)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    keep = []
    P = _common.make_problem(q, k, v, g, None, scales, decay=_cabi.DECAY_DIAGONAL, eta=eta, sigma=1.0, tau=1.0,
                             scale=scale, chunk_size=chunk_size, bits=bits, out=o, final_state=ht,
                             rot_signs=_common.signs_of(rot, K, q.device), dqk=None, keep=keep, unrot=unrot, initial_state=initial_state)
    _common.run("lq_gla_fwd", P, False, q, _debug)
    return o, ht
