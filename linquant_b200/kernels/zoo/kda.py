"""INT8 chunk_kda (delta rule with diagonal, per-channel decay) on sm_100a.

Same call as ``linquant/kernels/zoo/kda.py:154-203``; the device work is the C-ABI entry ``lq_kda_fwd``
(row pass -> A matrix -> per-channel WY prep -> chunk-serial state pass -> output kernel)."""

from __future__ import annotations

import torch

from . import _common
from ... import _cabi
from .gla import BC


def chunk_kda_int8(q, k, v, g, beta, scales, *, sigma=1.0, tau=1.0, eta=0.0, scale=None, chunk_size=64,
                   output_final_state=False, unrot=None, rot=None, fla_prep=True, bits=8, out_dtype=None, initial_state=None,
                   _debug=None):
    """q,k [B,T,H,K], v [B,T,H,V] (fp16/bf16), g [B,T,H,K] fp32 per-channel log-decay, beta [B,T,H].
    scales: 'q' (H,), 'k' (H,) [Hw local], 'kw' (H,K) [Hw write], 'w' (H,) [W read], 'el'/'ew' (H,V) [E local /
    write], 'state' (H,V). rot: signed-Hadamard R_QK for the anchored local operands. ``fla_prep`` is accepted for
    signature compatibility; the WY prep always runs in this library's own kernel.
    Returns (o [B,T,H,V] in v.dtype or out_dtype, final fp32 state or None)."""
    if not q.is_cuda:
        raise _cabi.LinQuantError("chunk_kda_int8 runs on CUDA tensors only (no CPU path)")
    q, k, v, beta = q.contiguous(), k.contiguous(), v.contiguous(), beta.contiguous()
    B, T, H, K = q.shape
    V = v.shape[-1]
    assert T % chunk_size == 0 and K <= 128 and chunk_size % BC == 0
    scale = K**-0.5 if scale is None else scale
    o = torch.empty(v.shape, dtype=out_dtype or v.dtype, device=v.device)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    keep = []
    P = _common.make_problem(q, k, v, g, beta, scales, decay=_cabi.DECAY_DIAGONAL, eta=eta, sigma=sigma, tau=tau,
                             scale=scale, chunk_size=chunk_size, bits=bits, out=o, final_state=ht,
                             rot_signs=_common.signs_of(rot, K, q.device), dqk=None, keep=keep, unrot=unrot, initial_state=initial_state)
    _common.run("lq_kda_fwd", P, True, q, _debug)
    return o, ht
