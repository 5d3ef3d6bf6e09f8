"""INT8 chunk_gated_delta_rule / chunk_delta_rule (delta family, no or scalar decay) on sm_100a.

Same call as ``linquant/kernels/zoo/gated_delta_rule.py:159-203``; the device work is the C-ABI entry
``lq_delta_fwd`` (WY prologue in fp32-grade tensor-core arithmetic -> chunk-serial state pass -> output kernel)."""

from __future__ import annotations

import torch

from . import _common
from ... import _cabi


def chunk_delta_int8(q, k, v, g, beta, scales, *, sigma=1.0, tau=1.0, eta=1.0, scale=None, chunk_size=64,
                     output_final_state=False, unrot=None, fla_prep=True, bits=8, out_dtype=None, rot=None, dqk=None,
                     initial_state=None, _debug=None):
    """q,k [B,T,H,K], v [B,T,H,V] (fp16/bf16), g [B,T,H] fp32 log-decay or None (DeltaNet), beta [B,T,H].
    scales: 'q' (H,) [on q*scale], 'k' (H,) [Hw, local], 'kw' (H,K) [Hw write], 'w' (H,) [W read],
    'el' (H,V) [E local], 'ew' (H,V) [E write], 'state' (H,V).
    unrot: optional (V,V) R_V^T for canonical storage when v was rotated by R_V (the output comes out canonical).
    ``fla_prep`` is accepted for signature compatibility; the WY prep always runs in this library's own kernel.
    ``rot`` / ``dqk`` fuse the persistent R_QK rotation and the D_QK rescale into the prologue.
    Returns (o, final fp32 state [B,H,K,V] or None)."""
    if not q.is_cuda:
        raise _cabi.LinQuantError("chunk_delta_int8 runs on CUDA tensors only (no CPU path)")
    q, k, v, beta = q.contiguous(), k.contiguous(), v.contiguous(), beta.contiguous()
    B, T, H, K = q.shape
    V = v.shape[-1]
    assert T % chunk_size == 0 and K <= 128
    scale = K**-0.5 if scale is None else scale
    o = torch.empty(v.shape, dtype=out_dtype or v.dtype, device=v.device)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if output_final_state else None
    keep = []
    P = _common.make_problem(q, k, v, g, beta, scales, decay=_cabi.DECAY_NONE if g is None else _cabi.DECAY_SCALAR,
                             eta=eta, sigma=sigma, tau=tau, scale=scale, chunk_size=chunk_size, bits=bits, out=o,
                             final_state=ht, rot_signs=_common.signs_of(rot, K, q.device), dqk=dqk, keep=keep, unrot=unrot, initial_state=initial_state)
    _common.run("lq_delta_fwd", P, True, q, _debug)
    return o, ht
