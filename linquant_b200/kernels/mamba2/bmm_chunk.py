"""Per-chunk INT8 C.B^T with a static per-group output scale (``linquant/kernels/mamba2/bmm_chunk.py:142-217``)."""

import torch

from . import _ssd


def _quant_bmm_chunk_fwd(a, a_scale, b, b_scale, chunk_size, static_cb_scale, b_is_fp=False):
    """a (B,L,G,K) int8 with (G,) scale; b (B,L,G,K) int8 or f16/bf16 (b_is_fp) with (G,) scale;
    static_cb_scale (G,) -> (B, nchunks, G, chunk, chunk) int8 on that scale."""
    _ssd.require_cuda(a, "_quant_bmm_chunk_fwd")
    B, L, G, K = a.shape
    nc = _ssd.nchunks(L, chunk_size)
    dev = a.device
    cb_scale = static_cb_scale.float().contiguous()
    assert cb_scale.shape == (G,), f"static_cb_scale must be (ngroups,), got {cb_scale.shape}"
    call = _ssd.Call(dev).dims(B=B, L=L, H=G, P=64, G=G, N=K, chunk=chunk_size)
    call.put("q_C", a.contiguous())
    if b_is_fp:
        bb = call.put("b_fp", b.contiguous())
        call.p.x_dtype = _ssd._cabi.dtype_code(bb.dtype)
    else:
        call.put("q_B", b.contiguous())
        call.p.x_dtype = _ssd._cabi.LQ_F16
    call.f32("C_scale", a_scale, (G,))
    call.f32("B_scale", b_scale, (G,))
    call.f32("cb_scale", cb_scale)
    out = call.put("cb", torch.empty(B, nc, G, chunk_size, chunk_size, device=dev, dtype=torch.int8))
    call.launch("lq_ssd_bmm_chunk", int(bool(b_is_fp)))
    return out
