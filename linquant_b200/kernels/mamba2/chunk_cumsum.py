"""dt softplus / clamp, dA = dt * A, chunk-local cumsum (``linquant/kernels/mamba2/chunk_cumsum.py:77-100``)."""

import torch

from . import _ssd


def _quant_chunk_cumsum_fwd(q_dt, dt_scale, q_A_log, A_log_scale, chunk_size, dt_bias=None, dt_softplus=False,
                            dt_limit=(0.0, float("inf"))):
    """q_dt [B,L,H], q_A_log [H] -> (dA_cumsum, dt_out), both [B,H,nchunks,chunk] fp32."""
    _ssd.require_cuda(q_dt, "_quant_chunk_cumsum_fwd")
    batch, seqlen, nheads = q_dt.shape
    assert q_A_log.shape == (nheads,)
    if dt_bias is not None:
        assert dt_bias.shape == (nheads,)
    nc = _ssd.nchunks(seqlen, chunk_size)
    dev = q_dt.device
    call = _ssd.Call(dev).dims(B=batch, L=seqlen, H=nheads, P=64, G=1, N=64, chunk=chunk_size, dt_softplus=bool(dt_softplus))
    call.f32("dt_in", q_dt)
    call.f32("A_log", q_A_log)
    call.f32("dt_bias", dt_bias)
    _ssd.scalar_or_dev(call, "dt_scale", dt_scale)
    _ssd.scalar_or_dev(call, "A_log_scale", A_log_scale)
    call.p.dt_min, call.p.dt_max = float(dt_limit[0]), float(dt_limit[1])
    dt_out = call.put("dt", torch.empty(batch, nheads, nc, chunk_size, device=dev, dtype=torch.float32))
    dA = call.put("dA", torch.empty(batch, nheads, nc, chunk_size, device=dev, dtype=torch.float32))
    call.launch("lq_ssd_chunk_cumsum")
    return dA, dt_out
