"""INT8 SSD combined forward: cumsum, chunk state, state passing, C.B^T, chunk scan
(``linquant/kernels/mamba2/ssd_combined.py:19-131``). The five sub-ops are module attributes under the reference's
names, so callers that wrap or replace them by name keep working."""

from .bmm_chunk import _quant_bmm_chunk_fwd
from .chunk_cumsum import _quant_chunk_cumsum_fwd
from .chunk_scan_v2 import _quant_chunk_scan_fwd as _chunk_scan_v2
from .chunk_state import _quant_chunk_state_fwd_xfp_static_int8
from .chunk_state_keyside import _chunk_state_keyside_fwd
from .state_passing import _fixedpoint_state_passing_fwd

_GATE_SHIFT = 7  # Q0.7 fixed-point gate


def _quant_mamba_chunk_scan_combined_fwd(x_fp, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale,
                                         chunk_size, q_D, D_scale, dt_bias=None, dt_softplus=True,
                                         dt_limit=(0.0, float("inf")), static_state_scale=None, static_cb_scale=None,
                                         alpha_hp=None, bscale_g=None, keyside=False, x_scale_hp=None, b_fp=None,
                                         b_gate_scale=None, _link=None):
    """FP x in, INT8 chunk states (value side: x weighted and quantised with ``alpha_hp`` against INT8 ``q_B``; key
    side: INT8 x with ``x_scale_hp`` against the gate-weighted ``b_fp`` quantised with ``b_gate_scale``), INT32
    fixed-point recurrence, INT8 CB on ``static_cb_scale``, INT8 chunk scan. Returns (out fp16 [B,L,H,P], None).
    ``_link`` (not in the reference signature) is the sequence-parallel hand-off of ``linquant_b200.seqpar``."""
    batch, seqlen, nheads, headdim = x_fp.shape
    _, _, ngroups, dstate = q_B.shape
    dA_cumsum, dt = _quant_chunk_cumsum_fwd(q_dt, dt_scale, q_A_log, A_log_scale, chunk_size, dt_bias=dt_bias,
                                            dt_softplus=dt_softplus, dt_limit=dt_limit)
    if keyside:
        states_i8 = _chunk_state_keyside_fwd(x_fp, x_scale_hp, b_fp, dt, dA_cumsum, static_state_scale, b_gate_scale)
    else:
        states_i8 = _quant_chunk_state_fwd_xfp_static_int8(x_fp, q_B, dt, dA_cumsum, alpha_hp, bscale_g, static_state_scale)
    states_flat_i8 = states_i8.reshape(batch, -1, nheads, headdim * dstate)
    sp_out_i8, _ = _fixedpoint_state_passing_fwd(states_flat_i8, dA_cumsum[:, :, :, -1], gate_shift=_GATE_SHIFT,
                                                 **({} if _link is None else {"link": _link}))
    states = sp_out_i8.reshape(batch, -1, nheads, headdim, dstate)
    cb_i8 = _quant_bmm_chunk_fwd(q_C, C_scale, b_fp if keyside else q_B, B_scale, chunk_size, static_cb_scale,
                                 b_is_fp=keyside)
    out = _chunk_scan_v2(cb_i8, x_fp, dt, dA_cumsum, q_C, C_scale, states, q_D, D_scale, static_state_scale,
                         static_cb_scale)
    return out, None
