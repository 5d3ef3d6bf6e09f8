"""CPU restatement of the SSDi8-lineage Mamba-2 SSD ops (TEST INFRASTRUCTURE, not a product path).

PARITY PINNED on outputs of the reference itself: the reference implements these ops only as Triton kernels (under
``linquant/kernels/mamba2/`` and ``linquant/kernels/hadamard.py``; the SSDi8 project they descend from is an
un-fetched submodule) and holds no test or golden vector for them, so the fixtures ``tests/golden/ssd_*.npz`` were
produced by running those kernels, unmodified, on the CPU with Triton's interpreter
(``tests/golden/make_golden_ssd.py``). ``tests/test_ssd_oracle_golden.py`` holds every function below to them:
integer results (chunk states, fixed-point recurrence, CB, rotated B/C codes) and the Hadamard outputs bit for bit,
the fp32 prefix sums and the fp16 scan output to summation-order tolerance. What the interpreter cannot pin is the
GPU's own transcendental rounding (exp, log); each function is a line-by-line restatement, in fp32 torch on the
CPU, of the arithmetic written in the Triton source it cites.

  chunk_cumsum        <- mamba2/chunk_cumsum.py:15-100
  chunk_state_value   <- mamba2/chunk_state.py:24-349          (value-side absorption, half-away rounding)
  chunk_state_key     <- mamba2/chunk_state_keyside.py:17-424  (key-side absorption, rint)
  state_passing       <- mamba2/state_passing.py:14-121        (INT32 recurrence, Q0.7 gate)
  bmm_chunk           <- mamba2/bmm_chunk.py:11-217            (rint)
  chunk_scan          <- mamba2/chunk_scan_v2.py:14-366
  ssd_combined        <- mamba2/ssd_combined.py:19-131
  kronecker_hadamard  <- kernels/hadamard.py:38-179
  split_rotate_quant  <- mamba2/fused_split_rotate_xBC.py:31-329
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

F32 = torch.float32


def _half_away(x):
    return torch.where(x >= 0, torch.floor(x + 0.5), torch.ceil(x - 0.5))


def _rint(x):
    return torch.round(x)  # ties to even, as libdevice.rint


def chunk_cumsum(dt, dt_scale, A_log, A_log_scale, chunk, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """dt [B,L,H] -> (dA_cumsum, dt_out) both [B,H,NC,C] fp32."""
    B, L, H = dt.shape
    nc = math.ceil(L / chunk)
    x = float(dt_scale) * dt.to(F32)
    if dt_bias is not None:
        x = x + dt_bias.to(F32)
    if dt_softplus:
        x = torch.where(x > 20.0, x, torch.log(1.0 + torch.exp(x)))
    x = torch.minimum(torch.maximum(x, torch.tensor(dt_limit[0], dtype=F32)), torch.tensor(dt_limit[1], dtype=F32))
    pad = nc * chunk - L
    if pad:
        x = F.pad(x, (0, 0, 0, pad))
    A = -torch.exp(float(A_log_scale) * A_log.to(F32))
    dt_out = x.view(B, nc, chunk, H).permute(0, 3, 1, 2).contiguous()
    dA = dt_out * A.view(1, H, 1, 1)
    return dA.cumsum(-1), dt_out


def _gate(dt, dA):
    return torch.exp(dA[..., -1:] - dA) * dt  # [B,H,NC,C]


def chunk_state_value(x, q_B, dt, dA, alpha_hp, bscale_g, out_qscale):
    """x [B,L,H,P] fp; q_B [B,L,G,N] int8 -> states int8 [B,NC,H,P,N]."""
    B, L, H, P = x.shape
    G, N = q_B.shape[2:]
    nc, C = dt.shape[2:]
    rep = H // G
    gate = _gate(dt, dA)  # [B,H,NC,C]
    xf = x.to(F32).view(B, nc, C, H, P).permute(0, 3, 1, 2, 4)  # [B,H,NC,C,P]
    inv_alpha = 1.0 / alpha_hp.to(F32).expand(H, P)
    xw = (xf * inv_alpha.view(1, H, 1, 1, P)) * gate.unsqueeze(-1)
    xq = _half_away(xw).clamp(-127, 127)
    Bi = q_B.to(torch.float64).view(B, nc, C, G, N).permute(0, 3, 1, 2, 4).repeat_interleave(rep, dim=1)  # [B,H,NC,C,N]
    acc = xq.double().transpose(-1, -2) @ Bi  # [B,H,NC,P,N] exact integers
    req = (alpha_hp.to(F32).expand(H, P) / out_qscale.to(F32).expand(H, P)).unsqueeze(-1) * \
        bscale_g.to(F32).repeat_interleave(rep).view(H, 1, 1)
    accf = acc.to(F32) * req.view(1, H, 1, P, 1)
    return _half_away(accf).clamp(-127, 127).to(torch.int8).permute(0, 2, 1, 3, 4).contiguous()


def chunk_state_key(x, x_scale_hp, b_fp, dt, dA, out_qscale, b_gate_scale):
    """Key-side absorption: x_i8 = rint(x/x_scale); B' = rint(gate*B*127/b_gate)."""
    B, L, H, P = x.shape
    G, N = b_fp.shape[2:]
    nc, C = dt.shape[2:]
    rep = H // G
    gate = _gate(dt, dA)
    xs = x_scale_hp.to(F32).expand(H, P)
    x_inv = 1.0 / torch.clamp_min(xs, 1e-10)
    xf = x.to(F32).view(B, nc, C, H, P).permute(0, 3, 1, 2, 4)
    xq = _rint(xf * x_inv.view(1, H, 1, 1, P)).clamp(-127, 127)
    bg = b_gate_scale.to(F32).expand(B, nc, H, N).permute(0, 2, 1, 3)  # [B,H,NC,N]
    b_inv = 127.0 / bg
    bf = b_fp.to(F32).view(B, nc, C, G, N).permute(0, 3, 1, 2, 4).repeat_interleave(rep, dim=1)
    bq = _rint((bf * gate.unsqueeze(-1)) * b_inv.unsqueeze(-2)).clamp(-127, 127)
    acc = xq.double().transpose(-1, -2) @ bq.double()
    accf = acc.to(F32) * (bg / 127.0).unsqueeze(-2)
    accf = accf * (xs / out_qscale.to(F32).expand(H, P)).view(1, H, 1, P, 1)
    return _rint(accf).clamp(-127, 127).to(torch.int8).permute(0, 2, 1, 3, 4).contiguous()


def state_passing(states_i8, dA_last, gate_shift=7, initial_carry=None, return_carry=False):
    """states [B,NC,H,D] int8, dA_last [B,H,NC] -> (out [B,NC,H,D] int8 entering states, final [B,H,D]).
    ``initial_carry`` [B,H,D] is the unclamped int32 carry entering the first chunk (the reference starts from zero,
    state_passing.py:54-60); ``return_carry`` appends the carry after the last chunk."""
    B, nc, H, D = states_i8.shape
    S = 1 << gate_shift
    s32 = torch.zeros(B, H, D, dtype=torch.int64) if initial_carry is None else initial_carry.to(torch.int64).clone()
    out = torch.empty_like(states_i8)
    final = None
    for c in range(nc):
        out[:, c] = s32.clamp(-127, 127).to(torch.int8)
        g = torch.exp(dA_last[:, :, c].to(F32)) * S
        gq = _half_away(g).clamp(-127.0, 127.0).to(torch.int64)
        s32 = ((s32 * gq.unsqueeze(-1) + (S >> 1)) >> gate_shift) + states_i8[:, c].to(torch.int64)
        s32 = ((s32 + 2**31) % 2**32) - 2**31  # int32 wrap-around
    final = s32.clamp(-127, 127).to(torch.int8)
    if return_carry:
        return out, final, s32.to(torch.int32)
    return out, final


def bmm_chunk(a, a_scale, b, b_scale, chunk, cb_scale, b_is_fp=False):
    """a (C operand) [B,L,G,K] int8; b int8 or fp -> CB int8 [B,NC,G,C,C]."""
    B, L, G, K = a.shape
    nc = math.ceil(L / chunk)
    ai = a.double().view(B, nc, chunk, G, K).permute(0, 1, 3, 2, 4)
    if b_is_fp:
        bq = _rint(b.to(F32) * (1.0 / b_scale.to(F32)).view(1, 1, G, 1)).clamp(-127, 127)
    else:
        bq = b.to(F32)
    bi = bq.double().view(B, nc, chunk, G, K).permute(0, 1, 3, 2, 4)
    acc = ai @ bi.transpose(-1, -2)
    inv = (a_scale.to(F32) * b_scale.to(F32)) / cb_scale.to(F32)
    q = _rint(acc.to(F32) * inv.view(1, 1, G, 1, 1)).clamp(-127, 127)
    return q.to(torch.int8)


def chunk_scan(cb_i8, x, dt, dA, q_C, C_scale, states, q_D, D_scale, state_scale, cb_scale):
    """-> out fp16 [B,L,H,P]."""
    B, L, H, P = x.shape
    G, N = q_C.shape[2:]
    nc, C = dt.shape[2:]
    rep = H // G
    Ci = q_C.double().view(B, nc, C, G, N).permute(0, 3, 1, 2, 4).repeat_interleave(rep, dim=1)  # [B,H,NC,C,N]
    Si = states.double().permute(0, 2, 1, 4, 3)  # [B,H,NC,N,P]
    acc = (Ci @ Si).to(F32)
    acc = acc * C_scale.to(F32).repeat_interleave(rep).view(1, H, 1, 1, 1)
    acc = acc * state_scale.to(F32).expand(H, P).view(1, H, 1, 1, P)
    acc = acc * torch.exp(dA).unsqueeze(-1)
    cb = cb_i8.to(F32).permute(0, 2, 1, 3, 4).repeat_interleave(rep, dim=1)  # [B,H,NC,C,C]
    cb = cb * cb_scale.to(F32).repeat_interleave(rep).view(1, H, 1, 1, 1)
    cb = cb * torch.exp(dA.unsqueeze(-1) - dA.unsqueeze(-2))
    cb = cb * dt.unsqueeze(-2)
    cb = torch.where(torch.ones(C, C, dtype=torch.bool).tril(), cb, torch.zeros(()))
    xf = x.to(F32).view(B, nc, C, H, P).permute(0, 3, 1, 2, 4)
    conv = cb.to(torch.float16).double() @ xf.to(torch.float16).double()
    acc = acc + conv.to(F32)
    if q_D is not None:
        D = float(D_scale) * q_D.to(F32)
        D = D.view(1, H, 1, 1, -1)
        acc = acc + xf * D
    return acc.permute(0, 2, 3, 1, 4).reshape(B, L, H, P).to(torch.float16)


def ssd_combined(x, dt, dt_scale, A_log, A_log_scale, q_B, B_scale, q_C, C_scale, chunk, q_D, D_scale, dt_bias=None,
                 dt_softplus=True, dt_limit=(0.0, float("inf")), static_state_scale=None, static_cb_scale=None,
                 alpha_hp=None, bscale_g=None, keyside=False, x_scale_hp=None, b_fp=None, b_gate_scale=None,
                 initial_carry=None):
    B, L, H, P = x.shape
    dA, dtc = chunk_cumsum(dt, dt_scale, A_log, A_log_scale, chunk, dt_bias, dt_softplus, dt_limit)
    if keyside:
        st = chunk_state_key(x, x_scale_hp, b_fp, dtc, dA, static_state_scale, b_gate_scale)
    else:
        st = chunk_state_value(x, q_B, dtc, dA, alpha_hp, bscale_g, static_state_scale)
    N = st.shape[-1]
    passed, _, carry = state_passing(st.reshape(B, -1, H, P * N), dA[..., -1], initial_carry=initial_carry, return_carry=True)
    passed = passed.reshape(B, -1, H, P, N)
    cb = bmm_chunk(q_C, C_scale, b_fp if keyside else q_B, B_scale, chunk, static_cb_scale, b_is_fp=keyside)
    out = chunk_scan(cb, x, dtc, dA, q_C, C_scale, passed, q_D, D_scale, static_state_scale, static_cb_scale)
    return out, dict(dA=dA, dt=dtc, states=st, passed=passed, cb=cb, carry=carry)


def hadamard_matrix(d):
    Hm = torch.ones(1, 1, dtype=F32)
    while Hm.shape[0] < d:
        Hm = torch.cat([torch.cat([Hm, Hm], 1), torch.cat([Hm, -Hm], 1)], 0)
    return Hm / math.sqrt(d)


def _kron2(x0, x1, s0, s1, bs, kron_scale):
    """(x*signs) -> bf16 -> dot with the bf16 H_bs block (fp32 accumulate) -> H_2 butterfly * kron_scale."""
    Hb = hadamard_matrix(bs).to(torch.bfloat16).double()
    w0 = ((x0 * s0).to(torch.bfloat16).double() @ Hb).to(F32)
    w1 = ((x1 * s1).to(torch.bfloat16).double() @ Hb).to(F32)
    return (w0 + w1) * kron_scale, (w0 - w1) * kron_scale


def kronecker_hadamard(x, signs):
    """x [B,T,H,D] fp16/bf16, signs [H,D] -> y same dtype: (x*signs) @ (H_2 (x) H_{D/2})."""
    D = x.shape[-1]
    bs = D // 2
    xf, sf = x.to(F32), signs.to(F32)
    y0, y1 = _kron2(xf[..., :bs], xf[..., bs:], sf[:, :bs], sf[:, bs:], bs, 1.0 / math.sqrt(2))
    return torch.cat([y0, y1], -1).to(x.dtype)


def split_rotate_quant(xBC, r_signs, nheads, ngroups, d_state, headdim, B_inv_scale, C_inv_scale, dqk_b=None, dqk_c=None):
    Bn, T, _ = xBC.shape
    d_ssm, gn = nheads * headdim, ngroups * d_state
    x = xBC[..., :d_ssm].view(Bn, T, nheads, headdim)
    bs = d_state // 2
    outs = []
    for off, inv, dq in ((d_ssm, B_inv_scale, dqk_b), (d_ssm + gn, C_inv_scale, dqk_c)):
        z = xBC[..., off:off + gn].to(F32).view(Bn, T, ngroups, d_state)
        if dq is not None:
            d16 = dq.reshape(ngroups, d_state).to(torch.float16).to(F32)
            z = (z * d16).to(torch.float16).to(F32)
        if r_signs is not None:
            sf = r_signs.to(F32).view(ngroups, d_state)
            y0, y1 = _kron2(z[..., :bs], z[..., bs:], sf[:, :bs], sf[:, bs:], bs, 1.0 / math.sqrt(2))
            y = torch.cat([y0, y1], -1).to(torch.float16).to(F32)
        else:
            y = z.to(torch.float16).to(F32)
        q = _rint(y * inv.to(F32).view(1, 1, ngroups, 1)).clamp(-128.0, 127.0)
        outs.append(q.to(torch.int8))
    return x, outs[0], outs[1]
