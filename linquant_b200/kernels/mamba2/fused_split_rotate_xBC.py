"""Mamba-2 prologue: split xBC, D_QK rescale, Kronecker-Hadamard R rotation and static INT8 quantisation of B and C in
one launch; x is returned as a view (``linquant/kernels/mamba2/fused_split_rotate_xBC.py:230-329``)."""

import ctypes as C

import torch

from ... import _cabi


def prepare_dqk(d: torch.Tensor) -> torch.Tensor:
    """Diagonal key scaling vector as the kernel wants it: fp16-rounded values in a contiguous fp32 tensor."""
    return d.reshape(-1).to(torch.float16).to(torch.float32).contiguous()


def fused_split_rotate_quant_xBC(xBC, r_signs, nheads, ngroups, d_state, headdim, B_inv_scale, C_inv_scale, dqk_b=None,
                                 dqk_c=None):
    """xBC (B, T, d_ssm + 2*G*N) f16/bf16; r_signs (G, N) +-1 or None; B_inv_scale / C_inv_scale (G,) fp32;
    dqk_b / dqk_c (G,N) or None. Returns (x view (B,T,H,P), q_B int8 (B,T,G,N), q_C int8 (B,T,G,N))."""
    if not xBC.is_cuda:
        raise _cabi.LinQuantError("fused_split_rotate_quant_xBC runs on CUDA tensors only (no CPU path)")
    batch, seq_len, xBC_dim = xBC.shape
    d_ssm, g_n = nheads * headdim, ngroups * d_state
    assert xBC_dim == d_ssm + 2 * g_n, f"xBC_dim={xBC_dim} != {d_ssm + 2 * g_n}"
    xBC = xBC.contiguous()
    dev = xBC.device
    f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()  # noqa: E731
    signs, ib, ic = f32(r_signs), f32(B_inv_scale), f32(C_inv_scale)
    db = None if dqk_b is None else prepare_dqk(dqk_b.to(dev))
    dc = None if dqk_c is None else prepare_dqk(dqk_c.to(dev))
    q_B = torch.empty(batch, seq_len, ngroups, d_state, device=dev, dtype=torch.int8)
    q_C = torch.empty(batch, seq_len, ngroups, d_state, device=dev, dtype=torch.int8)
    fn = _cabi.lib().lq_ssd_split_rotate_quant
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 8
    with torch.cuda.device(dev):
        _cabi.check(fn(_cabi.ptr(xBC), _cabi.dtype_code(xBC.dtype), batch, seq_len, d_ssm, ngroups, d_state, _cabi.ptr(signs),
                       _cabi.ptr(ib), _cabi.ptr(ic), _cabi.ptr(db), _cabi.ptr(dc), _cabi.ptr(q_B), _cabi.ptr(q_C),
                       _cabi.stream_of(xBC)), "lq_ssd_split_rotate_quant")
    x_out = xBC[..., :d_ssm].view(batch, seq_len, nheads, headdim)
    return x_out, q_B, q_C
