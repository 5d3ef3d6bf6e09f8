"""Kronecker-factored signed Hadamard rotation of the state axis (``linquant/kernels/hadamard.py:106-179``)."""

from __future__ import annotations

import ctypes as C
import math

import torch

from .. import _cabi


def hadamard_matrix(d: int, device=None, dtype=None) -> torch.Tensor:
    """Normalised Sylvester-Hadamard matrix of size d (a power of two)."""
    if d & (d - 1) != 0:
        raise ValueError(f"Hadamard rotation requires d to be a power of 2, got {d}")
    H = torch.ones(1, 1, device=device, dtype=torch.float32)
    while H.shape[0] < d:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    H = H / math.sqrt(d)
    return H.to(dtype) if dtype is not None else H


def kronecker_hadamard_fwd(x, signs, num_heads, n_chunks=2):
    """(x * signs) @ (H_2 (x) H_{D/2}) per head. x (B,T,H,D) f16/bf16 with any token stride; signs (H,D) +-1."""
    if not x.is_cuda:
        raise _cabi.LinQuantError("kronecker_hadamard_fwd runs on CUDA tensors only (no CPU path)")
    if n_chunks != 2:
        raise NotImplementedError("only the H_2 (x) H_{D/2} factorisation is implemented")
    B, T, H, D = x.shape
    assert D >= 64, f"Kronecker Hadamard needs D >= 64, got {D}"
    if x.stride(-1) != 1 or x.stride(2) != D or x.stride(0) != T * x.stride(1):
        x = x.contiguous()
    y = torch.empty(B, T, H, D, device=x.device, dtype=x.dtype)
    s = signs.to(device=x.device, dtype=torch.float32).contiguous()
    fn = _cabi.lib().lq_kronecker_hadamard
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p]
    with torch.cuda.device(x.device):
        _cabi.check(fn(_cabi.ptr(x), _cabi.ptr(y), _cabi.dtype_code(x.dtype), B, T, H, D, x.stride(1), _cabi.ptr(s),
                       _cabi.stream_of(x)), "lq_kronecker_hadamard")
    return y
