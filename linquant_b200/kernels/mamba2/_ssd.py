"""Host-side plumbing of the Mamba-2 SSD ops: the C descriptor (``lq_ssd_problem``) and one launcher per op."""

from __future__ import annotations

import ctypes as C
import math

import torch

from ... import _cabi


class SsdProblem(C.Structure):
    _fields_ = [("B", C.c_int), ("L", C.c_int), ("H", C.c_int), ("P", C.c_int), ("G", C.c_int), ("N", C.c_int),
                ("chunk", C.c_int), ("x_dtype", C.c_int),
                ("x_stride_b", C.c_longlong), ("x_stride_t", C.c_longlong), ("x_stride_h", C.c_longlong),
                ("x", C.c_void_p), ("dt_in", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p),
                ("dt_scale", C.c_float), ("A_log_scale", C.c_float), ("dt_min", C.c_float), ("dt_max", C.c_float),
                ("dt_scale_dev", C.c_void_p), ("A_log_scale_dev", C.c_void_p), ("dt_softplus", C.c_int),
                ("dt", C.c_void_p), ("dA", C.c_void_p), ("q_B", C.c_void_p), ("q_C", C.c_void_p), ("q_BT", C.c_void_p),
                ("b_fp", C.c_void_p), ("B_scale", C.c_void_p), ("C_scale", C.c_void_p), ("bscale_g", C.c_void_p),
                ("cb_scale", C.c_void_p), ("alpha_hp", C.c_void_p), ("x_scale_hp", C.c_void_p), ("state_scale", C.c_void_p),
                ("b_gate_scale", C.c_void_p), ("bgs_stride", C.c_longlong * 4),
                ("states", C.c_void_p), ("passed", C.c_void_p), ("final_state", C.c_void_p), ("cb", C.c_void_p),
                ("D", C.c_void_p), ("D_has_hdim", C.c_int), ("out", C.c_void_p), ("scan_kernel", C.c_int), ("status", C.c_void_p),
                ("carry_in", C.c_void_p), ("carry_out", C.c_void_p), ("wait_flags", C.c_void_p), ("post_flags", C.c_void_p),
                ("epoch", C.c_uint), ("wait_ns", C.c_ulonglong)]


def status_word(device):
    """The per-device status word (shared with the zoo ops) that a kernel raises when a bounded wait runs out."""
    return _cabi.status_word(device)


def check_status(device):
    """Synchronises and raises if any kernel on ``device`` reported an expired wait since the last check."""
    _cabi.check_status(device)


class Call:
    """Collects tensors into an ``SsdProblem`` (keeping them alive) and launches one entry of the C ABI."""

    def __init__(self, device, status=True):
        self.p = SsdProblem()
        self.keep = []
        self.device = device
        # status=None / False: no word (the kernels then skip the report); True: the per-device word, created on first use
        if status is True:
            status = status_word(device)
        self.p.status = status.data_ptr() if torch.is_tensor(status) else None

    def dims(self, **kw):
        for k, v in kw.items():
            setattr(self.p, k, int(v))
        return self

    def put(self, name, t):
        self.keep.append(t)
        setattr(self.p, name, None if t is None else t.data_ptr())
        return t

    def x(self, x, copy_ok=True):
        if x.stride(-1) != 1:
            assert copy_ok, "x must have a unit stride along headdim (this entry copies nothing)"
            x = x.contiguous()
        self.keep.append(x)
        self.p.x = x.data_ptr()
        self.p.x_dtype = _cabi.dtype_code(x.dtype)
        self.p.x_stride_b, self.p.x_stride_t, self.p.x_stride_h = x.stride(0), x.stride(1), x.stride(2)
        return x

    def f32(self, name, t, shape=None):
        """Dense fp32 copy on the device; ``shape`` materialises stride-0 (coarser granularity) views."""
        if t is None:
            setattr(self.p, name, None)
            return None
        t = torch.as_tensor(t, device=self.device).to(torch.float32)
        if shape is not None:
            t = t.expand(shape)
        return self.put(name, t.contiguous())

    def launch(self, entry, *extra):
        fn = getattr(_cabi.lib(), entry)
        fn.argtypes = [C.POINTER(SsdProblem)] + [C.c_int] * len(extra) + [C.c_void_p]
        with torch.cuda.device(self.device):
            stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            _cabi.check(fn(C.byref(self.p), *extra, stream), entry)


def require_cuda(t, what):
    if not t.is_cuda:
        raise _cabi.LinQuantError(f"{what} runs on CUDA tensors only (no CPU path)")


def scalar_or_dev(call, name, v):
    """A Python number goes into the descriptor; a tensor stays on the device (no host synchronisation)."""
    if torch.is_tensor(v):
        call.put(name + "_dev", v.to(device=call.device, dtype=torch.float32).reshape(-1)[:1].contiguous())
        setattr(call.p, name, 1.0)
    else:
        setattr(call.p, name + "_dev", None)
        setattr(call.p, name, float(v))


def nchunks(L, chunk):
    assert L % chunk == 0, f"seqlen {L} must be a multiple of the chunk size {chunk}"
    return math.ceil(L / chunk)
