"""ctypes binding of ``liblinquant_b200.so`` (the C ABI declared in ``include/linquant_b200.h``).

There is no fallback: if the library is missing or an entry fails, the caller gets an exception."""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblinquant_b200.so")

LQ_F16, LQ_BF16, LQ_F32 = 0, 1, 2
DECAY_NONE, DECAY_SCALAR, DECAY_DIAGONAL = 0, 1, 2
_STATUS = {1: "null pointer", 2: "bad shape", 3: "bad alignment", 4: "unsupported configuration", 5: "launch failure",
           6: "device wait timed out", 7: "workspace too small"}
_DTYPE = {torch.float16: LQ_F16, torch.bfloat16: LQ_BF16, torch.float32: LQ_F32}

_fp = C.POINTER(C.c_float)


class ZooProblem(C.Structure):
    _fields_ = [("B", C.c_int), ("T", C.c_int), ("H", C.c_int), ("K", C.c_int), ("V", C.c_int), ("chunk", C.c_int),
                ("act_dtype", C.c_int), ("out_dtype", C.c_int), ("decay", C.c_int),
                ("scale", C.c_float), ("eta", C.c_float), ("sigma", C.c_float), ("tau", C.c_float), ("qmax", C.c_float),
                ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
                ("rot_signs", C.c_void_p), ("dqk", C.c_void_p),
                ("sq", C.c_void_p), ("sk", C.c_void_p), ("skw", C.c_void_p), ("svl", C.c_void_p), ("svw", C.c_void_p),
                ("sstate", C.c_void_p), ("sw", C.c_void_p), ("sel", C.c_void_p), ("sew", C.c_void_p),
                ("o", C.c_void_p), ("final_state", C.c_void_p), ("initial_state", C.c_void_p), ("unrot_t", C.c_void_p),
                ("status", C.c_void_p)]


class ZooWorkspace(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("qq", "kl", "kwT", "vlT", "vwT", "hT", "wq", "gc", "u", "fw", "amat", "genv", "gcl", "status")]


class LinQuantError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded library. Raises if it has not been built (``python -m linquant_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LinQuantError(f"{LIB_PATH} is missing: build it with `python -m linquant_b200.build` "
                                "(there is no CPU or eager fallback for these kernels)")
        L = C.CDLL(LIB_PATH)
        L.lq_version.restype = C.c_int
        L.lq_last_error_string.restype = C.c_char_p
        L.lq_zoo_workspace_bytes.restype = C.c_size_t
        L.lq_zoo_workspace_bytes.argtypes = [C.POINTER(ZooProblem), C.c_int]
        L.lq_zoo_carve_workspace.argtypes = [C.POINTER(ZooProblem), C.c_int, C.c_void_p, C.c_size_t, C.POINTER(ZooWorkspace)]
        _lib = L
    return _lib


_STATUS_WORDS = {}


def status_word(device):
    """The per-device int32 that every kernel with a bounded device-side wait (TMA / MMA barriers of the tcgen05
    kernels, the hand-off flag of the sequence-parallel state passing) raises when its wait runs out. It lives as long
    as the process, so it can be read long after the call that might have raised it."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _STATUS_WORDS:
        _STATUS_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _STATUS_WORDS[key]


def check_status(device=None):
    """Deferred error check: drains the current stream of ``device``, and raises ``LinQuantError`` if any kernel
    launched through this package on that device gave up on a bounded wait since the previous check (its outputs, and
    those of the calls after it, are then not valid). The ops themselves return without synchronising, so call this
    where a synchronisation is acceptable -- once per forward pass, or before results leave the GPU."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    fn = lib().lq_status_poll
    fn.argtypes = [C.c_void_p, C.c_void_p]
    with torch.cuda.device(dev):
        check(fn(C.c_void_p(w.data_ptr()), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "check_status")


def check(status, what=""):
    if status == 0:
        return
    msg = lib().lq_last_error_string().decode()
    kind = _STATUS.get(status, f"status {status}")
    if status == 2:
        raise AssertionError(f"{what}: {msg}")
    if status == 4:
        raise NotImplementedError(f"{what}: {msg}")
    raise LinQuantError(f"{what}: {kind}: {msg}")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_of(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def dtype_code(dt):
    if dt not in _DTYPE:
        raise NotImplementedError(f"dtype {dt} is not supported by the CUDA kernels")
    return _DTYPE[dt]


def f32c(t, dev):
    """fp32, contiguous, on ``dev`` (scale tensors may arrive as expanded / stride-0 views)."""
    return None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()


_WS_LAYOUT = {  # name -> (torch dtype, lambda(BH,NT,C,K,V) -> shape)
    "qq": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, Cc, K)),
    "kl": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, Cc, K)),
    "kwT": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, K, Cc)),
    "vlT": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, V, Cc)),
    "vwT": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, V, Cc)),
    "hT": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, V, K)),
    "wq": (torch.int8, lambda BH, NT, Cc, K, V: (BH, NT, Cc, K)),
    "gc": (torch.float32, lambda BH, NT, Cc, K, V: (BH, NT, Cc)),
    "u": (None, lambda BH, NT, Cc, K, V: (BH, NT, Cc, V)),  # activation dtype
    "fw": (torch.float32, lambda BH, NT, Cc, K, V: (BH, NT, Cc)),
    "amat": (torch.float16, lambda BH, NT, Cc, K, V: (BH, NT, Cc, Cc)),
    "gcl": (torch.float32, lambda BH, NT, Cc, K, V: (BH, NT, K)),
    "genv": (torch.float32, lambda BH, NT, Cc, K, V: (BH, NT, Cc)),
    "status": (torch.int32, lambda BH, NT, Cc, K, V: (1,)),
}


class Workspace:
    """Device scratch of one zoo call, carved by the library; ``view(name)`` exposes a tile set as a tensor."""

    def __init__(self, prob: ZooProblem, delta: bool, device):
        self.prob, self.delta = prob, delta
        n = lib().lq_zoo_workspace_bytes(C.byref(prob), int(delta))
        self.buf = torch.empty(n + 256, dtype=torch.uint8, device=device)
        off = (-self.buf.data_ptr()) % 256
        self.base = self.buf.data_ptr() + off
        self.off0 = off
        self.nbytes = n
        self.desc = ZooWorkspace()
        check(lib().lq_zoo_carve_workspace(C.byref(prob), int(delta), C.c_void_p(self.base), C.c_size_t(n),
                                           C.byref(self.desc)), "carve workspace")
        self.view("status").zero_()

    def check_status(self):
        """After the stream has drained: raises if a kernel's bounded device-side wait expired."""
        if int(self.view("status").item()) != 0:
            raise LinQuantError("a device-side wait timed out (status word set by the kernel)")
        if self.prob.status:  # the descriptor redirected the kernels to the per-device word
            check_status(self.buf.device)

    def view(self, name):
        p = getattr(self.desc, name)
        if not p:
            return None
        dt, shp = _WS_LAYOUT[name]
        pr = self.prob
        if dt is None:
            dt = torch.float16 if pr.act_dtype == LQ_F16 else torch.bfloat16
        shape = shp(pr.B * pr.H, pr.T // pr.chunk, pr.chunk, pr.K, pr.V)
        if name == "gc" and pr.decay == DECAY_DIAGONAL:
            shape = shape + (pr.K,)
        numel = 1
        for s in shape:
            numel *= s
        start = p - self.base + self.off0
        raw = self.buf[start:start + numel * torch.empty((), dtype=dt).element_size()]
        t = raw.view(dt).view(shape)
        if name == "kl":  # rows are stored in MMA-column order: undo the permutation (copy) for inspection
            tok = torch.arange(shape[2], device=t.device)
            pos = (tok & ~15) | (((tok >> 1) & 1) << 3) | (((tok >> 2) & 3) << 1) | (tok & 1)
            t = t[:, :, pos]
        elif name == "hT":
            v = torch.arange(shape[2], device=t.device)
            pos = (v & ~31) | (((v >> 1) & 3) << 3) | (((v >> 3) & 3) << 1) | (v & 1)
            t = t[:, :, pos]
        return t
