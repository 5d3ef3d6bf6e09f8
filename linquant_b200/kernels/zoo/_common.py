"""Host-side plumbing shared by the zoo chunk ops: problem descriptor, launch, debug views."""

from __future__ import annotations

import ctypes as C

import torch

from ... import _cabi


def signs_of(rot, K, device):
    """Accepts a (K,) +-1 sign vector or a (K,K) signed-Hadamard matrix as built by
    ``linquant.reference.hadamard_rotation`` (reference.py:232-239: Sylvester H / sqrt(K) with the signs on the
    columns) and returns the (K,) fp32 sign vector the fused Walsh-Hadamard butterfly needs."""
    if rot is None:
        return None
    rot = torch.as_tensor(rot)
    if rot.dim() == 1:
        s = rot
    else:
        assert rot.shape == (K, K), f"rotation must be ({K},{K}) or ({K},)"
        s = torch.sign(rot[0])  # row 0 of the Sylvester matrix is all ones
        ref = _sylvester(K).to(rot.dtype).to(rot.device) / K**0.5 * s
        if not torch.allclose(ref, rot, atol=1e-3):
            raise NotImplementedError("only signed Sylvester-Hadamard rotations are fused into the prologue")
    return s.to(device=device, dtype=torch.float32).contiguous()


def _sylvester(n):
    Hm = torch.ones(1, 1, dtype=torch.float64)
    while Hm.shape[0] < n:
        Hm = torch.cat([torch.cat([Hm, Hm], 1), torch.cat([Hm, -Hm], 1)], 0)
    return Hm


def make_problem(q, k, v, g, beta, scales, *, decay, eta, sigma, tau, scale, chunk_size, bits, out, final_state,
                 rot_signs, dqk, keep, initial_state=None, unrot=None):
    """Builds the C descriptor. ``keep`` collects every temporary tensor whose storage the descriptor points to."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    P = _cabi.ZooProblem()
    P.B, P.T, P.H, P.K, P.V, P.chunk = B, T, H, K, V, chunk_size
    P.act_dtype, P.out_dtype, P.decay = _cabi.dtype_code(q.dtype), _cabi.dtype_code(out.dtype), decay
    P.scale, P.eta, P.sigma, P.tau = float(scale), float(eta), float(sigma), float(tau)
    P.qmax = float(2 ** (bits - 1) - 1)

    def put(name, t):
        keep.append(t)
        setattr(P, name, None if t is None else t.data_ptr())

    put("q", q); put("k", k); put("v", v)
    put("g", None if g is None else g.to(torch.float32).contiguous())
    put("beta", None if beta is None else beta.to(torch.float32).contiguous())
    put("rot_signs", rot_signs)
    put("dqk", _cabi.f32c(dqk, dev))
    for name, key in (("sq", "q"), ("sk", "k"), ("skw", "kw"), ("svl", "vl"), ("svw", "vw"), ("sstate", "state"),
                      ("sw", "w"), ("sel", "el"), ("sew", "ew")):
        put(name, _cabi.f32c(scales.get(key), dev))
    put("o", out)
    put("final_state", final_state)
    put("initial_state", None if initial_state is None else initial_state.to(device=dev, dtype=torch.float32).contiguous())
    if unrot is not None:  # the kernels want the fp16 matrix with the input index contiguous: element [v'][v] = unrot[v][v']
        assert tuple(unrot.shape) == (V, V), f"unrot must be ({V},{V})"
        unrot = unrot.to(device=dev, dtype=torch.float16).t().contiguous()
    put("unrot_t", unrot)
    P.status = _cabi.status_word(dev).data_ptr()  # sticky per-device word: read by linquant_b200.check_status()
    return P


def run(entry, P, delta, like, debug=None):
    L = _cabi.lib()
    ws = _cabi.Workspace(P, delta, like.device)
    fn = getattr(L, entry)
    fn.argtypes = [C.POINTER(_cabi.ZooProblem), C.c_void_p, C.c_size_t, C.c_void_p]
    with torch.cuda.device(like.device):
        _cabi.check(fn(C.byref(P), C.c_void_p(ws.base), C.c_size_t(ws.nbytes), _cabi.stream_of(like)), entry)
    if debug is not None:
        debug["workspace"] = ws
    return ws


def run_stage(entry, P, ws, like):
    """Launch one pipeline stage (``lq_zoo_prologue_linear`` ...) on an already carved workspace."""
    L = _cabi.lib()
    fn = getattr(L, entry)
    fn.argtypes = [C.POINTER(_cabi.ZooProblem), C.POINTER(_cabi.ZooWorkspace), C.c_void_p]
    with torch.cuda.device(like.device):
        _cabi.check(fn(C.byref(P), C.byref(ws.desc), _cabi.stream_of(like)), entry)
