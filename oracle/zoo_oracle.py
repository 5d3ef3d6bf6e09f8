"""Float64 CPU oracle of the zoo-lineage INT8 chunk prefill (TEST INFRASTRUCTURE, not a product path).

Restates, in torch-on-CPU float64, the semantics the CUDA kernels must reproduce:

* ``RoleQuantizer``  <- ``linquant/invariances.py:28-138`` (``FakeQuant``): per-role static scales from
  absmax calibration, the three realizable policies (``:13-25``), the role tie q_local -> q_read (``:54``),
  half-away-from-zero rounding (``:97-100``) and the fp32 "operand times reciprocal scale" code rule (``:91-92``).
* ``chunk_prefill``   <- ``linquant/reference.py:24-73`` (``chunk_core``) with the per-chunk cells
  ``_chunk_linear`` (``:190-199``) and ``_chunk_delta`` (``:202-229``), the decay helpers (``:107-163``),
  the secondary-chunk local product (``:125-152``) and the fp32-carry INT8 state update (``:77-103``).
* ``signed_hadamard`` <- ``linquant/reference.py:232-239``.

Unlike the reference it can *record* the integer codes of every quantised operand and of the stored state,
chunk by chunk, which is what the bit-exact parity tests compare against.

Parity pin: ``tests/golden/`` holds outputs of the reference itself (generated where the reference is
importable, by ``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks this file against them.
A second pin comes from the reference's INT8 Triton kernels themselves, run on the CPU with Triton's interpreter
(``tests/golden/make_golden_zoo_kernels.py`` -> ``zoo_kernel_*.npz``): ``tests/test_zoo_kernel_golden.py`` holds
the kernel-lineage emulation here to their outputs and final carries.
"""

from __future__ import annotations

import torch

F64 = torch.float64
SUB = 16  # secondary chunk of the diagonal-decay local product (reference.py:21)

ROLE_NAMES = ("q_read", "q_local", "k_local", "w_read", "v_local", "e_local", "k_write", "v_write", "e_write", "state")
_PER_HEAD = ("q_read", "q_local", "k_local", "w_read")
_KEY_ROLES = ("q_read", "q_local", "k_local", "k_write", "w_read")


def policy_table(name):
    """role -> granularity ("pt" per tensor, "ph" per head, "pc" per head and channel).

    invariances.py:13-25: kernel_static = heads for the read/local key roles, channels for value/write/state;
    kernel_pt = one scalar per role except the state; kernel_ptk = key roles per tensor, value roles per channel."""
    static = {r: ("ph" if r in _PER_HEAD else "pc") for r in ROLE_NAMES}
    if name == "kernel_static":
        return static
    if name == "kernel_pt":
        return {r: ("pc" if r == "state" else "pt") for r in ROLE_NAMES}
    if name == "kernel_ptk":
        return {r: ("pt" if r in _KEY_ROLES else g) for r, g in static.items()}
    raise KeyError(name)


class RoleQuantizer:
    """Static per-role fake quantiser in kernel-lineage mode (tied q roles, half-away rounding, fp32 code rule,
    fp16 local value product). ``lineage=False`` gives the exact-arithmetic variant used for the noise floor."""

    def __init__(self, policy="kernel_static", bits=8, state_bits=8, lineage=True):
        self.gran = policy_table(policy)
        self.policy = policy
        self.bits, self.state_bits = bits, state_bits
        self.qmax = 2 ** (bits - 1) - 1
        self.lineage = lineage  # fp32 code rule, fp32 cumsum/carry, activation-dtype materialisation
        self.local_fp16 = True  # the intra-chunk value product is an fp16 dot in every kernel lineage
        self.calibrating = False
        self.enabled = True
        self.amax: dict[str, torch.Tensor] = {}
        self.scales: dict[str, torch.Tensor] = {}
        self.recording = False
        self.trace: dict[str, list[torch.Tensor]] = {}

    # -- bookkeeping
    @staticmethod
    def _slot(role):
        return "q_read" if role == "q_local" else role  # invariances.py:54

    def start_calibration(self):
        self.amax, self.scales, self.calibrating = {}, {}, True

    def finish_calibration(self):
        """scale = absmax / qmax; the state always uses the 8-bit range (invariances.py:132-135)."""
        smax = 2 ** (self.state_bits - 1) - 1
        self.scales = {r: a / (smax if r == "state" else self.qmax) for r, a in self.amax.items()}
        self.calibrating = False

    def start_recording(self):
        self.recording, self.trace = True, {}

    def half_away(self, y):
        return torch.where(y >= 0, torch.floor(y + 0.5), torch.ceil(y - 0.5))

    def _codes(self, x, scale):
        if self.lineage:  # fp32 operand times fp32 reciprocal, rounded in float64 (invariances.py:91-92)
            return self.half_away((x.float() * (1.0 / scale.float())).double())
        return self.half_away(x / scale)

    def _observe(self, slot, x, gran):
        a = x.abs()
        a = a.amax(dim=(0, 2)) if gran == "pc" else a.amax(dim=(0, 2, 3)) if gran == "ph" else a.amax()
        self.amax[slot] = torch.maximum(self.amax[slot], a) if slot in self.amax else a

    def _broadcast(self, slot, gran):
        s = self.scales[slot]
        if gran == "pc":
            return s.unsqueeze(0).unsqueeze(2)
        if gran == "ph":
            return s.view(1, -1, 1, 1)
        return s

    # -- operand roles: x is [B,H,rows,D]
    def __call__(self, role, x):
        if not self.enabled:
            return x
        slot, gran = self._slot(role), self.gran[role]
        if self.calibrating:
            self._observe(slot, x, gran)
            return x
        scale = self._broadcast(slot, gran).clamp_min(1e-12)
        codes = self._codes(x, scale).clamp(-self.qmax, self.qmax)
        if self.recording:
            self.trace.setdefault(role, []).append(codes.to(torch.int8))
        return codes * scale

    # -- stored state (reference.py:77-103): fp32 carry, INT8 stored copy, no error feedback
    def pass_state(self, S, carry, gam, local):
        if not self.enabled or not self.state_bits:
            return gam * S + local, None
        nxt = (gam * S + local) if carry is None else (gam * carry + local)
        if self.calibrating:
            self._observe("state", nxt, self.gran["state"])
            return nxt, nxt
        sc = self._broadcast("state", self.gran["state"]).to(S.dtype).clamp_min(1e-12)
        smax = 2 ** (self.state_bits - 1) - 1
        if self.lineage:
            sc = sc.float().to(S.dtype)
            nxt = nxt.float().to(S.dtype)
            codes = self.half_away((nxt.float() * (1.0 / sc.float())).double())
        else:
            codes = self.half_away(nxt / sc)
        codes = codes.clamp(-smax, smax)
        if self.recording:
            self.trace.setdefault("state", []).append(codes.to(torch.int8))
        return codes * sc, nxt

    # -- export (invariances.py:102-112 and tests/test_kernel_delta.py:23-33), device-agnostic
    def kernel_scales(self, H, K, V, device="cpu"):
        def grab(role, shape, floor):
            s = self.scales.get(self._slot(role))
            if s is None:
                return torch.ones(shape, dtype=torch.float32, device=device)
            s = s.float()
            if floor:
                s = s.clamp_min(1e-6)
            s = s.reshape(shape) if s.numel() > 1 else s.expand(shape).contiguous()
            return s.to(device)

        return {"q": grab("q_read", (H,), True), "k": grab("k_local", (H,), True), "kw": grab("k_write", (H, K), True),
                "vw": grab("v_write", (H, V), True), "vl": grab("v_local", (H, V), True),
                "state": grab("state", (H, V), True), "w": grab("w_read", (H,), False),
                "el": grab("e_local", (H, V), False), "ew": grab("e_write", (H, V), False)}


def signed_hadamard(n, seed, device=None):
    """Orthogonal Sylvester-Hadamard matrix / sqrt(n) with a seeded +-1 pattern on its columns
    (reference.py:232-239). Returns (R [n,n] float64, signs [n] float64)."""
    Hm = torch.ones(1, 1, dtype=F64)
    while Hm.shape[0] < n:
        Hm = torch.cat([torch.cat([Hm, Hm], 1), torch.cat([Hm, -Hm], 1)], 0)
    signs = torch.randint(0, 2, (n,), generator=torch.Generator().manual_seed(seed)).double() * 2 - 1
    return (Hm / n**0.5 * signs).to(device), signs


# ------------------------------------------------------------------------------------------ chunk pieces
def _to_fp16_grid(x):
    return x.float().to(torch.float16).to(x.dtype)


def _apply_unrot(x, M, qz):
    """Value-basis change of a dequantised product; the kernels do it as an fp16 dot (reference.py:174-179)."""
    if M is None:
        return x
    if qz.lineage:
        return (_to_fp16_grid(x) @ _to_fp16_grid(M)).float().to(x.dtype)
    return x @ M


class _Decay:
    """Per-chunk decay factors (reference.py:107-122)."""

    def __init__(self, gcc, kind, C, like):
        self.kind = kind
        self.tril = torch.ones(C, C, dtype=torch.bool).tril()
        if gcc is None:
            one = like.new_ones(1, 1, 1, 1)
            self.read, self.write, self.carry, self.mask = one, one, one, self.tril.to(like.dtype)
        elif kind == "scalar":
            self.read = gcc.exp().unsqueeze(-1)
            self.write = (gcc[..., -1:] - gcc).exp().unsqueeze(-1)
            self.carry = gcc[..., -1:].exp().unsqueeze(-1)
            self.mask = (gcc.unsqueeze(-1) - gcc.unsqueeze(-2)).masked_fill(~self.tril, -torch.inf).exp()
        else:
            self.read = gcc.exp()
            self.write = (gcc[..., -1:, :] - gcc).exp()
            self.carry = gcc[..., -1, :].unsqueeze(-1).exp()
            self.mask = None

    def split_write(self, eta):
        """(key factor, value factor) of the terminal write (reference.py:155-163)."""
        if self.kind != "diagonal":
            return self.write ** (1 - eta), self.write**eta
        env = self.write.amax(dim=-1, keepdim=True)
        kf = self.write * env ** (-eta)
        if eta > 0:
            kf = torch.where(env > 0, kf, torch.zeros_like(kf))
        return kf, env**eta


def _intra_product(X, Y, gcc, dec, qz, role_x, role_y, local_rot, strict):
    """A_ij = sum_n X_in Y_jn exp(gc_in - gc_jn) below (strict) or on and below the diagonal (reference.py:125-152).
    role None keeps that operand unquantised (delta Gram)."""
    fx = (lambda t: t) if role_x is None else (lambda t: qz(role_x, t))
    fy = (lambda t: t) if role_y is None else (lambda t: qz(role_y, t))
    if dec.kind != "diagonal":
        A = (fx(X) @ fy(Y).transpose(-1, -2)) * dec.mask
        return A.tril(-1) if strict else A
    C = X.shape[-2]
    A = X.new_zeros(*X.shape[:-1], C)
    quantised = qz.enabled and (role_x is not None or role_y is not None)
    for s in range(0, C, SUB):
        rows = slice(s, s + SUB)
        anchor = gcc[..., s : s + 1, :]
        if s > 0:
            Xa = X[..., rows, :] * (gcc[..., rows, :] - anchor).exp()
            Ya = Y[..., :s, :] * (anchor - gcc[..., :s, :]).exp()
            if local_rot is not None and quantised:
                Xa, Ya = _apply_unrot(Xa, local_rot, qz), _apply_unrot(Ya, local_rot, qz)
            A[..., rows, :s] = fx(Xa) @ fy(Ya).transpose(-1, -2)
        gd = gcc[..., rows, :]
        n = gd.shape[-2]
        keep = torch.ones(n, n, dtype=torch.bool).tril(-1 if strict else 0).unsqueeze(-1)
        w = (gd.unsqueeze(-2) - gd.unsqueeze(-3)).masked_fill(~keep, -torch.inf).exp()
        blk = torch.einsum("...in,...jn,...ijn->...ij", fx(X[..., rows, :]), fy(Y[..., rows, :]), w)
        A[..., rows, rows] = blk.tril(-1 if strict else 0)
    return A


def _read_state(Q, dec, S, qz, read_post):
    if read_post and dec.kind != "diagonal":
        return (qz("q_read", Q) @ S) * dec.read
    return qz("q_read", Q * dec.read) @ S


def _local_value(A, Vq, qz):
    if qz.local_fp16:  # fp16 dot on the codes, fp32 accumulate (reference.py:182-187)
        A = _to_fp16_grid(A)
    return A @ Vq


def _cell_linear(Q, Kc, Vc, gcc, bt, S, carry, o):
    qz, dec = o["qz"], _Decay(gcc, o["decay"], Q.shape[-2], Q)
    Y = _read_state(Q, dec, S, qz, o["read_post"])
    A = _intra_product(Q, Kc, gcc, dec, qz, "q_local", "k_local", o["local_rot"], strict=False)
    Y = Y + _apply_unrot(_local_value(A, qz("v_local", Vc), qz), o["unrot"], qz)
    wk, wv = dec.split_write(o["eta"])
    local = _apply_unrot(qz("k_write", Kc * wk).transpose(-1, -2) @ qz("v_write", Vc * wv), o["unrot"], qz)
    S, carry = qz.pass_state(S, carry, dec.carry, local)
    return Y, S, carry


def _cell_delta(Q, Kc, Vc, gcc, bt, S, carry, o):
    qz, dec, sig, tau, mat = o["qz"], _Decay(gcc, o["decay"], Q.shape[-2], Q), o["sigma"], o["tau"], o["mat"]
    C = Q.shape[-2]
    Lf = bt**sig * Kc
    Rf = bt ** (1 - sig) * Kc
    Hw = mat(bt ** ((1 - sig) * tau) * Kc)
    fw = bt ** ((1 - sig) * (1 - tau))
    G = _intra_product(Lf, Rf, gcc, dec, qz, None, None, o["local_rot"], strict=True)
    eye = torch.eye(C, dtype=Q.dtype)
    Tm = torch.linalg.solve_triangular(eye + G, eye.expand(G.shape).clone(), upper=False, unitriangular=True)
    W = mat(Tm @ (Lf * dec.read))
    U = mat(Tm @ (bt**sig * Vc))
    ws = qz("w_read", W) @ S
    if o["unrot"] is not None:
        ws = _apply_unrot(ws, o["unrot"].T, qz)
    E = (U - ws) * fw
    Y = _read_state(Q, dec, S, qz, o["read_post"])
    A = _intra_product(Q, Hw, gcc, dec, qz, "q_local", "k_local", o["local_rot"], strict=False)
    Y = Y + _apply_unrot(_local_value(A, qz("e_local", mat(E)), qz), o["unrot"], qz)
    wk, wv = dec.split_write(o["eta"])
    local = _apply_unrot(qz("k_write", Hw * wk).transpose(-1, -2) @ qz("e_write", E * wv), o["unrot"], qz)
    S, carry = qz.pass_state(S, carry, dec.carry, local)
    return Y, S, carry


def chunk_prefill(q, k, v, g, beta, *, family, decay, scale, qz, rot_qk=None, rot_v=None, eta=0.0, sigma=1.0,
                  tau=1.0, chunk=64, read_post=True, storage="rotated", out_dtype=None, act_dtype=None,
                  return_final_state=False, initial_state=None):
    """Chunkwise forward of one (family, decay) cell on CPU in float64 (reference.py:24-73).

    q,k [B,T,H,K]; v [B,T,H,V]; g [B,T,H] (scalar decay), [B,T,H,K] (diagonal) or None; beta [B,T,H] or None.
    Returns o [B,T,H,V] (and the final fp32-carry state [B,H,K,V] when asked)."""
    B, T, H, K = q.shape
    assert T % chunk == 0, f"T={T} must be a multiple of the chunk size {chunk}"
    odt = out_dtype or q.dtype
    adt = act_dtype or q.dtype
    mat = (lambda x: x.float().to(adt).to(F64)) if qz.lineage else (lambda x: x)
    q, k, v = q.to(F64), k.to(F64), v.to(F64)
    if rot_qk is not None and decay != "diagonal":
        q, k = mat(q @ rot_qk), mat(k @ rot_qk)
    if rot_v is not None:
        v = mat(v @ rot_v)
    q = q * scale
    nc = T // chunk
    tile = lambda x: x.reshape(B, nc, chunk, H, x.shape[-1]).permute(0, 3, 1, 2, 4)  # noqa: E731 [B,H,nc,C,D]
    Qt, Kt, Vt = tile(q), tile(k), tile(v)
    gc = None
    if g is not None:
        gc = g.to(F64).reshape(B, nc, chunk, H, *g.shape[3:]).movedim(3, 1)
        gc = gc.float().cumsum(dim=3).to(F64) if qz.lineage else gc.cumsum(dim=3)
    bt = beta.to(F64).reshape(B, nc, chunk, H).permute(0, 3, 1, 2).unsqueeze(-1) if beta is not None else None
    opts = dict(qz=qz, decay=decay, eta=eta, sigma=sigma, tau=tau, read_post=read_post, mat=mat,
                local_rot=rot_qk if (rot_qk is not None and decay == "diagonal") else None,
                unrot=rot_v.T if (rot_v is not None and storage == "canonical") else None)
    S = q.new_zeros(B, H, K, Vt.shape[-1])
    carry = None
    if initial_state is not None:  # fp32 carry handed over from an earlier segment: the first chunk reads its INT8 copy
        S, carry = qz.pass_state(S, initial_state.to(F64), 1.0, 0.0)
    out = torch.empty_like(Vt)
    cell = _cell_linear if family == "linear" else _cell_delta
    for c in range(nc):
        out[:, :, c], S, carry = cell(Qt[:, :, c], Kt[:, :, c], Vt[:, :, c], gc[:, :, c] if gc is not None else None,
                                      bt[:, :, c] if bt is not None else None, S, carry, opts)
    o = out.permute(0, 2, 3, 1, 4).reshape(B, T, H, -1)
    if rot_v is not None and opts["unrot"] is None:
        o = o @ rot_v.T
    o = o.to(odt)
    if return_final_state:
        return o, (carry if carry is not None else S)
    return o


def calibrate(qz, run):
    """absmax calibration on the very inputs that are then measured (tests/test_kernel_simple_gla.py:56-58)."""
    qz.start_calibration()
    run()
    qz.finish_calibration()


def stacked_trace(qz, role):
    """Recorded codes of ``role`` as one tensor [B,H,NC,rows,D] (int8)."""
    return torch.stack(qz.trace[role], dim=2)
