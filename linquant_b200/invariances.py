"""Scale policies of the INT8 chunk kernels and absmax calibration of their static scales (host logic, torch).

Mirrors the policy surface of ``linquant/invariances.py``: the role list (``:8``), the three realizable policies
``kernel_static`` / ``kernel_pt`` / ``kernel_ptk`` (``:13-25``), the q_local -> q_read tie (``:54``), absmax / qmax
scales with the state always on the 8-bit range (``:132-135``) and the exported kernel scale dict
(``:102-112`` plus the delta extras of ``tests/test_kernel_delta.py:23-33``).

The observers run the *unquantised* recurrence with plain torch ops on whatever device the inputs live on; they
are calibration plumbing, not the prefill hot path (that is ``linquant_b200.kernels``)."""

from __future__ import annotations

import torch

ROLES = ("q_read", "q_local", "k_local", "w_read", "v_local", "e_local", "k_write", "v_write", "e_write", "state")
POLICIES = {
    "kernel_static": {"q_read": "ph_static", "q_local": "ph_static", "k_local": "ph_static", "w_read": "ph_static",
                      "v_local": "pc_static", "e_local": "pc_static", "k_write": "pc_static", "v_write": "pc_static",
                      "e_write": "pc_static", "state": "pc_static"},
}
POLICIES["kernel_pt"] = {r: ("pt_static" if r != "state" else s) for r, s in POLICIES["kernel_static"].items()}
_KEY_ROLES = ("q_read", "q_local", "k_local", "k_write", "w_read")
POLICIES["kernel_ptk"] = {**POLICIES["kernel_static"], **{r: "pt_static" for r in _KEY_ROLES}}
TIES = {"q_local": "q_read"}


class StaticScales:
    """Running absmax per role at the granularity the policy names; ``kernel_scales`` exports fp32 tensors."""

    def __init__(self, policy="kernel_static", bits=8, state_bits=8):
        if policy not in POLICIES:
            raise KeyError(f"unknown policy {policy!r}; choose from {sorted(POLICIES)}")
        self.policy, self.bits, self.state_bits = policy, bits, state_bits
        self.qmax = 2 ** (bits - 1) - 1
        self.absmax: dict[str, torch.Tensor] = {}
        self.scales: dict[str, torch.Tensor] = {}

    def observe(self, role, x):
        """x is [B,H,rows,D] (operands) or [B,H,K,V] (state)."""
        slot = TIES.get(role, role)
        scheme = POLICIES[self.policy][role]
        a = x.detach().abs()
        a = a.amax(dim=(0, 2)) if scheme == "pc_static" else a.amax(dim=(0, 2, 3)) if scheme == "ph_static" else a.amax()
        self.absmax[slot] = torch.maximum(self.absmax[slot], a) if slot in self.absmax else a

    def finalize(self):
        smax = 2 ** (self.state_bits - 1) - 1
        self.scales = {r: a / (smax if r == "state" else self.qmax) for r, a in self.absmax.items()}
        return self

    def kernel_scales(self, H, K, V, device=None):
        def grab(role, shape, floor=True):
            s = self.scales.get(TIES.get(role, role))
            if s is None:
                return torch.ones(shape, dtype=torch.float32, device=device)
            s = s.float()
            s = s.clamp_min(1e-6) if floor else s  # an all-zero channel must not export 1/0
            s = s.reshape(shape) if s.numel() > 1 else s.expand(shape).contiguous()
            return s.to(device) if device is not None else s

        out = {"q": grab("q_read", (H,)), "k": grab("k_local", (H,)), "kw": grab("k_write", (H, K)),
               "vw": grab("v_write", (H, V)), "vl": grab("v_local", (H, V)), "state": grab("state", (H, V))}
        if "w_read" in self.scales:
            out.update(w=grab("w_read", (H,), False), el=grab("e_local", (H, V), False), ew=grab("e_write", (H, V), False))
        return out


def hadamard_signs(n, seed):
    """Sign pattern of ``linquant.reference.hadamard_rotation(n, seed)`` (reference.py:237-238)."""
    gen = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, (n,), generator=gen).double() * 2 - 1).float()


def signed_hadamard_matrix(signs):
    n = signs.numel()
    Hm = torch.ones(1, 1, dtype=torch.float64)
    while Hm.shape[0] < n:
        Hm = torch.cat([torch.cat([Hm, Hm], 1), torch.cat([Hm, -Hm], 1)], 0)
    return Hm / n**0.5 * signs.double().cpu()


def dqk_from_stats(q, k, alpha):
    """D = (max|k| / max|q|)^alpha per (H,K): q*D, k/D (harness.py:68-79)."""
    aq = q.detach().abs().amax(dim=(0, 1)).double().clamp_min(1e-8)
    ak = k.detach().abs().amax(dim=(0, 1)).double().clamp_min(1e-8)
    return ((ak / aq) ** alpha).float()


def _prepare_qk(q, k, rot_signs, dqk, scale):
    act = q.dtype
    qf, kf = q.float(), k.float()
    if dqk is not None:
        qf, kf = qf * dqk.to(qf.device), kf / dqk.to(kf.device)
    if rot_signs is not None:
        R = signed_hadamard_matrix(rot_signs).float().to(qf.device)
        qf, kf = (qf @ R).to(act).float(), (kf @ R).to(act).float()
    return qf * scale, kf


@torch.no_grad()
def calibrate_linear(sc: StaticScales, q, k, v, g, *, eta=1.0, scale=None, chunk_size=64, rot_signs=None, dqk=None):
    """Observe every role of the linear family with none / scalar decay on one batch (reference.py:190-199 with the
    quantiser in calibration mode: operands pass through, the fp carry is observed as the state)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    C = chunk_size
    nc = T // C
    scale = K**-0.5 if scale is None else scale
    qf, kf = _prepare_qk(q, k, rot_signs, dqk, scale)
    tile = lambda x: x.reshape(B, nc, C, H, x.shape[-1]).permute(0, 3, 1, 2, 4)  # noqa: E731
    Q, Kt, Vt = tile(qf), tile(kf), tile(v.float())
    sc.observe("q_read", Q.reshape(B, H, nc * C, K))
    sc.observe("k_local", Kt.reshape(B, H, nc * C, K))
    sc.observe("v_local", Vt.reshape(B, H, nc * C, V))
    if g is not None:
        gc = g.float().reshape(B, nc, C, H).permute(0, 3, 1, 2).cumsum(-1)  # [B,H,nc,C]
        d = gc[..., -1:] - gc
        wk, wv = ((1 - eta) * d).exp().unsqueeze(-1), (eta * d).exp().unsqueeze(-1)
        gam = gc[..., -1].exp()
    else:
        wk = wv = 1.0
        gam = None
    Kw, Vw = Kt * wk, Vt * wv
    sc.observe("k_write", Kw.reshape(B, H, nc * C, K))
    sc.observe("v_write", Vw.reshape(B, H, nc * C, V))
    carry = torch.zeros(B, H, K, V, dtype=torch.float32, device=q.device)
    for c in range(nc):
        local = Kw[:, :, c].transpose(-1, -2) @ Vw[:, :, c]
        carry = carry * gam[:, :, c, None, None] + local if gam is not None else carry + local
        sc.observe("state", carry)
    return sc


@torch.no_grad()
def calibrate_delta(sc: StaticScales, q, k, v, g, beta, *, eta=1.0, sigma=1.0, tau=1.0, scale=None, chunk_size=64,
                    rot_signs=None, dqk=None):
    """Observe every role of the delta family with none / scalar decay on one batch: the unquantised WY recurrence of
    reference.py:202-229 in float64 on the inputs' device (W, U and the readout key rounded to the activation dtype as
    the kernels see them), with the fp carry observed as the state."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    C = chunk_size
    nc = T // C
    act = q.dtype
    scale = K**-0.5 if scale is None else scale
    qf, kf = _prepare_qk(q, k, rot_signs, dqk, scale)
    rnd = lambda x: x.float().to(act).double()  # noqa: E731
    tile = lambda x: x.reshape(B, nc, C, H, x.shape[-1]).permute(0, 3, 1, 2, 4).double()  # noqa: E731
    Q, Kt, Vt = tile(qf), tile(kf), tile(v.float())
    bt = beta.double().reshape(B, nc, C, H).permute(0, 3, 1, 2).unsqueeze(-1)  # [B,H,nc,C,1]
    if g is not None:
        gc = g.float().reshape(B, nc, C, H).permute(0, 3, 1, 2).cumsum(-1).double()  # [B,H,nc,C]
        read = gc.exp().unsqueeze(-1)
        write = (gc[..., -1:] - gc).exp().unsqueeze(-1)
        gam = gc[..., -1].exp()
        tril = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
        mask = (gc.unsqueeze(-1) - gc.unsqueeze(-2)).masked_fill(~tril, -torch.inf).exp()
    else:
        read = write = torch.ones(1, 1, 1, 1, 1, dtype=torch.float64, device=q.device)
        gam = None
        mask = torch.ones(C, C, dtype=torch.float64, device=q.device).tril()
    Lf = bt**sigma * Kt
    Rf = bt ** (1 - sigma) * Kt
    Hw = rnd(bt ** ((1 - sigma) * tau) * Kt)
    fw = bt ** ((1 - sigma) * (1 - tau))
    G = ((Lf @ Rf.transpose(-1, -2)) * mask).tril(-1)
    eye = torch.eye(C, dtype=torch.float64, device=q.device)
    Tm = torch.linalg.solve_triangular(eye + G, eye.expand(G.shape).clone(), upper=False, unitriangular=True)
    W = rnd(Tm @ (Lf * read))
    U = rnd(Tm @ (bt**sigma * Vt))
    wk, wv = write ** (1 - eta), write**eta
    Kw = Hw * wk
    sc.observe("q_read", Q.reshape(B, H, nc * C, K))
    sc.observe("k_local", Hw.reshape(B, H, nc * C, K))
    sc.observe("k_write", Kw.reshape(B, H, nc * C, K))
    sc.observe("w_read", W.reshape(B, H, nc * C, K))
    S = torch.zeros(B, H, K, V, dtype=torch.float64, device=q.device)
    for c in range(nc):
        E = (U[:, :, c] - W[:, :, c] @ S) * fw[:, :, c]
        sc.observe("e_local", rnd(E))
        Ew = E * (wv[:, :, c] if g is not None else 1.0)
        sc.observe("e_write", Ew)
        local = Kw[:, :, c].transpose(-1, -2) @ Ew
        S = S * gam[:, :, c, None, None] + local if gam is not None else S + local
        sc.observe("state", S)
    return sc


SUB = 16  # secondary chunk of the diagonal-decay local product (reference.py:21)


def _fp16_grid(x):
    return x.float().to(torch.float16).to(x.dtype)


@torch.no_grad()
def calibrate_diagonal(sc: StaticScales, q, k, v, g, beta=None, *, eta=0.0, sigma=1.0, tau=1.0, scale=None, chunk_size=64,
                       rot_signs=None):
    """Observe every role of the per-channel-decay cells on one batch: GLA (``beta`` None, reference.py:190-199) and
    KDA (reference.py:202-229), float64 on the inputs' device. The local product is observed as the kernels form
    it (reference.py:125-152): in 16-token secondary chunks, operands below the diagonal block re-scaled around the
    block's anchor row and, with ``rot_signs``, rotated on the fp16 grid; the diagonal block on the bare operands."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    C, nc = chunk_size, T // chunk_size
    act = q.dtype
    dev = q.device
    scale = K**-0.5 if scale is None else scale
    rnd = lambda x: x.float().to(act).double()  # noqa: E731
    tile = lambda x: x.reshape(B, nc, C, H, x.shape[-1]).permute(0, 3, 1, 2, 4).double()  # noqa: E731
    Q, Kt, Vt = tile(q.float() * scale), tile(k.float()), tile(v.float())
    gc = g.float().reshape(B, nc, C, H, K).permute(0, 3, 1, 2, 4).cumsum(-2).double()  # [B,H,nc,C,K]
    read = gc.exp()
    write = (gc[..., -1:, :] - gc).exp()
    gam = gc[..., -1, :].exp().unsqueeze(-1)  # [B,H,nc,K,1]
    env = write.amax(dim=-1, keepdim=True)
    kf = write * env ** (-eta)
    if eta > 0:
        kf = torch.where(env > 0, kf, torch.zeros_like(kf))
    vfac = env**eta
    R = _fp16_grid(signed_hadamard_matrix(rot_signs).to(dev)) if rot_signs is not None else None
    delta = beta is not None

    def observe_local(X, Y):
        """roles q_local (tied to q_read) and k_local on the operands of the local product A = X . Y^T"""
        for s in range(0, C, SUB):
            rows = slice(s, s + SUB)
            if s > 0:
                anchor = gc[..., s : s + 1, :]
                Xa = X[..., rows, :] * (gc[..., rows, :] - anchor).exp()
                Ya = Y[..., :s, :] * (anchor - gc[..., :s, :]).exp()
                if R is not None:
                    Xa, Ya = (_fp16_grid(Xa) @ R).float().double(), (_fp16_grid(Ya) @ R).float().double()
                sc.observe("q_local", Xa.reshape(B, H, -1, K))
                sc.observe("k_local", Ya.reshape(B, H, -1, K))
            sc.observe("q_local", X[..., rows, :].reshape(B, H, -1, K))
            sc.observe("k_local", Y[..., rows, :].reshape(B, H, -1, K))

    def gram(X, Y):
        """strictly lower A_ij = sum_n X_in Y_jn exp(gc_in - gc_jn), secondary-chunk form, unquantised"""
        A = X.new_zeros(*X.shape[:-1], C)
        for s in range(0, C, SUB):
            rows = slice(s, s + SUB)
            if s > 0:
                anchor = gc[..., s : s + 1, :]
                A[..., rows, :s] = (X[..., rows, :] * (gc[..., rows, :] - anchor).exp()) @ \
                    (Y[..., :s, :] * (anchor - gc[..., :s, :]).exp()).transpose(-1, -2)
            gd = gc[..., rows, :]
            keep = torch.ones(SUB, SUB, dtype=torch.bool, device=dev).tril(-1).unsqueeze(-1)
            w = (gd.unsqueeze(-2) - gd.unsqueeze(-3)).masked_fill(~keep, -torch.inf).exp()
            A[..., rows, rows] = torch.einsum("...in,...jn,...ijn->...ij", X[..., rows, :], Y[..., rows, :], w).tril(-1)
        return A

    sc.observe("q_read", (Q * read).reshape(B, H, nc * C, K))
    if not delta:
        observe_local(Q, Kt)
        Kw, Vw = Kt * kf, Vt * vfac
        sc.observe("v_local", Vt.reshape(B, H, nc * C, V))
        sc.observe("k_write", Kw.reshape(B, H, nc * C, K))
        sc.observe("v_write", Vw.reshape(B, H, nc * C, V))
        S = torch.zeros(B, H, K, V, dtype=torch.float64, device=dev)
        for c in range(nc):
            S = S * gam[:, :, c] + Kw[:, :, c].transpose(-1, -2) @ Vw[:, :, c]
            sc.observe("state", S)
        return sc
    bt = beta.double().reshape(B, nc, C, H).permute(0, 3, 1, 2).unsqueeze(-1)
    Lf, Rf = bt**sigma * Kt, bt ** (1 - sigma) * Kt
    Hw = rnd(bt ** ((1 - sigma) * tau) * Kt)
    fw = bt ** ((1 - sigma) * (1 - tau))
    eye = torch.eye(C, dtype=torch.float64, device=dev)
    G = gram(Lf, Rf)
    Tm = torch.linalg.solve_triangular(eye + G, eye.expand(G.shape).clone(), upper=False, unitriangular=True)
    W = rnd(Tm @ (Lf * read))
    U = rnd(Tm @ (bt**sigma * Vt))
    observe_local(Q, Hw)
    Kw = Hw * kf
    sc.observe("w_read", W.reshape(B, H, nc * C, K))
    sc.observe("k_write", Kw.reshape(B, H, nc * C, K))
    S = torch.zeros(B, H, K, V, dtype=torch.float64, device=dev)
    for c in range(nc):
        E = (U[:, :, c] - W[:, :, c] @ S) * fw[:, :, c]
        sc.observe("e_local", rnd(E))
        Ew = E * vfac[:, :, c]
        sc.observe("e_write", Ew)
        S = S * gam[:, :, c] + Kw[:, :, c].transpose(-1, -2) @ Ew
        sc.observe("state", S)
    return sc
