"""Shared test helpers: seeded inputs in the reference tests' conventions, oracle drivers, acceptance rules."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from oracle import zoo_oracle as zo


def zoo_inputs(B, T, H, K, V, *, decay, delta=False, dtype=torch.float16, seed=0, normalize_q=True, gscale=1.0):
    """tests/test_kernel_simple_gla.py:32-38, tests/test_kernel_delta.py:13-20, tests/test_kernel_gla.py:14-20 of
    the reference: CPU generator, L2-normalise, then cast."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=g)
    q = F.normalize(q, dim=-1) if normalize_q else q
    k = F.normalize(torch.randn(B, T, H, K, generator=g), dim=-1)
    v = torch.randn(B, T, H, V, generator=g)
    if decay == "scalar":
        gd = (F.logsigmoid(torch.randn(B, T, H, generator=g) * 3) / 4).float() * gscale
    elif decay == "diagonal":
        gd = (F.logsigmoid(torch.randn(B, T, H, K, generator=g) * 3) / 4).float() * gscale
    else:
        gd = None
    beta = torch.rand(B, T, H, generator=g).float() if delta else None
    return q.to(dtype), k.to(dtype), v.to(dtype), gd, beta


class OracleRun:
    """Calibrates a RoleQuantizer on the given inputs (as the reference tests do) and produces the lineage
    output, the exact-arithmetic output (noise floor) and the recorded codes."""

    def __init__(self, q, k, v, g, beta, *, family, decay, policy="kernel_static", bits=8, eta=1.0, sigma=1.0, tau=1.0,
                 rot_qk=None, scale=None, chunk=64, dqk=None, rot_v=None, storage="rotated", calib=None):
        K = q.shape[-1]
        self.qz = zo.RoleQuantizer(policy, bits, 8, True)
        qd, kd = q, k
        if dqk is not None:  # harness.py:81-88: q*D, k/D in float64 ahead of chunk_core
            qd, kd = q.double() * dqk.double(), k.double() / dqk.double()
        self.kw = dict(family=family, decay=decay, scale=K**-0.5 if scale is None else scale, qz=self.qz, rot_qk=rot_qk,
                       rot_v=rot_v, storage=storage, eta=eta, sigma=sigma, tau=tau, chunk=chunk, read_post=True, out_dtype=torch.float64,
                       act_dtype=q.dtype)
        self.args = (qd, kd, v, g, beta)
        if calib is None:
            zo.calibrate(self.qz, self.run)
        else:  # scales from OTHER batches of the same distribution (a list of (q, k, v, g, beta)), absmax over all
            self.qz.start_calibration()
            for cq, ck, cv, cg, cb in calib:
                if dqk is not None:
                    cq, ck = cq.double() * dqk.double(), ck.double() / dqk.double()
                zo.chunk_prefill(cq, ck, cv, cg, cb, **self.kw)
            self.qz.finish_calibration()
        self.H, self.K, self.V = q.shape[2], K, v.shape[-1]

    def run(self, **over):
        return zo.chunk_prefill(*self.args, **{**self.kw, **over})

    def lineage(self, record=True):
        if record:
            self.qz.start_recording()
        o = self.run(return_final_state=True)
        self.qz.recording = False
        return o

    def exact(self):
        self.qz.lineage = False
        try:
            return self.run()
        finally:
            self.qz.lineage = True

    def scales(self, device):
        return self.qz.kernel_scales(self.H, self.K, self.V, device)

    def codes(self, role):
        return zo.stacked_trace(self.qz, role)  # [B,H,NT,rows,D] int8


def code_mismatch(got, want, label, budget=1e-3, max_step=1):
    """Bit-exact codes, boundary ties excepted: at most ``budget`` of the codes may differ, each by one step."""
    got, want = got.cpu().to(torch.int16), want.cpu().to(torch.int16)
    assert got.shape == want.shape, f"{label}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    d = (got - want).abs()
    frac = (d != 0).float().mean().item()
    worst = int(d.max())
    assert worst <= max_step and frac <= budget, f"{label}: {frac:.3e} of codes differ (budget {budget:.1e}), worst |diff| {worst}"
    return frac


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def reference_check(out, ref, exact, label):
    """Acceptance rule of the reference's kernel tests (tests/test_kernel_simple_gla.py:12-24)."""
    out, ref, exact = out.float().cpu(), ref.float().cpu(), exact.float().cpu()
    d, n = (out - ref).abs(), (ref - exact).abs()
    err_max, err_mean = d.max().item() / ref.abs().max().item(), d.mean().item() / ref.abs().mean().item()
    noise_max, noise_mean = n.max().item() / ref.abs().max().item(), n.mean().item() / ref.abs().mean().item()
    assert torch.isfinite(out).all() and err_max <= max(5e-3, 2 * noise_max) and err_mean <= max(2e-4, 2 * noise_mean), \
        f"{label}: rel max {err_max:.2e} rel mean {err_mean:.2e} (noise floor {noise_max:.2e} / {noise_mean:.2e})"


def passed_states_mismatch(got, want, dA_last, label):
    """Fixed-point state passing is integer arithmetic once the Q0.7 gate code round(exp(dA_last) * 128) is formed, so
    its outputs must equal the oracle's exactly -- except downstream of a chunk whose gate sits on a rounding boundary,
    where the GPU's exp and the CPU's may round the code to different sides. ``got`` / ``want`` are the entering states
    [B,NC,H,D] (or a final state [B,H,D], treated as the state after the last chunk). Sequences (b,h) with no gate within
    1e-4 of a boundary must match bit for bit; a sequence with such a gate at chunk c must match up to and including the
    state entering chunk c. Returns (number of boundary gates, number of differing codes, all of them excused)."""
    got, want = got.cpu().to(torch.int16), want.cpu().to(torch.int16)
    final = got.dim() == 3
    g = torch.exp(dA_last.detach().cpu().float()) * 128.0  # [B,H,NC]
    tie = ((g - torch.floor(g)) - 0.5).abs() < 1e-4
    B, H, NC = g.shape
    first = torch.where(tie.any(-1), tie.float().argmax(-1), torch.full((B, H), NC + 1))  # first boundary chunk per (b,h)
    if final:
        strict = (first > NC).view(B, H, 1)  # the final state is downstream of every chunk
        bad = (got != want) & strict
    else:
        c = torch.arange(NC).view(1, NC, 1)
        strict = (c <= first.unsqueeze(1)).unsqueeze(-1)  # [B,NC,H,1]
        bad = (got != want) & strict
    nbad, ndiff = int(bad.sum()), int((got != want).sum())
    assert nbad == 0, f"{label}: {nbad} codes differ where no gate code is on a rounding boundary (of {ndiff} differing)"
    return int(tie.sum()), ndiff
