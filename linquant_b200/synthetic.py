"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

They stand in for model activations (the reference measures on unreleased checkpoints and text corpora).
Generation follows the reference tests' convention: CPU ``torch.Generator``, normalise, then cast
(tests/test_kernel_simple_gla.py:32-38 of the reference)."""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CONFIGS = {
    # Simple GLA / linear attention INT8 chunk prefill (kernel_pt, R_QK, INT8 state)
    "simple_gla": dict(op="simple_gla", B=4, H=16, K=128, V=128, T=4096, chunk=64, policy="kernel_pt", eta=1.0,
                       rot=True, gmean=3.0, dtype="bf16"),
    # Mamba-2 SSD mapped onto the linear/scalar cell: q=C, k=B, v=x*dt, g=dt*A (CPU-sized case)
    "mamba2_small": dict(op="simple_gla", B=1, H=8, K=64, V=64, T=2048, chunk=64, policy="kernel_static", eta=1.0,
                         rot=True, dtype="f16", mamba=True),
    # Gated DeltaNet (kernel_ptk, sqk=0.5, sigma=0.5)
    "gated_deltanet": dict(op="delta", B=4, H=16, K=128, V=128, T=8192, chunk=64, policy="kernel_ptk", eta=1.0,
                           sigma=0.5, tau=1.0, sqk=0.5, rot=True, gmean=3.0, dtype="bf16"),
    # KDA (per-channel decay, key outliers)
    "kda": dict(op="kda", B=8, H=32, K=128, V=128, T=8192, chunk=64, policy="kernel_static", eta=0.0, sigma=1.0,
                tau=1.0, rot=True, gmean=4.0, outliers=0.01, dtype="bf16"),
}
_DT = {"bf16": torch.bfloat16, "f16": torch.float16}


def make_inputs(cfg, seed=0, B=None, T=None):
    """Returns dict(q,k,v,g,beta) on the CPU for configuration ``cfg`` (optionally a smaller batch / length)."""
    c = dict(CONFIGS[cfg]) if isinstance(cfg, str) else dict(cfg)
    B = B or c["B"]
    T = T or c["T"]
    H, K, V = c["H"], c["K"], c["V"]
    dt = _DT[c["dtype"]]
    g = torch.Generator().manual_seed(seed)
    if c.get("mamba"):
        x = torch.randn(B, T, H, V, generator=g)
        Bm = torch.randn(B, T, 1, K, generator=g).expand(B, T, H, K)
        Cm = torch.randn(B, T, 1, K, generator=g).expand(B, T, H, K)
        dtv = F.softplus(torch.randn(B, T, H, generator=g) * 0.5 - 2.0)
        A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
        return dict(q=Cm.contiguous().to(dt), k=Bm.contiguous().to(dt), v=(x * dtv.unsqueeze(-1)).to(dt),
                    g=(dtv * A).float(), beta=None)
    q = torch.randn(B, T, H, K, generator=g)
    k = torch.randn(B, T, H, K, generator=g)
    if c["op"] == "delta":
        q = F.normalize(q, dim=-1)
    if c.get("outliers"):
        # heavy key channels: scaled in the raw draw, so that k keeps unit norm after the normalisation below. A delta
        # rule needs beta * |k|^2 < 2 to stay bounded; scaling after the normalisation (|k|^2 about 4) makes the
        # recurrence grow without bound over a long sequence, which no model activation does.
        nout = max(1, int(round(c["outliers"] * K)))
        idx = torch.randperm(K, generator=g)[:nout]
        k[..., idx] *= 20.0
    k = F.normalize(k, dim=-1)
    v = torch.randn(B, T, H, V, generator=g)
    gshape = (B, T, H, K) if c["op"] in ("kda", "gla") else (B, T, H)
    gd = F.logsigmoid(torch.randn(*gshape, generator=g) + c["gmean"]).float()
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g)).float() if c["op"] in ("delta", "kda") else None
    return dict(q=q.to(dt), k=k.to(dt), v=v.to(dt), g=gd, beta=beta)
