"""Absmax observers for the static scale buffers of the Mamba-2 SSD ops (host logic, torch on the inputs' device).

The reference defines how these buffers are calibrated only through its Nemotron-H observers
(``scripts/nemotron_h_calibration.py:193-651``, ``scripts/nemotron_h_w4a8.py:126-169,470-515``), which hook a model
forward. The same running-absmax statistics are computed here from the operands of one SSD call, with R / D_QK already
applied to B and C by the caller:

  alpha_hp        (H,P)      amax |x * exp(dA_last - dA) * dt|  / 127     value-side x quantiser
  x_scale_hp      (H,P)      amax |x| / 127                               key-side x quantiser
  B_scale, C_scale (G,)      amax |B|, |C| / 127
  b_gate_scale    (1,1,H,1)  amax |exp(dA_last - dA) * dt * B|   (raw, not / 127)  key-side gated B
  state_scale     (H,P)      amax |local fp chunk state| / 127
  cb_scale        (G,)       amax |C . B^T| / 127
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


class SsdObservers:
    """Running maxima over calibration batches; ``scales()`` exports the buffers the SSD ops take."""

    def __init__(self):
        self.amax: dict[str, torch.Tensor] = {}

    def _upd(self, name, a):
        self.amax[name] = torch.maximum(self.amax[name], a) if name in self.amax else a

    @torch.no_grad()
    def observe(self, x, dt_raw, A_log, B, C, chunk, *, dt_bias=None, dt_softplus=True, dt_limit=(0.0, float("inf"))):
        """x [b,L,H,P]; dt_raw [b,L,H]; A_log [H]; B, C [b,L,G,N] (already rotated / rescaled); L a multiple of chunk."""
        b, L, H, P = x.shape
        G, N = B.shape[2:]
        nc = L // chunk
        dt = dt_raw.double()
        if dt_bias is not None:
            dt = dt + dt_bias.double()
        if dt_softplus:
            dt = F.softplus(dt)
        dt = dt.clamp(dt_limit[0], dt_limit[1])
        dA = (dt * (-torch.exp(A_log.double()))).reshape(b, nc, chunk, H).cumsum(2)          # [b,nc,C,H]
        gate = (dA[:, :, -1:] - dA).exp() * dt.reshape(b, nc, chunk, H)                       # [b,nc,C,H]
        xf = x.double().reshape(b, nc, chunk, H, P)
        Bf = B.double().reshape(b, nc, chunk, G, N)
        Cf = C.double().reshape(b, nc, chunk, G, N)
        rep = H // G
        xg = xf * gate.unsqueeze(-1)
        self._upd("alpha_hp", xg.abs().amax(dim=(0, 1, 2)))
        self._upd("x_hp", xf.abs().amax(dim=(0, 1, 2)))
        self._upd("b_g", Bf.abs().amax(dim=(0, 1, 2, 4)))
        self._upd("c_g", Cf.abs().amax(dim=(0, 1, 2, 4)))
        Bh = Bf.repeat_interleave(rep, dim=3)                                                 # [b,nc,C,H,N]
        self._upd("b_gate_h", (Bh * gate.unsqueeze(-1)).abs().amax(dim=(0, 1, 2, 4)))
        states = torch.einsum("bclhp,bclhn->bchpn", xg, Bh)
        self._upd("state_hp", states.abs().amax(dim=(0, 1, 4)))
        cb = torch.einsum("bclgn,bcsgn->bcgls", Cf, Bf)
        self._upd("cb_g", cb.abs().amax(dim=(0, 1, 3, 4)))
        return self

    def scales(self, floor=1e-6):
        a = {k: v.float().clamp_min(floor) for k, v in self.amax.items()}
        H = a["b_gate_h"].numel()
        return {"alpha_hp": a["alpha_hp"] / 127, "x_scale_hp": a["x_hp"] / 127, "B_scale": a["b_g"] / 127,
                "C_scale": a["c_g"] / 127, "b_gate_scale": a["b_gate_h"].view(1, 1, H, 1), "state_scale": a["state_hp"] / 127,
                "cb_scale": a["cb_g"] / 127}
