"""The torch-side absmax observers (linquant_b200/invariances.py) against the oracle's calibration pass.

They produce the static scales every kernel call consumes; the oracle calibrates as the reference does
(``FakeQuant`` in calibration mode inside ``chunk_core``, invariances.py:77-81,132-135 of the reference)."""

import pytest
import torch

from linquant_b200 import invariances as inv
from oracle import zoo_oracle as zo
from tests.helpers import OracleRun, zoo_inputs

B, T, H, K, V = 2, 256, 3, 64, 128


def _compare(got, ref, rtol):
    for name, r in ref.items():
        if name not in got:
            continue
        err = float(((got[name].double() - r.double()).abs() / r.double().abs().clamp_min(1e-30)).max())
        assert err <= rtol, f"scale {name}: relative difference {err:.2e}"


@pytest.mark.parametrize("decay", ["scalar", "none"])
@pytest.mark.parametrize("rot", [False, True])
@pytest.mark.parametrize("policy", ["kernel_static", "kernel_pt", "kernel_ptk"])
def test_linear_observers_match_oracle(decay, rot, policy):
    q, k, v, g, _ = zoo_inputs(B, T, H, K, V, decay=decay, dtype=torch.bfloat16, seed=3)
    eta = 0.5 if decay == "scalar" else 1.0
    R, signs = zo.signed_hadamard(K, 3) if rot else (None, None)
    ref = OracleRun(q, k, v, g, None, family="linear", decay=decay, policy=policy, eta=eta, rot_qk=R).scales("cpu")
    sc = inv.StaticScales(policy, 8, 8)
    inv.calibrate_linear(sc, q, k, v, g, eta=eta, chunk_size=64, rot_signs=None if signs is None else signs.float())
    _compare(sc.finalize().kernel_scales(H, K, V, "cpu"), ref, 1e-6)


@pytest.mark.parametrize("decay", ["scalar", "none"])
@pytest.mark.parametrize("sigma,tau,eta", [(1.0, 1.0, 1.0), (0.5, 0.5, 1.0), (0.0, 1.0, 0.5)])
@pytest.mark.parametrize("policy", ["kernel_static", "kernel_ptk"])
def test_delta_observers_match_oracle(decay, sigma, tau, eta, policy):
    if decay == "none" and eta != 1.0:
        pytest.skip("eta needs a decay")
    q, k, v, g, beta = zoo_inputs(B, T, H, K, V, decay=decay, delta=True, dtype=torch.float16, seed=4)
    R, signs = zo.signed_hadamard(K, 3)
    ref = OracleRun(q, k, v, g, beta, family="delta", decay=decay, policy=policy, eta=eta, sigma=sigma, tau=tau,
                    rot_qk=R).scales("cpu")
    sc = inv.StaticScales(policy, 8, 8)
    inv.calibrate_delta(sc, q, k, v, g, beta, eta=eta, sigma=sigma, tau=tau, chunk_size=64, rot_signs=signs.float())
    got = sc.finalize().kernel_scales(H, K, V, "cpu")
    assert {"w", "el", "ew"} <= set(got)
    _compare(got, ref, 1e-5)


@pytest.mark.parametrize("cell", ["gla", "kda"])
@pytest.mark.parametrize("rot", [False, True])
@pytest.mark.parametrize("eta", [0.0, 0.5])
def test_diagonal_observers_match_oracle(cell, rot, eta):
    delta = cell == "kda"
    q, k, v, g, beta = zoo_inputs(B, T, H, K, V, decay="diagonal", delta=delta, dtype=torch.float16, seed=5)
    R, signs = zo.signed_hadamard(K, 3) if rot else (None, None)
    ref = OracleRun(q, k, v, g, beta, family="delta" if delta else "linear", decay="diagonal", eta=eta, rot_qk=R).scales("cpu")
    sc = inv.StaticScales("kernel_static", 8, 8)
    inv.calibrate_diagonal(sc, q, k, v, g, beta, eta=eta, chunk_size=64, rot_signs=None if signs is None else signs.float())
    _compare(sc.finalize().kernel_scales(H, K, V, "cpu"), ref, 1e-5)


def test_ssd_observers_fill_the_code_range_without_saturating():
    """Scales from the SSD observers, fed to the oracle's SSD ops on the calibration batch itself: every quantised
    tensor reaches its top code somewhere and none saturates (the defining property of absmax calibration)."""
    from linquant_b200.kernels.mamba2.calibration import SsdObservers
    from oracle import ssd_oracle as so

    g = torch.Generator().manual_seed(21)
    b, L, Hh, P, G, N, C = 2, 256, 4, 64, 1, 64, 64
    x = torch.randn(b, L, Hh, P, generator=g).half()
    Bm, Cm = torch.randn(b, L, G, N, generator=g), torch.randn(b, L, G, N, generator=g)
    dt_raw, A_log = torch.randn(b, L, Hh, generator=g) * 0.5 - 2, torch.rand(Hh, generator=g) * 2.7
    obs = SsdObservers().observe(x, dt_raw, A_log, Bm, Cm, C)
    s = obs.scales()
    qB = torch.round(Bm / s["B_scale"].view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    qC = torch.round(Cm / s["C_scale"].view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    assert int(qB.abs().max()) == 127 and int(qC.abs().max()) == 127
    dA, dt = so.chunk_cumsum(dt_raw, 1.0, A_log, 1.0, C, None, True)
    st = so.chunk_state_value(x, qB, dt, dA, s["alpha_hp"], s["B_scale"], s["state_scale"])
    assert 100 <= int(st.abs().max()) <= 127, int(st.abs().max())            # quantised operands: close to, not above, the top code
    stk = so.chunk_state_key(x, s["x_scale_hp"], Bm.half(), dt, dA, s["state_scale"], s["b_gate_scale"])
    assert 100 <= int(stk.abs().max()) <= 127
    cb = so.bmm_chunk(qC, s["C_scale"], qB, s["B_scale"], C, s["cb_scale"])
    assert 110 <= int(cb.abs().max()) <= 127
