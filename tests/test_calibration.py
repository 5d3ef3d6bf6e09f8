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
