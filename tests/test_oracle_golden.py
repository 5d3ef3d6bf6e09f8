"""The CPU oracle against golden vectors produced by the reference implementation itself (tests/golden/)."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle import zoo_oracle as zo
from tests.golden.make_golden import CASES, C, K, case_name

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_every_case_has_a_fixture():
    have = {os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "*.npz"))}
    assert {case_name(c) for c in CASES} <= have


@pytest.mark.parametrize("case", CASES, ids=case_name)
def test_oracle_matches_reference_output(case):
    z = np.load(os.path.join(GOLD, case_name(case) + ".npz"))
    t = lambda n: torch.from_numpy(z[n]) if n in z.files else None  # noqa: E731
    q, k, v, g, beta = t("q"), t("k"), t("v"), t("g"), t("beta")
    qz = zo.RoleQuantizer(case["policy"], 8, 8, True)
    R = zo.signed_hadamard(K, 3)[0] if case["rot_qk"] else None
    run = lambda: zo.chunk_prefill(q, k, v, g, beta, family=case["family"], decay=case["decay"], scale=K**-0.5, qz=qz,  # noqa: E731
                                   rot_qk=R, eta=case["eta"], sigma=case["sigma"], tau=case["tau"], chunk=C,
                                   read_post=True, out_dtype=torch.float32)
    zo.calibrate(qz, run)
    for role, s in qz.scales.items():  # calibrated scales are the reference's, bit for bit
        assert torch.equal(s, t("scale_" + role)), role
    o = run()
    assert torch.equal(o, t("o")), f"max abs diff {(o - t('o')).abs().max().item():.3e}"


def test_hadamard_is_orthogonal_and_signed():
    for n in (64, 128):
        R, s = zo.signed_hadamard(n, 3)
        assert torch.allclose(R @ R.T, torch.eye(n, dtype=torch.float64), atol=1e-12)
        assert torch.equal(torch.sign(R[0]), s)


def test_policies_granularity():
    st, pt, ptk = (zo.policy_table(p) for p in ("kernel_static", "kernel_pt", "kernel_ptk"))
    assert st["q_read"] == "ph" and st["k_write"] == "pc" and st["state"] == "pc"
    assert all(g == "pt" for r, g in pt.items() if r != "state") and pt["state"] == "pc"
    assert ptk["k_write"] == "pt" and ptk["v_write"] == "pc" and ptk["w_read"] == "pt" and ptk["e_local"] == "pc"


def test_fp32_carry_has_no_error_feedback():
    """tests/test_reference.py:204-217 of the reference: the stored INT8 copy never feeds back into the carry."""
    torch.manual_seed(0)
    qz = zo.RoleQuantizer("kernel_static", 8, 8, True)
    S = torch.zeros(1, 2, 4, 4, dtype=torch.float64)
    loc = torch.randn(1, 2, 4, 4, dtype=torch.float64)
    qz.start_calibration()
    qz.pass_state(S, None, 1.0, loc * 3)
    qz.finish_calibration()
    s1, c1 = qz.pass_state(S, None, 0.5, loc)
    s2, c2 = qz.pass_state(s1, c1, 0.5, loc)
    assert torch.allclose(c2, (0.5 * c1 + loc).float().double())
    assert not torch.equal(s2, c2)
