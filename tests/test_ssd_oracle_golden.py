"""The Mamba-2 SSD oracle against golden vectors produced by the reference's own Triton kernels.

The fixtures under tests/golden/ssd_*.npz were written by tests/golden/make_golden_ssd.py, which runs the
reference's kernels (linquant/kernels/mamba2/*.py, linquant/kernels/hadamard.py) on the CPU with Triton's
interpreter. Integer results (INT8 chunk states, the fixed-point recurrence, INT8 CB, rotated INT8 B/C codes) and
the fp16/bf16 Hadamard outputs must match bit for bit; fp32 prefix sums and the fp16 scan output within the
stated tolerances (summation order differs)."""

import os

import numpy as np
import pytest
import torch

from oracle import ssd_oracle as so

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    return {k: torch.from_numpy(np.ascontiguousarray(z[k])) for k in z.files}


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


DA_ABS_TOL = 2e-4  # fp32 prefix sum over a chunk of |dA| up to ~50: summation order only
OUT_REL_TOL = 2e-5  # fp16 output of fp32 accumulations


@pytest.mark.parametrize("name", ["ssd_value_n128", "ssd_key_n64"])
def test_ssd_chain_matches_reference_kernels(name):
    g = load(name)
    key, C = bool(g["keyside"]), int(g["chunk"])
    one = torch.ones(1)
    dA, dt = so.chunk_cumsum(g["dt_raw"], one, g["A_log"], one, C, g["dt_bias"], True)
    assert float((dt - g["dt"]).abs().max()) <= 1e-6
    assert float((dA - g["dA"]).abs().max()) <= DA_ABS_TOL
    # each op on the reference's own inputs to that op
    if key:
        st = so.chunk_state_key(g["x"], g["x_scale_hp"], g["b_fp"], g["dt"], g["dA"], g["state_scale"], g["b_gate_scale"])
    else:
        st = so.chunk_state_value(g["x"], g["q_B"], g["dt"], g["dA"], g["alpha_hp"], g["B_scale"], g["state_scale"])
    assert torch.equal(st, g["states"]), "INT8 chunk states"
    B, NC, H, P, N = g["states"].shape
    passed, final = so.state_passing(g["states"].reshape(B, NC, H, P * N), g["dA"][..., -1])
    assert torch.equal(passed, g["passed"]), "fixed-point recurrence, entering states"
    assert torch.equal(final.to(g["final"].dtype), g["final"]), "fixed-point recurrence, final state"
    cb = so.bmm_chunk(g["q_C"], g["C_scale"], g["b_fp"] if key else g["q_B"], g["B_scale"], C, g["cb_scale"], b_is_fp=key)
    assert torch.equal(cb, g["cb"]), "INT8 CB"
    out = so.chunk_scan(g["cb"], g["x"], g["dt"], g["dA"], g["q_C"], g["C_scale"], g["passed"].reshape(B, NC, H, P, N),
                        g["D"], one, g["state_scale"], g["cb_scale"])
    assert rel_l2(out, g["out"]) <= OUT_REL_TOL
    # and the whole chain from the raw inputs
    out2, mid = so.ssd_combined(g["x"], g["dt_raw"], one, g["A_log"], one, g["q_B"], g["B_scale"], g["q_C"], g["C_scale"],
                                C, g["D"], one, dt_bias=g["dt_bias"], dt_softplus=True,
                                static_state_scale=g["state_scale"], static_cb_scale=g["cb_scale"],
                                alpha_hp=g["alpha_hp"], bscale_g=g["B_scale"], keyside=key, x_scale_hp=g["x_scale_hp"],
                                b_fp=g["b_fp"], b_gate_scale=g["b_gate_scale"])
    frac = float((mid["states"] != g["states"]).float().mean())
    assert frac <= 1e-3, f"chunk states from the oracle's own prefix sums: {frac:.2e} of codes differ"
    assert rel_l2(out2, g["out"]) <= 1e-3


@pytest.mark.parametrize("name", ["ssd_split_rotate", "ssd_split_rotate_dqk"])
def test_split_rotate_quant_matches_reference_kernel(name):
    g = load(name)
    xv, qB, qC = so.split_rotate_quant(g["xBC"], g["signs"], int(g["nheads"]), int(g["G"]), int(g["N"]),
                                       int(g["headdim"]), g["B_inv"], g["C_inv"], g.get("dqk_b"), g.get("dqk_c"))
    assert torch.equal(xv.contiguous(), g["x_view"])
    assert torch.equal(qB, g["q_B"])
    assert torch.equal(qC, g["q_C"])


@pytest.mark.parametrize("name", ["ssd_kron_hadamard_f16", "ssd_kron_hadamard_bf16"])
def test_kronecker_hadamard_matches_reference_kernel(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    bf = bool(z["bf16"])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16) if bf else torch.from_numpy(np.ascontiguousarray(a))  # noqa: E731
    x, s, y = t(z["x"]), t(z["signs"]), t(z["y"])
    assert torch.equal(so.kronecker_hadamard(x, s), y)
