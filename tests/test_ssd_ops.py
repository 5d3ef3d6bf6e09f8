"""Mamba-2 SSD ops (CUDA, through the C ABI) against the CPU restatement in oracle/ssd_oracle.py.

The reference has no tests for these ops; the oracle is a line-by-line restatement of its Triton sources, so these
tests pin the CUDA kernels to that restatement only (INT8 outputs bit-exact up to rounding-boundary ties)."""

import math

import pytest
import torch
import torch.nn.functional as F

from oracle import ssd_oracle as so
from tests.helpers import code_mismatch, passed_states_mismatch, rel_l2

pytestmark = pytest.mark.gpu


def make_case(B=2, L=512, H=4, P=64, G=1, N=128, chunk=256, dtype=torch.float16, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H, P, generator=g)
    x[..., :2] *= 8.0  # a few heavy channels
    Bm = torch.randn(B, L, G, N, generator=g)
    Cm = torch.randn(B, L, G, N, generator=g)
    dt_raw = torch.randn(B, L, H, generator=g) * 0.5 - 2.0
    A_log = torch.log(torch.exp(torch.rand(H, generator=g) * math.log(16.0)))
    D = torch.randn(H, generator=g)
    x, Bm, Cm = x.to(dtype), Bm.to(dtype), Cm.to(dtype)
    sB = (Bm.float().abs().amax(dim=(0, 1, 3)) / 127).clamp_min(1e-6)
    sC = (Cm.float().abs().amax(dim=(0, 1, 3)) / 127).clamp_min(1e-6)
    qB = torch.round(Bm.float() / sB.view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    qC = torch.round(Cm.float() / sC.view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    dA, dtc = so.chunk_cumsum(dt_raw, 1.0, A_log, 1.0, chunk, None, True)
    nc = L // chunk
    gate = torch.exp(dA[..., -1:] - dA) * dtc  # [B,H,NC,C]
    xw = x.float().view(B, nc, chunk, H, P).permute(0, 3, 1, 2, 4) * gate.unsqueeze(-1)
    alpha = (xw.abs().amax(dim=(0, 2, 3)) / 127).clamp_min(1e-8)  # (H,P)
    x_scale = (x.float().abs().amax(dim=(0, 1)) / 127).clamp_min(1e-8)
    rep = H // G
    Bf = Bm.float().view(B, nc, chunk, G, N).permute(0, 3, 1, 2, 4).repeat_interleave(rep, 1)
    local = xw.transpose(-1, -2) @ Bf  # [B,H,NC,P,N]
    run, amax = torch.zeros(B, H, P, N), torch.zeros(H, P)
    for c in range(nc):
        run = run * torch.exp(dA[:, :, c, -1]).view(B, H, 1, 1) + local[:, :, c]
        amax = torch.maximum(amax, run.abs().amax(dim=(0, 3)))
    state_scale = (amax / 127).clamp_min(1e-8)
    b_gate = (Bf * gate.unsqueeze(-1)).abs().amax(dim=(0, 2, 3)).clamp_min(1e-8).view(1, 1, H, N)  # raw amax, not /127
    Cf = Cm.float().view(B, nc, chunk, G, N).permute(0, 1, 3, 2, 4)
    Bg = Bm.float().view(B, nc, chunk, G, N).permute(0, 1, 3, 2, 4)
    cb_scale = ((Cf @ Bg.transpose(-1, -2)).abs().amax(dim=(0, 1, 3, 4)) / 127).clamp_min(1e-8)
    return dict(x=x, Bm=Bm, Cm=Cm, qB=qB, qC=qC, sB=sB, sC=sC, dt_raw=dt_raw, A_log=A_log, D=D, alpha=alpha, x_scale=x_scale,
                state_scale=state_scale, b_gate=b_gate, cb_scale=cb_scale, chunk=chunk, dA=dA, dt=dtc)


def cu(t):
    return t.cuda() if torch.is_tensor(t) else t


@pytest.mark.parametrize("chunk,N,dtype", [(256, 128, torch.float16), (64, 64, torch.float16), (128, 128, torch.bfloat16),
                                           (256, 64, torch.bfloat16), (128, 64, torch.float16), (192, 128, torch.float16)])
def test_sub_ops_match_oracle(chunk, N, dtype):
    from linquant_b200.kernels.mamba2 import ssd_combined as sc

    k = make_case(N=N, chunk=chunk, dtype=dtype, L=512 if 512 % chunk == 0 else 3 * chunk)
    dA, dt = sc._quant_chunk_cumsum_fwd(cu(k["dt_raw"]), 1.0, cu(k["A_log"]), torch.tensor(1.0).cuda(), chunk, None, True)
    assert rel_l2(dt, k["dt"]) < 1e-6 and (dA.cpu() - k["dA"]).abs().max() < 1e-5 * k["dA"].abs().max()
    # the remaining ops are checked on the oracle's own dt / dA so that each is isolated
    dtd, dAd = cu(k["dt"]), cu(k["dA"])
    st_ref = so.chunk_state_value(k["x"], k["qB"], k["dt"], k["dA"], k["alpha"], k["sB"], k["state_scale"])
    st = sc._quant_chunk_state_fwd_xfp_static_int8(cu(k["x"]), cu(k["qB"]), dtd, dAd, cu(k["alpha"]), cu(k["sB"]), cu(k["state_scale"]))
    code_mismatch(st, st_ref, "value-side chunk states")
    stk_ref = so.chunk_state_key(k["x"], k["x_scale"], k["Bm"], k["dt"], k["dA"], k["state_scale"], k["b_gate"])
    stk = sc._chunk_state_keyside_fwd(cu(k["x"]), cu(k["x_scale"]), cu(k["Bm"]), dtd, dAd, cu(k["state_scale"]), cu(k["b_gate"]))
    code_mismatch(stk, stk_ref, "key-side chunk states")
    B, nc, H, P, Nn = st_ref.shape
    sp_ref, fin_ref = so.state_passing(st_ref.reshape(B, nc, H, P * Nn), k["dA"][..., -1])
    sp, fin = sc._fixedpoint_state_passing_fwd(cu(st_ref).reshape(B, nc, H, P * Nn), dAd[..., -1])
    ties, nd = passed_states_mismatch(sp, sp_ref, k["dA"][..., -1], "passed states")
    passed_states_mismatch(fin, fin_ref, k["dA"][..., -1], "final state")
    print(f"\nstate passing chunk={chunk} N={N}: {ties} gate codes on a rounding boundary, {nd} stored codes differ downstream of them")
    cb_ref = so.bmm_chunk(k["qC"], k["sC"], k["qB"], k["sB"], chunk, k["cb_scale"])
    cb = sc._quant_bmm_chunk_fwd(cu(k["qC"]), cu(k["sC"]), cu(k["qB"]), cu(k["sB"]), chunk, cu(k["cb_scale"]))
    code_mismatch(cb, cb_ref, "CB codes")
    cbk_ref = so.bmm_chunk(k["qC"], k["sC"], k["Bm"], k["sB"], chunk, k["cb_scale"], b_is_fp=True)
    cbk = sc._quant_bmm_chunk_fwd(cu(k["qC"]), cu(k["sC"]), cu(k["Bm"]), cu(k["sB"]), chunk, cu(k["cb_scale"]), b_is_fp=True)
    code_mismatch(cbk, cbk_ref, "CB codes (B quantised in-kernel)")
    passed = sp_ref.reshape(B, nc, H, P, Nn)
    out_ref = so.chunk_scan(cb_ref, k["x"], k["dt"], k["dA"], k["qC"], k["sC"], passed, k["D"], 1.0, k["state_scale"], k["cb_scale"])
    out = sc._chunk_scan_v2(cu(cb_ref), cu(k["x"]), dtd, dAd, cu(k["qC"]), cu(k["sC"]), cu(passed), cu(k["D"]), torch.tensor(1.0).cuda(),
                            cu(k["state_scale"]), cu(k["cb_scale"]))
    assert out.dtype == torch.float16 and rel_l2(out, out_ref) < 2e-3, f"chunk scan rel-L2 {rel_l2(out, out_ref):.2e}"
    if N == 128 and chunk % 128 == 0:  # the tcgen05 variants of the same op
        for kern in ("tcgen05", "warp_mma"):
            out_tc = sc._chunk_scan_v2(cu(cb_ref), cu(k["x"]), dtd, dAd, cu(k["qC"]), cu(k["sC"]), cu(passed), cu(k["D"]),
                                       torch.tensor(1.0).cuda(), cu(k["state_scale"]), cu(k["cb_scale"]), kernel=kern)
            assert rel_l2(out_tc, out_ref) < 2e-3, f"chunk scan ({kern}) rel-L2 {rel_l2(out_tc, out_ref):.2e}"
            assert rel_l2(out_tc, out) < 1e-3, f"the chunk-scan kernels agree ({kern})"
    from linquant_b200.kernels.mamba2 import _ssd

    _ssd.check_status(out.device)  # no tcgen05 kernel gave up on a barrier


@pytest.mark.parametrize("H,chunk", [(40, 128), (80, 256), (33, 64)])
def test_cumsum_and_state_passing_many_heads(H, chunk):
    """More heads than one 32-head block of the cumsum kernel (with a ragged last block), a dt bias and dt limits; state
    passing both through the chunk-end view of the cumsum (read in place) and through a dense copy of it."""
    from linquant_b200.kernels.mamba2 import ssd_combined as sc

    g = torch.Generator().manual_seed(5)
    B, L, dim = 2, 4 * chunk, 1024
    dt_raw = torch.randn(B, L, H, generator=g) * 0.5 - 2.0
    A_log = torch.rand(H, generator=g) * 2.7
    bias = torch.randn(H, generator=g) * 0.3
    dA_ref, dt_ref = so.chunk_cumsum(dt_raw, 0.7, A_log, 1.1, chunk, bias, True, (0.01, 0.5))
    dA, dt = sc._quant_chunk_cumsum_fwd(cu(dt_raw), 0.7, cu(A_log), 1.1, chunk, cu(bias), True, (0.01, 0.5))
    assert rel_l2(dt, dt_ref) < 1e-6 and (dA.cpu() - dA_ref).abs().max() < 1e-5 * dA_ref.abs().max()
    states = torch.randint(-127, 128, (B, L // chunk, H, dim), generator=g, dtype=torch.int8)
    sp_ref, fin_ref = so.state_passing(states, dA_ref[..., -1])
    dAd = cu(dA_ref)
    for arg in (dAd[..., -1], dAd[..., -1].contiguous()):
        sp, fin = sc._fixedpoint_state_passing_fwd(cu(states), arg)
        passed_states_mismatch(sp, sp_ref, dA_ref[..., -1], "passed states")
        passed_states_mismatch(fin, fin_ref, dA_ref[..., -1], "final state")


@pytest.mark.parametrize("keyside", [False, True])
def test_combined_matches_oracle(keyside):
    from linquant_b200.kernels.mamba2.ssd_combined import _quant_mamba_chunk_scan_combined_fwd as fwd

    k = make_case(B=2, L=1024, H=8, chunk=256, seed=1)
    kw = dict(dt_softplus=True, static_state_scale=k["state_scale"], static_cb_scale=k["cb_scale"], alpha_hp=k["alpha"],
              bscale_g=k["sB"], keyside=keyside, x_scale_hp=k["x_scale"], b_fp=k["Bm"], b_gate_scale=k["b_gate"])
    ref, _ = so.ssd_combined(k["x"], k["dt_raw"], 1.0, k["A_log"], 1.0, k["qB"], k["sB"], k["qC"], k["sC"], 256, k["D"], 1.0, **kw)
    out, none = fwd(cu(k["x"]), cu(k["dt_raw"]), 1.0, cu(k["A_log"]), 1.0, cu(k["qB"]), cu(k["sB"]), cu(k["qC"]), cu(k["sC"]), 256,
                    cu(k["D"]), 1.0, **{n: cu(v) for n, v in kw.items()})
    assert none is None
    err = rel_l2(out, ref)
    assert err < 2e-3, f"combined SSD keyside={keyside}: rel-L2 {err:.2e}"


def test_x_as_strided_view_of_xBC_and_prologue():
    from linquant_b200.kernels.mamba2.chunk_state import _quant_chunk_state_fwd_xfp_static_int8 as cs
    from linquant_b200.kernels.mamba2.fused_split_rotate_xBC import fused_split_rotate_quant_xBC

    H, P, G, N, B, T = 4, 64, 1, 128, 2, 512
    g = torch.Generator().manual_seed(3)
    xBC = torch.randn(B, T, H * P + 2 * G * N, generator=g).half()
    signs = torch.randint(0, 2, (G, N), generator=g).float() * 2 - 1
    dq = torch.rand(G, N, generator=g) + 0.5
    binv = torch.tensor([127.0 / 4.0])
    cinv = torch.tensor([127.0 / 5.0])
    for rs, db, dc in ((signs, dq, 1.0 / dq), (signs, None, None), (None, None, None)):
        x_ref, qB_ref, qC_ref = so.split_rotate_quant(xBC, rs, H, G, N, P, binv, cinv, db, dc)
        x, qB, qC = fused_split_rotate_quant_xBC(xBC.cuda(), cu(rs), H, G, N, P, binv.cuda(), cinv.cuda(), cu(db), cu(dc))
        assert torch.equal(x.cpu(), x_ref) and x.stride(1) == H * P + 2 * G * N
        code_mismatch(qB, qB_ref, "q_B codes")
        code_mismatch(qC, qC_ref, "q_C codes")
    k = make_case(B=B, L=T, H=H, N=N, chunk=256, seed=3)
    st_ref = so.chunk_state_value(x_ref, k["qB"], k["dt"], k["dA"], k["alpha"], k["sB"], k["state_scale"])
    st = cs(x, cu(k["qB"]), cu(k["dt"]), cu(k["dA"]), cu(k["alpha"]), cu(k["sB"]), cu(k["state_scale"]))
    code_mismatch(st, st_ref, "chunk states from a strided x view")


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.bfloat16)])
def test_kronecker_hadamard(D, dtype):
    from linquant_b200.kernels.hadamard import hadamard_matrix, kronecker_hadamard_fwd

    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 100, 3, D, generator=g).to(dtype)
    signs = torch.randint(0, 2, (3, D), generator=g).float() * 2 - 1
    y = kronecker_hadamard_fwd(x.cuda(), signs.cuda(), 3)
    ref = so.kronecker_hadamard(x, signs)
    assert y.dtype == dtype and rel_l2(y, ref) < 1e-3
    exact = (x.float() * signs) @ hadamard_matrix(D)
    assert rel_l2(y, exact) < 1e-2


# ---------------------------------------------------------------------------------------------------------------
# CUDA ops against the golden vectors written by the reference's own Triton kernels (tests/golden/ssd_*.npz)
def _gold(name):
    import os

    import numpy as np

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    return {k: torch.from_numpy(np.ascontiguousarray(z[k])) for k in z.files}


@pytest.mark.parametrize("name", ["ssd_value_n128", "ssd_key_n64"])
def test_ops_match_reference_kernel_golden(name):
    from linquant_b200.kernels.mamba2 import ssd_combined as sc

    g = _gold(name)
    key, C = bool(g["keyside"]), int(g["chunk"])
    one = torch.ones(1).cuda()
    dA, dt = sc._quant_chunk_cumsum_fwd(cu(g["dt_raw"]), one, cu(g["A_log"]), one, C, cu(g["dt_bias"]), True)
    assert float((dt.cpu() - g["dt"]).abs().max()) <= 1e-6
    assert float((dA.cpu() - g["dA"]).abs().max()) <= 2e-4
    dtd, dAd = cu(g["dt"]), cu(g["dA"])
    if key:
        st = sc._chunk_state_keyside_fwd(cu(g["x"]), cu(g["x_scale_hp"]), cu(g["b_fp"]), dtd, dAd, cu(g["state_scale"]),
                                         cu(g["b_gate_scale"]))
    else:
        st = sc._quant_chunk_state_fwd_xfp_static_int8(cu(g["x"]), cu(g["q_B"]), dtd, dAd, cu(g["alpha_hp"]), cu(g["B_scale"]),
                                                       cu(g["state_scale"]))
    code_mismatch(st, g["states"], f"{name}: chunk states vs the reference kernel")
    B, NC, H, P, N = g["states"].shape
    sp, fin = sc._fixedpoint_state_passing_fwd(cu(g["states"]).reshape(B, NC, H, P * N), dAd[..., -1])
    passed_states_mismatch(sp, g["passed"], g["dA"][..., -1], f"{name}: entering states vs the reference kernel")
    passed_states_mismatch(fin, g["final"], g["dA"][..., -1], f"{name}: final state vs the reference kernel")
    cb = sc._quant_bmm_chunk_fwd(cu(g["q_C"]), cu(g["C_scale"]), cu(g["b_fp"] if key else g["q_B"]), cu(g["B_scale"]), C,
                                 cu(g["cb_scale"]), b_is_fp=key)
    code_mismatch(cb, g["cb"], f"{name}: CB codes vs the reference kernel")
    out = sc._chunk_scan_v2(cu(g["cb"]), cu(g["x"]), dtd, dAd, cu(g["q_C"]), cu(g["C_scale"]),
                            cu(g["passed"]).reshape(B, NC, H, P, N), cu(g["D"]), one, cu(g["state_scale"]), cu(g["cb_scale"]))
    err = rel_l2(out, g["out"])
    assert err <= 2e-3, f"{name}: chunk scan rel-L2 {err:.2e} vs the reference kernel"
    if N == 128 and C % 128 == 0:
        for kern in ("tcgen05", "warp_mma"):
            out_tc = sc._chunk_scan_v2(cu(g["cb"]), cu(g["x"]), dtd, dAd, cu(g["q_C"]), cu(g["C_scale"]),
                                       cu(g["passed"]).reshape(B, NC, H, P, N), cu(g["D"]), one, cu(g["state_scale"]), cu(g["cb_scale"]),
                                       kernel=kern)
            err = rel_l2(out_tc, g["out"])
            assert err <= 2e-3, f"{name}: chunk scan ({kern}) rel-L2 {err:.2e} vs the reference kernel"
    full, _ = sc._quant_mamba_chunk_scan_combined_fwd(
        cu(g["x"]), cu(g["dt_raw"]), one, cu(g["A_log"]), one, cu(g["q_B"]), cu(g["B_scale"]), cu(g["q_C"]), cu(g["C_scale"]), C,
        cu(g["D"]), one, dt_bias=cu(g["dt_bias"]), dt_softplus=True, static_state_scale=cu(g["state_scale"]),
        static_cb_scale=cu(g["cb_scale"]), alpha_hp=cu(g["alpha_hp"]), bscale_g=cu(g["B_scale"]), keyside=key,
        x_scale_hp=cu(g["x_scale_hp"]), b_fp=cu(g["b_fp"]), b_gate_scale=cu(g["b_gate_scale"]))
    err = rel_l2(full, g["out"])
    assert err <= 2e-3, f"{name}: combined forward rel-L2 {err:.2e} vs the reference kernels"


@pytest.mark.parametrize("name", ["ssd_split_rotate", "ssd_split_rotate_dqk"])
def test_split_rotate_matches_reference_kernel_golden(name):
    from linquant_b200.kernels.mamba2.fused_split_rotate_xBC import fused_split_rotate_quant_xBC

    g = _gold(name)
    x, qB, qC = fused_split_rotate_quant_xBC(cu(g["xBC"]), cu(g["signs"]), int(g["nheads"]), int(g["G"]), int(g["N"]),
                                             int(g["headdim"]), cu(g["B_inv"]), cu(g["C_inv"]), cu(g.get("dqk_b")),
                                             cu(g.get("dqk_c")))
    assert torch.equal(x.cpu().contiguous(), g["x_view"])
    code_mismatch(qB, g["q_B"], f"{name}: q_B vs the reference kernel")
    code_mismatch(qC, g["q_C"], f"{name}: q_C vs the reference kernel")


@pytest.mark.parametrize("name", ["ssd_kron_hadamard_f16", "ssd_kron_hadamard_bf16"])
def test_kronecker_hadamard_matches_reference_kernel_golden(name):
    import os

    import numpy as np

    from linquant_b200.kernels.hadamard import kronecker_hadamard_fwd

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    bf = bool(z["bf16"])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16) if bf else torch.from_numpy(np.ascontiguousarray(a))  # noqa: E731
    x, s, y = t(z["x"]), t(z["signs"]), t(z["y"])
    got = kronecker_hadamard_fwd(x.cuda(), s.cuda(), x.shape[2]).cpu()
    assert got.dtype == y.dtype
    frac = float((got != y).float().mean())
    assert frac <= 1e-3 and float((got.float() - y.float()).abs().max()) <= 0.04, f"{name}: {frac:.2e} of outputs differ"


@pytest.mark.gpu
@pytest.mark.parametrize("chunk", [128, 256])
def test_bmm_chunk_two_groups_on_the_tensor_core_kernel(chunk):
    """C.B^T at d_state 128 with two groups (the group picks the 128-byte column block of the INT8 rows that the TMA
    box starts at) and a ragged number of chunks: codes bit for bit against the CPU restatement."""
    from linquant_b200.kernels.mamba2 import ssd_combined as sc

    k = make_case(B=2, L=3 * chunk, H=4, G=2, N=128, chunk=chunk, seed=11)
    ref = so.bmm_chunk(k["qC"], k["sC"], k["qB"], k["sB"], chunk, k["cb_scale"])
    got = sc._quant_bmm_chunk_fwd(cu(k["qC"]), cu(k["sC"]), cu(k["qB"]), cu(k["sB"]), chunk, cu(k["cb_scale"]))
    assert got.shape == ref.shape and torch.equal(got.cpu(), ref), "CB codes differ"
    import linquant_b200

    linquant_b200.check_status("cuda")


@pytest.mark.gpu
@pytest.mark.parametrize("chunk,dtype", [(128, torch.float16), (256, torch.bfloat16)])
def test_chunk_states_two_groups_on_the_tensor_core_kernels(chunk, dtype):
    """Value- and key-side chunk states at d_state 128 with two groups of two heads (the head pair of a CTA picks its
    group's B lanes): INT8 state codes against the CPU restatement, and the key side's C.B^T from the unquantised B."""
    from linquant_b200.kernels.mamba2 import ssd_combined as sc

    k = make_case(B=2, L=2 * chunk, H=4, G=2, N=128, chunk=chunk, dtype=dtype, seed=12)
    dtd, dAd = cu(k["dt"]), cu(k["dA"])
    st_ref = so.chunk_state_value(k["x"], k["qB"], k["dt"], k["dA"], k["alpha"], k["sB"], k["state_scale"])
    st = sc._quant_chunk_state_fwd_xfp_static_int8(cu(k["x"]), cu(k["qB"]), dtd, dAd, cu(k["alpha"]), cu(k["sB"]), cu(k["state_scale"]))
    code_mismatch(st, st_ref, "value-side chunk states, two groups")
    stk_ref = so.chunk_state_key(k["x"], k["x_scale"], k["Bm"], k["dt"], k["dA"], k["state_scale"], k["b_gate"])
    stk = sc._chunk_state_keyside_fwd(cu(k["x"]), cu(k["x_scale"]), cu(k["Bm"]), dtd, dAd, cu(k["state_scale"]), cu(k["b_gate"]))
    code_mismatch(stk, stk_ref, "key-side chunk states, two groups")
    cbk_ref = so.bmm_chunk(k["qC"], k["sC"], k["Bm"], k["sB"], chunk, k["cb_scale"], b_is_fp=True)
    cbk = sc._quant_bmm_chunk_fwd(cu(k["qC"]), cu(k["sC"]), cu(k["Bm"]), cu(k["sB"]), chunk, cu(k["cb_scale"]), b_is_fp=True)
    code_mismatch(cbk, cbk_ref, "key-side CB codes, two groups")
    import linquant_b200

    linquant_b200.check_status("cuda")
