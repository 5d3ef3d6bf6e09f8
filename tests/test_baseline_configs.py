"""Parity at the sizes of the benchmark configurations, through the C ABI, against the CPU oracles.

* configuration 0 (the Mamba-2 SSD written as the linear / scalar-decay cell: q = C, k = B, v = x dt, g = dt A, scale 1,
  plus the D x skip) at its full size;
* one full-length batch element, all heads, of configurations 1 (Simple GLA), 2 (Gated DeltaNet) and 3 (KDA), with each
  configuration's policy, rotation, D_QK rescale and outliers;
* a layer slice of configuration 4 (bf16, 80 heads, d_state 128, chunk 256, x20 heavy channels) on every SSD sub-op and
  on the combined forward.

Scales come from further seeded batches of the same distribution (absmax), never from the measured batch. Operand and
stored-state codes must match bit for bit, rounding-boundary ties excepted: the fraction of differing codes is printed
per role and bounded by 0.1 %, each by one step. Outputs: relative L2 <= 2e-3 against the quantised emulation."""

import math

import pytest
import torch
import torch.nn.functional as F

from tests.helpers import OracleRun, code_mismatch, passed_states_mismatch, reference_check, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _batches(name, seeds, B, T):
    from linquant_b200.synthetic import make_inputs

    return [make_inputs(name, seed=s, B=B, T=T) for s in seeds]


def _tuple(x):
    return (x["q"], x["k"], x["v"], x["g"], x["beta"])


def _tiles(ws, name, B, H, NT):
    t = ws.view(name)
    return t.view(B, H, NT, *t.shape[2:])


def _report(label, fr, err):
    print(f"\n{label}: fraction of codes off by one step per role "
          + ", ".join(f"{k} {v:.2e}" for k, v in fr.items()) + f"; output rel-L2 {err:.2e}")


def test_config0_mamba2_as_linear_scalar_cell_full_size():
    """B=1, H=8, P=V=64, N=K=64, L=2048, chunk 64, kernel_static, R_QK on the state axis, INT8 state."""
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8
    from linquant_b200.synthetic import CONFIGS
    from oracle import zoo_oracle as zo

    cfg = CONFIGS["mamba2_small"]
    x = _batches("mamba2_small", [100], cfg["B"], cfg["T"])[0]
    calib = [_tuple(b) for b in _batches("mamba2_small", [101, 102, 103, 104], cfg["B"], cfg["T"])]
    B, T, H, K, V = cfg["B"], cfg["T"], cfg["H"], cfg["K"], cfg["V"]
    R, signs = zo.signed_hadamard(K, 0)
    orc = OracleRun(*_tuple(x), family="linear", decay="scalar", policy="kernel_static", eta=1.0, rot_qk=R, scale=1.0, calib=calib)
    ref, ref_state = orc.lineage()
    exact = orc.exact()
    dbg = {}
    out, ht = chunk_simple_gla_int8(x["q"].to(DEV), x["k"].to(DEV), x["v"].to(DEV), x["g"].to(DEV), orc.scales(DEV), eta=1.0,
                                    scale=1.0, chunk_size=64, output_final_state=True, rot=signs, _debug=dbg)
    torch.cuda.synchronize()
    ws = dbg["workspace"]
    ws.check_status()
    NT = T // 64
    fr = {}
    fr["q_read"] = code_mismatch(_tiles(ws, "qq", B, H, NT), orc.codes("q_read"), "cfg0 q codes")
    fr["k_local"] = code_mismatch(_tiles(ws, "kl", B, H, NT), orc.codes("k_local"), "cfg0 k_local codes")
    fr["k_write"] = code_mismatch(_tiles(ws, "kwT", B, H, NT).transpose(-1, -2), orc.codes("k_write"), "cfg0 k_write codes")
    fr["v_local"] = code_mismatch(_tiles(ws, "vlT", B, H, NT).transpose(-1, -2), orc.codes("v_local"), "cfg0 v_local codes")
    fr["v_write"] = code_mismatch(_tiles(ws, "vwT", B, H, NT).transpose(-1, -2), orc.codes("v_write"), "cfg0 v_write codes")
    hT = _tiles(ws, "hT", B, H, NT).transpose(-1, -2)
    fr["state"] = code_mismatch(hT[:, :, 1:], orc.codes("state")[:, :, :-1], "cfg0 stored state codes")
    # the D x skip of the SSD is a host-side epilogue of this mapping: same fp32 arithmetic on both sides
    g = torch.Generator().manual_seed(7)
    D = torch.randn(H, generator=g)
    xs = torch.randn(B, T, H, V, generator=g)
    y = out.float().cpu() + D.view(1, 1, H, 1) * xs
    y_ref = ref.float() + D.view(1, 1, H, 1) * xs
    err = rel_l2(out, ref)
    _report("configuration 0", fr, err)
    assert err <= 2e-3 and rel_l2(y, y_ref) <= 2e-3
    reference_check(out, ref, exact, "cfg0")
    assert rel_l2(ht, ref_state) <= 1e-4


def test_config1_simple_gla_one_full_length_batch_element():
    """H=16, K=V=128, L=4096, bf16, kernel_pt, fused R_QK, eta=1: 4096 chunk tiles, the prologue's persistent grid
    walks more tiles than it has CTAs."""
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8
    from linquant_b200.synthetic import CONFIGS
    from oracle import zoo_oracle as zo

    cfg = CONFIGS["simple_gla"]
    H, K, V, T = cfg["H"], cfg["K"], cfg["V"], cfg["T"]
    x = _batches("simple_gla", [200], 1, T)[0]
    calib = [_tuple(b) for b in _batches("simple_gla", [201, 202, 203, 204], 1, 1024)]
    R, signs = zo.signed_hadamard(K, 0)
    orc = OracleRun(*_tuple(x), family="linear", decay="scalar", policy="kernel_pt", eta=1.0, rot_qk=R, calib=calib)
    ref, ref_state = orc.lineage()
    dbg = {}
    out, ht = chunk_simple_gla_int8(x["q"].to(DEV), x["k"].to(DEV), x["v"].to(DEV), x["g"].to(DEV), orc.scales(DEV), eta=1.0,
                                    output_final_state=True, rot=signs, _debug=dbg)
    torch.cuda.synchronize()
    ws = dbg["workspace"]
    ws.check_status()
    NT = T // 64
    fr = {}
    fr["q_read"] = code_mismatch(_tiles(ws, "qq", 1, H, NT), orc.codes("q_read"), "cfg1 q codes")
    fr["k_local"] = code_mismatch(_tiles(ws, "kl", 1, H, NT), orc.codes("k_local"), "cfg1 k_local codes")
    fr["k_write"] = code_mismatch(_tiles(ws, "kwT", 1, H, NT).transpose(-1, -2), orc.codes("k_write"), "cfg1 k_write codes")
    fr["v_local"] = code_mismatch(_tiles(ws, "vlT", 1, H, NT).transpose(-1, -2), orc.codes("v_local"), "cfg1 v_local codes")
    fr["v_write"] = code_mismatch(_tiles(ws, "vwT", 1, H, NT).transpose(-1, -2), orc.codes("v_write"), "cfg1 v_write codes")
    hT = _tiles(ws, "hT", 1, H, NT).transpose(-1, -2)
    fr["state"] = code_mismatch(hT[:, :, 1:], orc.codes("state")[:, :, :-1], "cfg1 stored state codes")
    err = rel_l2(out, ref)
    _report("configuration 1 (one batch element)", fr, err)
    assert err <= 2e-3
    assert rel_l2(ht, ref_state) <= 1e-4


def test_config2_gated_deltanet_one_full_length_batch_element():
    """H=16, K=V=128, L=8192, bf16, kernel_ptk, D_QK with sqk=0.5 from a statistics pass, sigma=0.5, tau=1, fused R_QK."""
    from linquant_b200 import invariances as inv
    from linquant_b200.kernels.zoo.gated_delta_rule import chunk_delta_int8
    from linquant_b200.synthetic import CONFIGS
    from oracle import zoo_oracle as zo

    cfg = CONFIGS["gated_deltanet"]
    H, K, V, T = cfg["H"], cfg["K"], cfg["V"], cfg["T"]
    x = _batches("gated_deltanet", [300], 1, T)[0]
    cal = _batches("gated_deltanet", [301, 302, 303, 304], 1, 1024)
    dqk = inv.dqk_from_stats(torch.cat([b["q"] for b in cal]), torch.cat([b["k"] for b in cal]), cfg["sqk"])
    R, signs = zo.signed_hadamard(K, 0)
    orc = OracleRun(*_tuple(x), family="delta", decay="scalar", policy="kernel_ptk", eta=1.0, sigma=cfg["sigma"], tau=cfg["tau"],
                    rot_qk=R, dqk=dqk, calib=[_tuple(b) for b in cal])
    ref, ref_state = orc.lineage()
    dbg = {}
    out, ht = chunk_delta_int8(x["q"].to(DEV), x["k"].to(DEV), x["v"].to(DEV), x["g"].to(DEV), x["beta"].to(DEV), orc.scales(DEV),
                               sigma=cfg["sigma"], tau=cfg["tau"], eta=1.0, output_final_state=True, rot=signs, dqk=dqk.to(DEV),
                               _debug=dbg)
    torch.cuda.synchronize()
    ws = dbg["workspace"]
    ws.check_status()
    NT = T // 64
    fr = {}
    fr["q_read"] = code_mismatch(_tiles(ws, "qq", 1, H, NT), orc.codes("q_read"), "cfg2 q codes")
    fr["k_local"] = code_mismatch(_tiles(ws, "kl", 1, H, NT), orc.codes("k_local"), "cfg2 Hw local codes")
    fr["k_write"] = code_mismatch(_tiles(ws, "kwT", 1, H, NT).transpose(-1, -2), orc.codes("k_write"), "cfg2 Hw write codes")
    fr["w_read"] = code_mismatch(_tiles(ws, "wq", 1, H, NT), orc.codes("w_read"), "cfg2 W codes")
    fr["e_local"] = code_mismatch(_tiles(ws, "vlT", 1, H, NT).transpose(-1, -2), orc.codes("e_local"), "cfg2 E local codes")
    hT = _tiles(ws, "hT", 1, H, NT).transpose(-1, -2)
    upstream_ties = fr["e_local"] > 0 or fr["w_read"] > 0  # a flipped E / W code moves the state by several grid steps
    fr["state"] = code_mismatch(hT[:, :, 1:], orc.codes("state")[:, :, :-1], "cfg2 stored state codes", max_step=4 if upstream_ties else 1)
    err = rel_l2(out, ref)
    _report("configuration 2 (one batch element)", fr, err)
    assert err <= 2e-3
    assert rel_l2(ht, ref_state) <= 1e-3


def test_config3_kda_one_full_length_batch_element():
    """H=32, K=V=128, L=8192, bf16, per-channel decay, 1 % of the key channels x20, kernel_static, local R_QK."""
    from linquant_b200.kernels.zoo.kda import chunk_kda_int8
    from linquant_b200.synthetic import CONFIGS
    from oracle import zoo_oracle as zo

    cfg = CONFIGS["kda"]
    H, K, V, T = cfg["H"], cfg["K"], cfg["V"], cfg["T"]
    x = _batches("kda", [400], 1, T)[0]
    calib = [_tuple(b) for b in _batches("kda", [401, 402, 403, 404], 1, 512)]
    R, signs = zo.signed_hadamard(K, 0)
    orc = OracleRun(*_tuple(x), family="delta", decay="diagonal", policy="kernel_static", eta=0.0, sigma=1.0, tau=1.0, rot_qk=R,
                    calib=calib)
    ref, ref_state = orc.lineage()
    dbg = {}
    out, ht = chunk_kda_int8(x["q"].to(DEV), x["k"].to(DEV), x["v"].to(DEV), x["g"].to(DEV), x["beta"].to(DEV), orc.scales(DEV),
                             sigma=1.0, tau=1.0, eta=0.0, output_final_state=True, rot=signs, _debug=dbg)
    torch.cuda.synchronize()
    ws = dbg["workspace"]
    ws.check_status()
    NT = T // 64
    fr = {}
    fr["q_read"] = code_mismatch(_tiles(ws, "qq", 1, H, NT), orc.codes("q_read"), "cfg3 q_read codes")
    fr["k_write"] = code_mismatch(_tiles(ws, "kwT", 1, H, NT).transpose(-1, -2), orc.codes("k_write"), "cfg3 k_write codes")
    fr["w_read"] = code_mismatch(_tiles(ws, "wq", 1, H, NT), orc.codes("w_read"), "cfg3 W codes")
    fr["e_local"] = code_mismatch(_tiles(ws, "vlT", 1, H, NT).transpose(-1, -2), orc.codes("e_local"), "cfg3 E local codes")
    hT = _tiles(ws, "hT", 1, H, NT).transpose(-1, -2)
    upstream_ties = fr["e_local"] > 0 or fr["w_read"] > 0  # a flipped E / W code moves the state by several grid steps
    fr["state"] = code_mismatch(hT[:, :, 1:], orc.codes("state")[:, :, :-1], "cfg3 stored state codes", max_step=4 if upstream_ties else 1)
    err = rel_l2(out, ref)
    _report("configuration 3 (one batch element)", fr, err)
    assert err <= 2e-3
    assert rel_l2(ht, ref_state) <= 1e-3


# ---------------------------------------------------------------------------------------------------------------
def mamba2_layer_case(B, L, H, P, G, N, chunk, seed, dtype=torch.bfloat16, heavy=0.01):
    """One layer's post-conv operands in the distribution of configuration 4: x, B, C ~ N(0,1) with `heavy` of the
    channels x20, dt = softplus(N(-2, 0.5)) (passed raw, softplus in the op), A = -exp(U(0, ln 16)), D ~ N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H * P, generator=g)
    Bm = torch.randn(B, L, G, N, generator=g)
    Cm = torch.randn(B, L, G, N, generator=g)
    for t, width in ((x, H * P), (Bm, N), (Cm, N)):
        idx = torch.randperm(width, generator=g)[: max(1, int(round(heavy * width)))]
        t[..., idx] *= 20.0
    dt_raw = torch.randn(B, L, H, generator=g) * 0.5 - 2.0
    A_log = torch.rand(H, generator=g) * math.log(16.0)
    D = torch.randn(H, generator=g)
    return dict(x=x.view(B, L, H, P).to(dtype), Bm=Bm.to(dtype), Cm=Cm.to(dtype), dt_raw=dt_raw, A_log=A_log, D=D)


def test_config4_layer_slice_every_sub_op_and_combined():
    """bf16, H=80, P=64, N=128, G=1, chunk 256, L=4096, B=1; scales from the observers on four further batches."""
    from linquant_b200.kernels.mamba2 import _ssd
    from linquant_b200.kernels.mamba2 import ssd_combined as sc
    from linquant_b200.kernels.mamba2.calibration import SsdObservers
    from oracle import ssd_oracle as so

    B, L, H, P, G, N, C = 1, 4096, 80, 64, 1, 128, 256
    obs = SsdObservers()
    for s in (501, 502, 503, 504):
        k = mamba2_layer_case(1, 1024, H, P, G, N, C, s)
        obs.observe(k["x"], k["dt_raw"], k["A_log"], k["Bm"], k["Cm"], C)
    S = obs.scales()
    k = mamba2_layer_case(B, L, H, P, G, N, C, 500)
    qB = torch.round(k["Bm"].float() / S["B_scale"].view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    qC = torch.round(k["Cm"].float() / S["C_scale"].view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    cu = lambda t: t.to(DEV) if torch.is_tensor(t) else t  # noqa: E731
    dA_ref, dt_ref = so.chunk_cumsum(k["dt_raw"], 1.0, k["A_log"], 1.0, C, None, True)
    dA, dt = sc._quant_chunk_cumsum_fwd(cu(k["dt_raw"]), 1.0, cu(k["A_log"]), 1.0, C, None, True)
    assert rel_l2(dt, dt_ref) < 1e-6 and (dA.cpu() - dA_ref).abs().max() < 1e-5 * dA_ref.abs().max()
    dtd, dAd = cu(dt_ref), cu(dA_ref)
    fr = {}
    st_ref = so.chunk_state_value(k["x"], qB, dt_ref, dA_ref, S["alpha_hp"], S["B_scale"], S["state_scale"])
    st = sc._quant_chunk_state_fwd_xfp_static_int8(cu(k["x"]), cu(qB), dtd, dAd, cu(S["alpha_hp"]), cu(S["B_scale"]), cu(S["state_scale"]))
    fr["states (value side)"] = code_mismatch(st, st_ref, "cfg4 value-side chunk states")
    stk_ref = so.chunk_state_key(k["x"], S["x_scale_hp"], k["Bm"], dt_ref, dA_ref, S["state_scale"], S["b_gate_scale"])
    stk = sc._chunk_state_keyside_fwd(cu(k["x"]), cu(S["x_scale_hp"]), cu(k["Bm"]), dtd, dAd, cu(S["state_scale"]), cu(S["b_gate_scale"]))
    fr["states (key side)"] = code_mismatch(stk, stk_ref, "cfg4 key-side chunk states")
    nc = L // C
    sp_ref, fin_ref = so.state_passing(st_ref.reshape(B, nc, H, P * N), dA_ref[..., -1])
    sp, fin = sc._fixedpoint_state_passing_fwd(cu(st_ref).reshape(B, nc, H, P * N), dAd[..., -1])
    ties, nd = passed_states_mismatch(sp, sp_ref, dA_ref[..., -1], "cfg4 passed states")
    passed_states_mismatch(fin, fin_ref, dA_ref[..., -1], "cfg4 final state")
    fr["passed states (gate codes on a rounding boundary: %d)" % ties] = nd / sp_ref.numel()
    cb_ref = so.bmm_chunk(qC, S["C_scale"], qB, S["B_scale"], C, S["cb_scale"])
    cb = sc._quant_bmm_chunk_fwd(cu(qC), cu(S["C_scale"]), cu(qB), cu(S["B_scale"]), C, cu(S["cb_scale"]))
    fr["CB"] = code_mismatch(cb, cb_ref, "cfg4 CB codes")
    passed = sp_ref.reshape(B, nc, H, P, N)
    out_ref = so.chunk_scan(cb_ref, k["x"], dt_ref, dA_ref, qC, S["C_scale"], passed, k["D"], 1.0, S["state_scale"], S["cb_scale"])
    errs = {}
    for kern in ("warp_mma", "tcgen05", None):
        out = sc._chunk_scan_v2(cu(cb_ref), cu(k["x"]), dtd, dAd, cu(qC), cu(S["C_scale"]), cu(passed), cu(k["D"]), 1.0,
                                cu(S["state_scale"]), cu(S["cb_scale"]), kernel=kern)
        errs[str(kern)] = rel_l2(out, out_ref)
    for keyside in (False, True):
        kw = dict(dt_softplus=True, static_state_scale=S["state_scale"], static_cb_scale=S["cb_scale"], alpha_hp=S["alpha_hp"],
                  bscale_g=S["B_scale"], keyside=keyside, x_scale_hp=S["x_scale_hp"], b_fp=k["Bm"], b_gate_scale=S["b_gate_scale"])
        ref, _ = so.ssd_combined(k["x"], k["dt_raw"], 1.0, k["A_log"], 1.0, qB, S["B_scale"], qC, S["C_scale"], C, k["D"], 1.0, **kw)
        full, _ = sc._quant_mamba_chunk_scan_combined_fwd(cu(k["x"]), cu(k["dt_raw"]), 1.0, cu(k["A_log"]), 1.0, cu(qB), cu(S["B_scale"]),
                                                          cu(qC), cu(S["C_scale"]), C, cu(k["D"]), 1.0, **{n: cu(v) for n, v in kw.items()})
        errs[f"combined keyside={keyside}"] = rel_l2(full, ref)
    _ssd.check_status(DEV)
    print("\nconfiguration 4 layer slice: fraction of codes off by one step "
          + ", ".join(f"{n} {v:.2e}" for n, v in fr.items()) + "; output rel-L2 " + ", ".join(f"{n} {v:.2e}" for n, v in errs.items()))
    assert all(e <= 2e-3 for e in errs.values()), errs


@pytest.mark.gpu
def test_config4_full_size_layer_properties():
    """One layer at the full size of configuration 4 (B=8, L=16384, H=80, P=64, N=128, chunk 256, bf16), where the CPU
    restatement would take hours: properties that do not depend on the size instead. (i) the forward is deterministic;
    (ii) a batch element evaluated alone equals its rows of the full call bit for bit (no exchange across the batch);
    (iii) the sequence evaluated as four chained segments, the INT32 carry handed from one to the next, equals the
    single call bit for bit; (iv) no device-side wait ran out. The persistent chunk scan walks 40 960 items here."""
    from linquant_b200 import check_status
    from linquant_b200.kernels.mamba2 import ssd_combined as sc
    from linquant_b200.kernels.mamba2.calibration import SsdObservers
    from linquant_b200.seqpar import ssd_segmented_on_one_device

    B, L, H, P, G, N, C = 8, 16384, 80, 64, 1, 128, 256
    obs = SsdObservers()
    for s in (601, 602):
        k = mamba2_layer_case(1, 1024, H, P, G, N, C, s)
        obs.observe(k["x"], k["dt_raw"], k["A_log"], k["Bm"], k["Cm"], C)
    S = {n: (v.to(DEV) if torch.is_tensor(v) else v) for n, v in obs.scales().items()}
    g = torch.Generator(device=DEV).manual_seed(600)
    x = torch.randn(B, L, H, P, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    x[..., 7] *= 20.0
    qB = torch.randint(-127, 128, (B, L, G, N), generator=g, device=DEV, dtype=torch.int32).to(torch.int8)
    qC = torch.randint(-127, 128, (B, L, G, N), generator=g, device=DEV, dtype=torch.int32).to(torch.int8)
    dt_raw = torch.randn(B, L, H, generator=g, device=DEV) * 0.5 - 2.0
    A_log = torch.rand(H, generator=g, device=DEV) * math.log(16.0)
    D = torch.randn(H, generator=g, device=DEV)
    kw = dict(dt_softplus=True, static_state_scale=S["state_scale"], static_cb_scale=S["cb_scale"], alpha_hp=S["alpha_hp"],
              bscale_g=S["B_scale"])

    def fwd(sl=slice(None)):
        o, _ = sc._quant_mamba_chunk_scan_combined_fwd(x[sl], dt_raw[sl], 1.0, A_log, 1.0, qB[sl], S["B_scale"], qC[sl], S["C_scale"],
                                                       C, D, 1.0, **kw)
        return o

    full = fwd()
    assert full.shape == (B, L, H, P) and bool(torch.isfinite(full.float()).all())
    assert torch.equal(fwd(), full), "two runs of the same call differ"
    assert torch.equal(fwd(slice(5, 6)), full[5:6]), "a batch element alone differs from its rows of the full call"
    seg = ssd_segmented_on_one_device(4, x, dt_raw, 1.0, A_log, 1.0, qB, S["B_scale"], qC, S["C_scale"], C, D, 1.0, **kw)
    assert torch.equal(seg, full), "four chained segments differ from the single call"
    check_status(DEV)
