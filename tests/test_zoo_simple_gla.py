"""chunk_simple_gla_int8 (CUDA, through the C ABI) against the CPU oracle: codes, stored states, outputs.

Mirrors tests/test_kernel_simple_gla.py and tests/test_kernel_regimes.py of the reference."""

import pytest
import torch

from tests.helpers import OracleRun, code_mismatch, reference_check, rel_l2, zoo_inputs

pytestmark = pytest.mark.gpu
B, T, H, K, V = 2, 512, 4, 64, 128


def run_case(q, k, v, g, *, policy="kernel_static", bits=8, eta=1.0, rot=False, dqk=None, label=""):
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8
    from oracle import zoo_oracle as zo

    Kd = q.shape[-1]
    R, signs = zo.signed_hadamard(Kd, 3) if rot else (None, None)
    orc = OracleRun(q, k, v, g, None, family="linear", decay="none" if g is None else "scalar", policy=policy, bits=bits,
                    eta=eta, rot_qk=R, dqk=dqk)
    ref, ref_state = orc.lineage()
    exact = orc.exact()
    dbg = {}
    dev = "cuda"
    out, ht = chunk_simple_gla_int8(q.to(dev), k.to(dev), v.to(dev), None if g is None else g.to(dev), orc.scales(dev),
                                    eta=eta, scale=Kd**-0.5, chunk_size=64, bits=bits, output_final_state=True,
                                    rot=signs, dqk=None if dqk is None else dqk.to(dev), _debug=dbg)
    torch.cuda.synchronize()
    ws = dbg["workspace"]
    ws.check_status()
    Bq, Tq, Hq, _ = q.shape
    Vd = v.shape[-1]
    NT = Tq // 64
    tile = lambda name: ws.view(name).view(Bq, Hq, NT, *ws.view(name).shape[2:])  # noqa: E731
    if g is not None:
        assert torch.allclose(tile("gc").cpu(), _oracle_gc(g, Bq, Hq, NT), atol=0, rtol=0), "chunk-local cumsum"
    code_mismatch(tile("qq"), orc.codes("q_read"), f"{label} q codes")
    code_mismatch(tile("kl"), orc.codes("k_local"), f"{label} k_local codes")
    code_mismatch(tile("kwT").transpose(-1, -2), orc.codes("k_write"), f"{label} k_write codes")
    code_mismatch(tile("vlT").transpose(-1, -2), orc.codes("v_local"), f"{label} v_local codes")
    code_mismatch(tile("vwT").transpose(-1, -2), orc.codes("v_write"), f"{label} v_write codes")
    st = orc.codes("state")  # state after chunk c == state entering chunk c+1
    hT = tile("hT").transpose(-1, -2)
    assert int(hT[:, :, 0].abs().max()) == 0, "the state entering chunk 0 is zero"
    if NT > 1:
        code_mismatch(hT[:, :, 1:], st[:, :, :-1], f"{label} stored state codes")
    err = rel_l2(out, ref)
    assert err <= 2e-3, f"{label}: output rel-L2 {err:.3e} vs the quantised emulation"
    reference_check(out, ref, exact, label)
    assert rel_l2(ht, ref_state) <= 1e-4, f"{label}: final fp32 carry"
    return out


def _oracle_gc(g, Bq, Hq, NT):
    return g.view(Bq, NT, 64, Hq).float().cumsum(2).permute(0, 3, 1, 2).contiguous()


@pytest.mark.parametrize("decay", [False, True])
@pytest.mark.parametrize("eta", [1.0, 0.0, 0.5])
def test_kernel_matches_oracle(decay, eta):
    if not decay and eta != 1.0:
        pytest.skip("eta needs a decay")
    q, k, v, g, _ = zoo_inputs(B, T, H, K, V, decay="scalar" if decay else "none")
    run_case(q, k, v, g, eta=eta, label=f"decay={decay} eta={eta}")


@pytest.mark.parametrize("eta", [0.0, 0.5, 1.0])
def test_strong_decay_no_nan(eta):
    q, k, v, g, _ = zoo_inputs(B, T, H, K, V, decay="scalar", gscale=40.0)
    out = run_case(q, k, v, g, eta=eta, label=f"strong decay eta={eta}")
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("policy,bits", [("kernel_pt", 8), ("kernel_pt", 6), ("kernel_ptk", 8), ("kernel_static", 6)])
def test_regime_and_bits(policy, bits):
    q, k, v, g, _ = zoo_inputs(B, T, H, K, V, decay="scalar")
    run_case(q, k, v, g, policy=policy, bits=bits, label=f"{policy} bits={bits}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Kd,Vd", [(128, 128), (64, 64), (128, 64)])
def test_shapes_dtypes_fused_rotation(dtype, Kd, Vd):
    q, k, v, g, _ = zoo_inputs(2, 256, 3, Kd, Vd, decay="scalar", dtype=dtype, seed=1)
    run_case(q, k, v, g, policy="kernel_pt", rot=True, label=f"rot {dtype} K={Kd} V={Vd}")


def test_fused_dqk_and_rotation():
    q, k, v, g, _ = zoo_inputs(2, 256, 2, 128, 128, decay="scalar", dtype=torch.bfloat16, seed=2, normalize_q=False)
    amax_q, amax_k = q.float().abs().amax(dim=(0, 1)), k.float().abs().amax(dim=(0, 1))
    dqk = ((amax_k.clamp_min(1e-8) / amax_q.clamp_min(1e-8)) ** 0.5).float()  # harness.py:68-79 with alpha=0.5
    run_case(q, k, v, g, policy="kernel_ptk", rot=True, dqk=dqk, label="dqk+rot")


def test_single_chunk_and_ragged_batch():
    q, k, v, g, _ = zoo_inputs(3, 64, 5, 64, 64, decay="scalar", seed=3)
    run_case(q, k, v, g, label="single chunk, odd B*H")


def test_shape_errors():
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8

    q, k, v, g, _ = zoo_inputs(1, 96, 2, 64, 64, decay="scalar")
    sc = {n: torch.ones(s, device="cuda") for n, s in (("q", (2,)), ("k", (2,)), ("kw", (2, 64)), ("vw", (2, 64)),
                                                         ("vl", (2, 64)), ("state", (2, 64)))}
    with pytest.raises(AssertionError):
        chunk_simple_gla_int8(q.cuda(), k.cuda(), v.cuda(), g.cuda(), sc)
    q, k, v, g, _ = zoo_inputs(1, 128, 2, 32, 64, decay="scalar")
    sc["kw"] = torch.ones(2, 32, device="cuda")
    with pytest.raises(NotImplementedError):
        chunk_simple_gla_int8(q.cuda(), k.cuda(), v.cuda(), g.cuda(), sc)


def test_initial_state_and_segmented_sequence():
    """A sequence cut into segments (what the sequence-parallel mode does across GPUs): the carry handed from one
    segment to the next reproduces the unsplit run up to fp32 rounding of the carry."""
    from linquant_b200 import seqpar
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8

    q, k, v, g, _ = zoo_inputs(2, 512, 3, 128, 128, decay="scalar", dtype=torch.bfloat16, seed=7)
    orc = OracleRun(q, k, v, g, None, family="linear", decay="scalar", policy="kernel_pt")
    ref = orc.run()
    dev = "cuda"
    sc = orc.scales(dev)
    qd, kd, vd, gd = q.to(dev), k.to(dev), v.to(dev), g.to(dev)
    whole, fs = chunk_simple_gla_int8(qd, kd, vd, gd, sc, output_final_state=True)
    # two calls chained through initial_state
    a, sa = chunk_simple_gla_int8(qd[:, :256], kd[:, :256], vd[:, :256], gd[:, :256], sc, output_final_state=True)
    b, sb = chunk_simple_gla_int8(qd[:, 256:], kd[:, 256:], vd[:, 256:], gd[:, 256:], sc, output_final_state=True,
                                  initial_state=sa)
    assert torch.equal(torch.cat([a, b], 1), whole) and torch.equal(sb, fs), "chained calls reproduce the unsplit call exactly"
    # four segments with the exclusive scan of the carries
    seg = seqpar.segmented_on_one_device(qd, kd, vd, gd, sc, 4)
    assert rel_l2(seg, whole) <= 1e-3 and rel_l2(seg, ref) <= 2e-3, f"{rel_l2(seg, whole):.2e} {rel_l2(seg, ref):.2e}"


def test_host_pipeline_matches_device_call():
    from linquant_b200.host_pipeline import SimpleGlaHostPipeline
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8

    q, k, v, g, _ = zoo_inputs(3, 256, 2, 128, 128, decay="scalar", dtype=torch.bfloat16, seed=8)
    orc = OracleRun(q, k, v, g, None, family="linear", decay="scalar", policy="kernel_pt")
    sc = orc.scales("cuda")
    want, _ = chunk_simple_gla_int8(q.cuda(), k.cuda(), v.cuda(), g.cuda(), sc)
    pipe = SimpleGlaHostPipeline(3, 256, 2, 128, 128, torch.bfloat16, "cuda")
    ho = torch.empty(v.shape, dtype=v.dtype).pin_memory()
    for _ in range(2):
        pipe(q.pin_memory(), k.pin_memory(), v.pin_memory(), g.pin_memory(), sc, ho)
        torch.cuda.synchronize()
        assert torch.equal(ho, want.cpu())


@pytest.mark.parametrize("decay", [False, True])
@pytest.mark.parametrize("n,Vd,dtype", [(128, 128, torch.float16), (512, 128, torch.float16), (256, 64, torch.bfloat16)])
def test_canonical_storage_rv(decay, n, Vd, dtype):
    """R_V with canonical storage (tests/test_kernel_simple_gla.py:84-104 of the reference): v is rotated in torch, the
    kernels un-rotate the write product before the fp32 carry and the local product before the output, so the stored
    INT8 state and the output are canonical."""
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8
    from oracle import zoo_oracle as zo

    q, k, v, g, _ = zoo_inputs(B, n, H, K, Vd, decay="scalar" if decay else "none", dtype=dtype)
    R, _ = zo.signed_hadamard(Vd, 7)
    orc = OracleRun(q, k, v, g, None, family="linear", decay="scalar" if decay else "none", eta=1.0, rot_v=R,
                    storage="canonical")
    ref, ref_state = orc.lineage()
    exact = orc.exact()
    vr = (v.double() @ R).to(dtype)
    dbg = {}
    out, ht = chunk_simple_gla_int8(q.cuda(), k.cuda(), vr.cuda(), None if g is None else g.cuda(), orc.scales("cuda"),
                                    eta=1.0, scale=K**-0.5, chunk_size=64, output_final_state=True, unrot=R.T.cuda(),
                                    _debug=dbg)
    torch.cuda.synchronize()
    ws = dbg["workspace"]
    NT = n // 64
    hT = ws.view("hT").view(B, H, NT, Vd, K).transpose(-1, -2)
    st = orc.codes("state")
    assert int(hT[:, :, 0].abs().max()) == 0
    code_mismatch(hT[:, :, 1:], st[:, :, :-1], "canonical stored state codes", budget=2e-3)
    label = f"canonical R_V decay={decay} T={n} V={Vd}"
    err = rel_l2(out, ref)
    assert err <= 2e-3, f"{label}: output rel-L2 {err:.3e}"
    reference_check(out, ref, exact, label)
    assert rel_l2(ht, ref_state) <= 1e-3, f"{label}: final fp32 carry {rel_l2(ht, ref_state):.2e}"
