"""The reference's own INT8 zoo kernels as the yardstick.

tests/golden/zoo_kernel_*.npz hold, for seeded inputs, what the reference's Triton kernels return (output and final
fp32 carry) when run with Triton's interpreter on the CPU (tests/golden/make_golden_zoo_kernels.py). The CPU part
checks the oracle's kernel-lineage emulation against them; the GPU part checks the CUDA kernels, through the C
ABI, against the very same vectors with the scales the reference kernels were given."""

import glob
import os

import numpy as np
import pytest
import torch

from tests.helpers import OracleRun, rel_l2

GOLD = os.path.join(os.path.dirname(__file__), "golden")
NAMES = sorted(os.path.basename(p)[len("zoo_kernel_"):-4] for p in glob.glob(os.path.join(GOLD, "zoo_kernel_*.npz")))

OUT_TOL = 2e-3  # rel-L2 of the output against the reference kernel (fp16 outputs, rounding-order ties in the codes)
CARRY_TOL = 1e-3  # rel-L2 of the final fp32 carry; cells without decay never forget a flipped code
CARRY_TOL_NO_DECAY = 5e-3


def load(name):
    z = np.load(os.path.join(GOLD, f"zoo_kernel_{name}.npz"))
    g = {k: (torch.from_numpy(np.ascontiguousarray(z[k])) if z[k].dtype.kind in "fiu" and z[k].ndim else z[k]) for k in z.files}
    g["family"], g["decay"] = str(z["family"]), str(z["decay"])
    for s in ("eta", "sigma", "tau"):
        g[s] = float(z[s])
    g["rot"] = bool(z["rot"])
    return g


def test_fixtures_present():
    assert len(NAMES) == 9, NAMES


@pytest.mark.parametrize("name", NAMES)
def test_oracle_lineage_matches_reference_kernel(name):
    g = load(name)
    R = g["R"].double() if g["rot"] else None
    orc = OracleRun(g["q"], g["k"], g["v"], g.get("g"), g.get("beta"), family=g["family"], decay=g["decay"],
                    policy="kernel_static", eta=g["eta"], sigma=g["sigma"], tau=g["tau"], rot_qk=R)
    # the oracle calibrates itself exactly as the reference run did: its kernel scales must be the stored ones
    sc = orc.scales("cpu")
    for n in sc:
        if "ks_" + n in g:
            assert torch.allclose(sc[n].float(), g["ks_" + n].float(), rtol=1e-6, atol=0), f"scale {n}"
    o, carry = orc.lineage(record=False)
    assert rel_l2(o.to(torch.float16), g["o_kernel"]) <= 2e-4
    tol = CARRY_TOL_NO_DECAY if g["decay"] == "none" else CARRY_TOL
    assert rel_l2(carry, g["ht_kernel"]) <= tol


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_cuda_matches_reference_kernel(name):
    from linquant_b200.kernels.zoo.gated_delta_rule import chunk_delta_int8
    from linquant_b200.kernels.zoo.gla import chunk_gla_int8
    from linquant_b200.kernels.zoo.kda import chunk_kda_int8
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8

    g = load(name)
    dev = "cuda"
    d = lambda n: g[n].to(dev) if n in g else None  # noqa: E731
    sc = {n[3:]: g[n].to(dev) for n in g if n.startswith("ks_")}
    K = g["q"].shape[-1]
    kw = dict(eta=g["eta"], scale=K**-0.5, chunk_size=64, output_final_state=True)
    R = g["R"].to(dev) if g["rot"] else None
    delta = g["family"] == "delta"
    if g["decay"] == "diagonal":
        if delta:
            o, ht = chunk_kda_int8(d("q"), d("k"), d("v"), d("g"), d("beta"), sc, sigma=g["sigma"], tau=g["tau"], rot=R, **kw)
        else:
            o, ht = chunk_gla_int8(d("q"), d("k"), d("v"), d("g"), sc, rot=R, **kw)
    elif delta:
        o, ht = chunk_delta_int8(d("q"), d("k"), d("v"), d("g"), d("beta"), sc, sigma=g["sigma"], tau=g["tau"], **kw)
    else:
        o, ht = chunk_simple_gla_int8(d("q"), d("k"), d("v"), d("g"), sc, **kw)
    torch.cuda.synchronize()
    assert o.dtype == g["o_kernel"].dtype
    err, cerr = rel_l2(o, g["o_kernel"]), rel_l2(ht, g["ht_kernel"])
    tol = CARRY_TOL_NO_DECAY if g["decay"] == "none" else CARRY_TOL
    print(f"{name}: output rel-L2 {err:.2e}, carry rel-L2 {cerr:.2e} vs the reference kernel")
    assert err <= OUT_TOL, f"{name}: output rel-L2 {err:.3e} vs the reference kernel"
    assert cerr <= tol, f"{name}: final carry rel-L2 {cerr:.3e} vs the reference kernel"
