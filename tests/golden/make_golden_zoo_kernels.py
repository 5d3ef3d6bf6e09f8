"""Golden outputs of the reference's own INT8 zoo KERNELS (Triton), run on the CPU with Triton's interpreter.

tests/golden/make_golden.py stores what the reference's fake-quant emulation produces; this script adds, for the
same seeded inputs, what the reference's Triton kernels themselves return (output and final fp32 carry), so the
CUDA kernels can be compared with the reference's product path as well as with its emulation. The kernels are run
unmodified; the adaptations of the interpreter and of the GPU-only plumbing around them are those of
tests/golden/make_golden_ssd.py (imported from there).

    TRITON_INTERPRET=1 python tests/golden/make_golden_zoo_kernels.py /path/to/reference

Writes tests/golden/zoo_kernel_*.npz.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import make_golden_ssd  # noqa: E402,F401  (interpreter adaptations; puts the reference on sys.path)
from make_golden import C, H, K, V, case_inputs  # noqa: E402

from linquant.invariances import POLICIES, FakeQuant  # noqa: E402
from linquant.kernels.zoo.gated_delta_rule import chunk_delta_int8  # noqa: E402
from linquant.kernels.zoo.gla import chunk_gla_int8  # noqa: E402
from linquant.kernels.zoo.kda import chunk_kda_int8  # noqa: E402
from linquant.kernels.zoo.simple_gla import chunk_simple_gla_int8  # noqa: E402
from linquant.reference import chunk_core, hadamard_rotation  # noqa: E402

CASES = [
    dict(name="simple_gla_scalar", family="linear", decay="scalar", eta=0.5, sigma=1.0, tau=1.0, rot=False),
    dict(name="simple_gla_none", family="linear", decay="none", eta=1.0, sigma=1.0, tau=1.0, rot=False),
    dict(name="gla_eta0", family="linear", decay="diagonal", eta=0.0, sigma=1.0, tau=1.0, rot=False),
    dict(name="gla_rot_eta05", family="linear", decay="diagonal", eta=0.5, sigma=1.0, tau=1.0, rot=True),
    dict(name="delta_none", family="delta", decay="none", eta=1.0, sigma=1.0, tau=1.0, rot=False),
    dict(name="delta_scalar_s05", family="delta", decay="scalar", eta=1.0, sigma=0.5, tau=0.5, rot=False),
    dict(name="delta_scalar_eta0", family="delta", decay="scalar", eta=0.0, sigma=1.0, tau=1.0, rot=False),
    dict(name="kda_eta0", family="delta", decay="diagonal", eta=0.0, sigma=1.0, tau=1.0, rot=False),
    dict(name="kda_rot_s0", family="delta", decay="diagonal", eta=0.5, sigma=0.0, tau=1.0, rot=True),
]


def cpu_scales(qz, delta):
    """FakeQuant.kernel_scales without its CUDA default for absent roles (invariances.py:102-113), plus the delta
    family's W / E roles as the reference's kernel tests assemble them (tests/test_kernel_delta.py:24-34)."""

    def get(role, shape):
        sc = qz.scales.get((0, role))
        if sc is None:
            return torch.ones(shape, dtype=torch.float32)
        sc = sc.float().clamp_min(1e-6)
        return sc.reshape(shape).contiguous() if sc.numel() > 1 else sc.expand(shape).contiguous()

    s = {"q": get("q_read", (H,)), "k": get("k_local", (H,)), "kw": get("k_write", (H, K)), "state": get("state", (H, V))}
    if delta:
        s.update(w=get("w_read", (H,)), el=get("e_local", (H, V)), ew=get("e_write", (H, V)))
    else:
        s.update(vw=get("v_write", (H, V)), vl=get("v_local", (H, V)))
    return s


def main():
    for c in CASES:
        q, k, v, g, beta = case_inputs(dict(decay=c["decay"], family=c["family"]))
        delta = c["family"] == "delta"
        R = hadamard_rotation(K, 3) if c["rot"] else None
        qz = FakeQuant("none", 8, ["ALL"], dict(POLICIES["kernel_static"]), state_bits=8, round_away=True)
        qz.tie_roles = qz.local_fp16 = qz.kernel_arith = True
        qz.layer = 0
        run = lambda: chunk_core(q, k, v, g, beta, family=c["family"], decay=c["decay"], scale=K**-0.5, qz=qz,  # noqa: E731
                                 rot_qk=R, eta=c["eta"], rho=c["sigma"], tau=c["tau"], read_post=True, C=C)
        qz.calibrating = True
        run()
        qz.finalize()
        emu = run()
        sc = cpu_scales(qz, delta)
        kw = dict(eta=c["eta"], scale=K**-0.5, chunk_size=C, output_final_state=True)
        if c["decay"] == "diagonal":
            if delta:
                o, ht = chunk_kda_int8(q, k, v, g, beta, sc, sigma=c["sigma"], tau=c["tau"], rot=R, fla_prep=False, **kw)
            else:
                o, ht = chunk_gla_int8(q, k, v, g, sc, rot=R, **kw)
        elif delta:
            o, ht = chunk_delta_int8(q, k, v, g, beta, sc, sigma=c["sigma"], tau=c["tau"], fla_prep=False, **kw)
        else:
            o, ht = chunk_simple_gla_int8(q, k, v, g, sc, **kw)
        err = float((o.float() - emu.float()).norm() / emu.float().norm())
        arrays = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), o_kernel=o.numpy(), ht_kernel=ht.numpy(), o_emulation=emu.numpy(),
                      eta=np.array(c["eta"]), sigma=np.array(c["sigma"]), tau=np.array(c["tau"]), rot=np.array(c["rot"]),
                      family=np.array(c["family"]), decay=np.array(c["decay"]))
        if g is not None:
            arrays["g"] = g.numpy()
        if beta is not None:
            arrays["beta"] = beta.numpy()
        if R is not None:
            arrays["R"] = R.float().numpy()
        for n, t in sc.items():
            arrays["ks_" + n] = t.numpy()
        np.savez_compressed(os.path.join(HERE, "zoo_kernel_" + c["name"] + ".npz"), **arrays)
        print(c["name"], "kernel vs emulation rel-L2", f"{err:.2e}", "|o| max", float(o.float().abs().max()))


if __name__ == "__main__":
    main()
