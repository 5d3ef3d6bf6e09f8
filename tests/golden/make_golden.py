"""Generate the golden vectors under tests/golden/ from the reference implementation itself.

Run where the reference checkout is importable (pass its path as the first argument); the GPU machines only see
the committed ``.npz`` files. Every case stores the seeded inputs, the calibrated scales and the output of the
reference's ``linquant.reference.chunk_core`` driven by ``linquant.invariances.FakeQuant`` in kernel-lineage
mode, which is what the reference's own kernel tests compare their kernels against
(``tests/test_kernel_simple_gla.py:41-60`` and siblings).

    python tests/golden/make_golden.py <path-to-reference-checkout>
"""

import itertools
import os
import sys

import numpy as np
import torch

CASES = []
for family, decay in itertools.product(("linear", "delta"), ("none", "scalar", "diagonal")):
    CASES.append(dict(family=family, decay=decay, policy="kernel_static", rot_qk=False, eta=1.0 if decay == "none" else 0.5,
                      sigma=1.0, tau=1.0))
    CASES.append(dict(family=family, decay=decay, policy="kernel_ptk" if family == "delta" else "kernel_pt", rot_qk=True,
                      eta=1.0, sigma=0.5, tau=0.5))

B, T, H, K, V, C = 1, 128, 2, 64, 64, 64


def case_name(c):
    return f"{c['family']}_{c['decay']}_{c['policy']}_rot{int(c['rot_qk'])}"


def case_inputs(c, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, K, generator=g), dim=-1).half()
    k = torch.nn.functional.normalize(torch.randn(B, T, H, K, generator=g), dim=-1).half()
    v = torch.randn(B, T, H, V, generator=g).half()
    if c["decay"] == "scalar":
        gd = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=g) * 3) / 4).float()
    elif c["decay"] == "diagonal":
        gd = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, generator=g) * 3) / 4).float()
    else:
        gd = None
    beta = torch.rand(B, T, H, generator=g).float() if c["family"] == "delta" else None
    return q, k, v, gd, beta


def main():
    sys.path.insert(0, sys.argv[1])
    from linquant.invariances import POLICIES, FakeQuant
    from linquant.reference import chunk_core, hadamard_rotation

    here = os.path.dirname(os.path.abspath(__file__))
    for c in CASES:
        q, k, v, g, beta = case_inputs(c)
        R = hadamard_rotation(K, 3) if c["rot_qk"] else None
        qz = FakeQuant("none", 8, ["ALL"], dict(POLICIES[c["policy"]]), state_bits=8, round_away=True)
        qz.tie_roles = qz.local_fp16 = qz.kernel_arith = True
        qz.layer = 0
        run = lambda: chunk_core(q, k, v, g, beta, family=c["family"], decay=c["decay"], scale=K**-0.5, qz=qz,  # noqa: E731
                                 rot_qk=R, eta=c["eta"], rho=c["sigma"], tau=c["tau"], read_post=True, C=C,
                                 out_dtype=torch.float32)
        qz.calibrating = True
        run()
        qz.finalize()
        o = run()
        arrays = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), o=o.numpy())
        if g is not None:
            arrays["g"] = g.numpy()
        if beta is not None:
            arrays["beta"] = beta.numpy()
        for (_, role), s in qz.scales.items():
            arrays["scale_" + role] = s.numpy()
        np.savez_compressed(os.path.join(here, case_name(c) + ".npz"), **arrays)
        print(case_name(c), float(o.abs().max()))


if __name__ == "__main__":
    main()
