"""Golden vectors for the Mamba-2 SSD ops, produced by the reference's own Triton kernels.

The reference implements these ops only as Triton kernels. They are executed here on the CPU with Triton's
interpreter (``TRITON_INTERPRET=1``), which runs the unmodified kernel bodies with numpy arithmetic, so no GPU is
needed. Six things outside the kernels are adapted for a CPU run, none of which touches reference code:
``torch.cuda.device`` (the wrappers enter it with the tensor's device index, None for a CPU tensor) becomes a null
context, and the autotuner's timing run (it needs a GPU driver) returns a constant so that the first listed
configuration is used (the results do not depend on the tile configuration beyond fp32 summation order); and a stub
stands in for the GPU driver object that one module queries for its backend name at import; and
``libdevice.rint`` (CUDA-only, not known to the interpreter) is bound to ``np.rint``, the same IEEE round-half-even; and the interpreter's matrix product, which
would multiply the raw bit patterns of bf16 operands, first widens them to fp32 (exact), and its fp32 -> bf16 cast, which truncates, rounds to nearest even as the GPU's
conversion does.

Run from the repository root, with the reference checkout on disk:

    TRITON_INTERPRET=1 python tests/golden/make_golden_ssd.py /path/to/reference

Writes tests/golden/ssd_*.npz (inputs and every intermediate and final tensor).
"""

import contextlib
import os
import sys
import types

import numpy as np
import torch
import triton
import triton.language as tl

assert os.environ.get("TRITON_INTERPRET") == "1", "run with TRITON_INTERPRET=1"
if len(sys.argv) < 2:
    raise SystemExit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden_ssd.py /path/to/reference")
REF = sys.argv[1]
sys.path.insert(0, REF)
torch.cuda.device = lambda *a, **k: contextlib.nullcontext()
import triton.runtime.autotuner as _ta  # noqa: E402
import triton.runtime.interpreter as _ti  # noqa: E402

_ta.Autotuner._bench = lambda self, *a, config=None, **k: [0.0, 0.0, 0.0]
os.environ["FLA_CACHE_RESULTS"] = "0"  # no on-disk autotune cache (its key asks the driver for the device)


class _NoGpuDriver:
    """Stands in for Triton's GPU driver: one reference module asks for the target's backend name on import."""

    def get_current_target(self):
        return types.SimpleNamespace(backend="cuda", arch=100, warp_size=32)


triton.runtime.driver.set_active(_NoGpuDriver())


def _rint(x, _semantic=None):
    """libdevice.rint for the interpreter (which implements tl.* but not libdevice): IEEE round-half-even = np.rint."""
    from triton.runtime.interpreter import TensorHandle

    return tl.tensor(TensorHandle(np.rint(x.handle.data), x.dtype.scalar), x.type)


tl.extra.cuda.libdevice.rint = _rint


def _dot_with_bf16(self, a, b, d, input_precision, max_num_imprecise_acc):
    """The interpreter keeps bf16 as raw uint16 and would multiply the bit patterns; widen them to fp32 first
    (exact), then accumulate in the accumulator's dtype as its own create_dot does."""
    from triton.runtime.interpreter import TensorHandle

    def widen(t):
        return (t.data.astype(np.uint32) << 16).view(np.float32) if t.dtype == tl.bfloat16 else t.data

    return TensorHandle(np.matmul(widen(a), widen(b), dtype=d.data.dtype) + d.data, d.dtype.scalar)


_ti.InterpreterBuilder.create_dot = _dot_with_bf16
_cast_impl = _ti.InterpreterBuilder.cast_impl


def _cast_rne(self, src, dst_type):
    """fp32 -> bf16 as the GPU converts (round to nearest even); the interpreter's own cast truncates."""
    if src.dtype.scalar == tl.float32 and dst_type.scalar == tl.bfloat16:
        bits = np.ascontiguousarray(src.data).view(np.uint32).astype(np.uint64)
        out = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
        return _ti.TensorHandle(out, dst_type.scalar)
    return _cast_impl(self, src, dst_type)


_ti.InterpreterBuilder.cast_impl = _cast_rne
for _n in ("create_fp_trunc",):
    setattr(_ti.InterpreterBuilder, _n, lambda self, src, dst_type: self.cast_impl(src, dst_type))

from linquant.kernels import hadamard as ref_had  # noqa: E402
from linquant.kernels.mamba2 import fused_split_rotate_xBC as ref_split  # noqa: E402
from linquant.kernels.mamba2 import ssd_combined as ref  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def npy(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()  # raw bits; the loader views them back
    return t.numpy()


def ssd_case(name, *, seed, B, L, H, P, G, N, C, keyside, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    x = rn(B, L, H, P)
    x[..., ::17] *= 6.0  # a few heavy channels
    x = x.to(dtype)
    Bm, Cm = rn(B, L, G, N), rn(B, L, G, N)
    dt_raw = rn(B, L, H) * 0.5 - 2.0
    dt_bias = rn(H) * 0.1
    A_log = torch.rand(H, generator=g) * 2.7
    D = rn(H)
    one = torch.ones(1)
    B_scale = (Bm.abs().amax(dim=(0, 1, 3)) / 127).contiguous()
    C_scale = (Cm.abs().amax(dim=(0, 1, 3)) / 127).contiguous()
    q_B = torch.round(Bm / B_scale.view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)
    q_C = torch.round(Cm / C_scale.view(1, 1, G, 1)).clamp(-127, 127).to(torch.int8)

    dA, dt = ref._quant_chunk_cumsum_fwd(dt_raw, one, A_log, one, C, dt_bias=dt_bias, dt_softplus=True)
    # calibration-like scales from a float pass over the same data
    nc = L // C
    gate = torch.exp(dA[..., -1:] - dA) * dt  # [B,H,NC,C]
    xg = x.float().view(B, nc, C, H, P).permute(0, 3, 1, 2, 4) * gate[..., None]
    Bf = (q_B.float() * B_scale.view(1, 1, G, 1)).view(B, nc, C, G, N).permute(0, 3, 1, 2, 4)
    Bh = Bf.repeat_interleave(H // G, dim=1)
    st_f = torch.einsum("bhclp,bhcln->bhcpn", xg, Bh)
    state_scale = (st_f.abs().amax(dim=(0, 2, 4)) * 1.5 / 127).clamp_min(1e-6).contiguous()  # [H,P]
    alpha_hp = (xg.abs().amax(dim=(0, 2, 3)) / 127).clamp_min(1e-6).contiguous()  # [H,P]
    x_scale_hp = (x.float().abs().amax(dim=(0, 1)) / 127).clamp_min(1e-6).contiguous()  # [H,P]
    b_fp = Bm.to(dtype)
    bg = b_fp.float().view(B, nc, C, G, N).permute(0, 3, 1, 2, 4).repeat_interleave(H // G, dim=1) * gate[..., None]
    b_gate_scale = bg.abs().amax(dim=(0, 2, 3, 4)).clamp_min(1e-6).view(1, 1, H, 1).contiguous()  # (B,C,H,N) broadcast
    Cf = (q_C.float() * C_scale.view(1, 1, G, 1)).view(B, nc, C, G, N)
    Bsrc = b_fp.float().view(B, nc, C, G, N) if keyside else Bf.permute(0, 2, 3, 1, 4)
    cb_f = torch.einsum("bclgn,bcsgn->bcgls", Cf, Bsrc)
    cb_scale = (cb_f.abs().amax(dim=(0, 1, 3, 4)) / 127).clamp_min(1e-6).contiguous()  # [G]

    if keyside:
        states = ref._chunk_state_keyside_fwd(x, x_scale_hp, b_fp, dt, dA, state_scale, b_gate_scale)
    else:
        states = ref._quant_chunk_state_fwd_xfp_static_int8(x, q_B, dt, dA, alpha_hp, B_scale, state_scale)
    passed, final = ref._fixedpoint_state_passing_fwd(states.reshape(B, -1, H, P * N), dA[:, :, :, -1],
                                                      gate_shift=ref._GATE_SHIFT)
    cb = ref._quant_bmm_chunk_fwd(q_C, C_scale, b_fp if keyside else q_B, B_scale, C, cb_scale, b_is_fp=keyside)
    out = ref._chunk_scan_v2(cb, x, dt, dA, q_C, C_scale, passed.reshape(B, -1, H, P, N), D, one, state_scale, cb_scale)
    out2, _ = ref._quant_mamba_chunk_scan_combined_fwd(
        x, dt_raw, one, A_log, one, q_B, B_scale, q_C, C_scale, C, D, one, dt_bias=dt_bias, dt_softplus=True,
        static_state_scale=state_scale, static_cb_scale=cb_scale, alpha_hp=alpha_hp, bscale_g=B_scale, keyside=keyside,
        x_scale_hp=x_scale_hp, b_fp=b_fp, b_gate_scale=b_gate_scale)
    assert torch.equal(out, out2), "the orchestrator and the op-by-op chain must agree"
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"), keyside=np.array(keyside), chunk=np.array(C), x=npy(x), dt_raw=npy(dt_raw),
        dt_bias=npy(dt_bias), A_log=npy(A_log), D=npy(D), q_B=npy(q_B), q_C=npy(q_C), B_scale=npy(B_scale),
        C_scale=npy(C_scale), b_fp=npy(b_fp), state_scale=npy(state_scale), alpha_hp=npy(alpha_hp),
        x_scale_hp=npy(x_scale_hp), b_gate_scale=npy(b_gate_scale), cb_scale=npy(cb_scale), dA=npy(dA), dt=npy(dt),
        states=npy(states), passed=npy(passed), final=npy(final), cb=npy(cb), out=npy(out))
    print(name, "out", tuple(out.shape), "|out| max", float(out.float().abs().max()),
          "state code absmax", int(states.abs().max()), "cb code absmax", int(cb.abs().max()))


def rotate_case(name, *, seed, Bn, T, nheads, headdim, G, N, with_dqk):
    g = torch.Generator().manual_seed(seed)
    d_ssm = nheads * headdim
    xBC = (torch.randn(Bn, T, d_ssm + 2 * G * N, generator=g) * 1.5).to(torch.float16)
    signs = (torch.randint(0, 2, (G, N), generator=g) * 2 - 1).to(torch.float16)
    B_inv = (torch.rand(G, generator=g) * 20 + 20).float()
    C_inv = (torch.rand(G, generator=g) * 20 + 20).float()
    dqk_b = dqk_c = None
    if with_dqk:
        d = torch.exp(torch.randn(G * N, generator=g) * 0.3).float()
        dqk_b, dqk_c = ref_split.prepare_dqk(1.0 / d), ref_split.prepare_dqk(d)
    xv, q_B, q_C = ref_split.fused_split_rotate_quant_xBC(xBC, signs, nheads, G, N, headdim, B_inv, C_inv, dqk_b, dqk_c)
    extra = {}
    if with_dqk:
        extra = dict(dqk_b=npy(dqk_b.float()), dqk_c=npy(dqk_c.float()))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), xBC=npy(xBC), signs=npy(signs), B_inv=npy(B_inv),
                        C_inv=npy(C_inv), nheads=np.array(nheads), headdim=np.array(headdim), G=np.array(G),
                        N=np.array(N), x_view=npy(xv.contiguous()), q_B=npy(q_B), q_C=npy(q_C), **extra)
    print(name, "codes absmax", int(q_B.abs().max()), int(q_C.abs().max()))


def hadamard_case(name, *, seed, Bn, T, H, D, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Bn, T, H, D, generator=g).to(dtype)
    signs = (torch.randint(0, 2, (H, D), generator=g) * 2 - 1).to(dtype)
    y = ref_had.kronecker_hadamard_fwd(x, signs, H)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=npy(x), signs=npy(signs), y=npy(y),
                        bf16=np.array(dtype == torch.bfloat16))
    print(name, "|y| max", float(y.float().abs().max()))


if __name__ == "__main__":
    ssd_case("ssd_value_n128", seed=11, B=1, L=512, H=2, P=64, G=1, N=128, C=128, keyside=False)
    ssd_case("ssd_key_n64", seed=12, B=2, L=256, H=2, P=64, G=1, N=64, C=64, keyside=True)
    rotate_case("ssd_split_rotate", seed=13, Bn=1, T=48, nheads=2, headdim=64, G=1, N=128, with_dqk=False)
    rotate_case("ssd_split_rotate_dqk", seed=14, Bn=1, T=48, nheads=2, headdim=64, G=2, N=64, with_dqk=True)
    hadamard_case("ssd_kron_hadamard_f16", seed=15, Bn=1, T=40, H=2, D=128, dtype=torch.float16)
    hadamard_case("ssd_kron_hadamard_bf16", seed=16, Bn=1, T=40, H=3, D=64, dtype=torch.bfloat16)
