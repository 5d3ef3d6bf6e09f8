"""Sequence-parallel prefill of the linear family (none / scalar decay): the sequence is cut into contiguous segments,
one per GPU, and only the fp32 carry crosses segment boundaries.

Each segment first runs the prologue and the state pass from a zero carry, which gives its end carry S_end and its total
decay Gamma = exp(sum of g). The carry entering segment r is the exclusive scan
    S_in(0) = 0,   S_in(r+1) = Gamma(r) * S_in(r) + S_end(r)
(the recurrence is linear in the carry). One all_gather of S_end [B,H,K,V] and Gamma [B,H] over NCCL delivers what
every rank needs; then the state pass is repeated from S_in and the output kernel runs. The INT8 operand tiles of the
prologue are reused. The fp32 carry is what travels: sending the INT8 copy would change the stored states downstream.
Against a single-GPU run the carries differ by fp32 rounding only (the scan associates differently), so stored-state
codes agree up to rounding-boundary ties.

The reference has no multi-GPU mode; ``segmented_on_one_device`` runs the same two passes for all segments on one GPU."""

from __future__ import annotations

import torch

from . import _cabi
from .kernels.zoo import _common


def incoming_carries(S_end, gamma):
    """S_end [W,B,H,K,V], gamma [W,B,H] -> S_in [W,B,H,K,V] by the exclusive scan above (fp32)."""
    W = S_end.shape[0]
    out = torch.zeros_like(S_end)
    for r in range(1, W):
        out[r] = gamma[r - 1][..., None, None] * out[r - 1] + S_end[r - 1]
    return out


def segment_gamma(g, B, H, device):
    if g is None:
        return torch.ones(B, H, dtype=torch.float32, device=device)
    return g.double().sum(dim=1).exp().float()


class _Segment:
    """One segment's problem descriptor and workspace; pass 1 = prologue + state from zero, pass 2 = state from the
    incoming carry + output."""

    def __init__(self, q, k, v, g, scales, *, eta, scale, chunk_size, bits, rot, dqk, out_dtype):
        B, T, H, K = q.shape
        V = v.shape[-1]
        assert T % chunk_size == 0
        self.q, self.k, self.v = q.contiguous(), k.contiguous(), v.contiguous()
        self.o = torch.empty(v.shape, dtype=out_dtype or v.dtype, device=v.device)
        self.s_end = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device)
        self.keep = []
        self.P = _common.make_problem(self.q, self.k, self.v, g, None, scales,
                                      decay=_cabi.DECAY_NONE if g is None else _cabi.DECAY_SCALAR, eta=eta, sigma=1.0, tau=1.0,
                                      scale=K**-0.5 if scale is None else scale, chunk_size=chunk_size, bits=bits, out=self.o,
                                      final_state=self.s_end, rot_signs=_common.signs_of(rot, K, q.device), dqk=dqk,
                                      keep=self.keep)
        self.ws = _cabi.Workspace(self.P, False, q.device)
        self.gamma = segment_gamma(g, B, H, q.device)

    def pass1(self):
        _common.run_stage("lq_zoo_prologue_linear", self.P, self.ws, self.q)
        _common.run_stage("lq_zoo_state_linear", self.P, self.ws, self.q)
        return self.s_end, self.gamma

    def pass2(self, s_in, final_state=None):
        if s_in is not None:
            s_in = s_in.contiguous()
            self.keep.append(s_in)
            self.P.initial_state = s_in.data_ptr()
            self.P.final_state = None if final_state is None else final_state.data_ptr()
            _common.run_stage("lq_zoo_state_linear", self.P, self.ws, self.q)
        _common.run_stage("lq_zoo_output_scalar", self.P, self.ws, self.q)
        return self.o


def chunk_simple_gla_int8_seqpar(q, k, v, g, scales, *, group=None, eta=1.0, scale=None, chunk_size=64, bits=8, rot=None,
                                 dqk=None, out_dtype=None):
    """This rank's segment of the sequence in, this rank's segment of the output out. q,k,v,g are [B, T/W, H, .] slices
    of the full tensors, rank r holding tokens [r*T/W, (r+1)*T/W). Needs an initialised NCCL process group."""
    import torch.distributed as dist

    seg = _Segment(q, k, v, g, scales, eta=eta, scale=scale, chunk_size=chunk_size, bits=bits, rot=rot, dqk=dqk,
                   out_dtype=out_dtype)
    s_end, gamma = seg.pass1()
    W, r = dist.get_world_size(group), dist.get_rank(group)
    ends = [torch.empty_like(s_end) for _ in range(W)]
    gams = [torch.empty_like(gamma) for _ in range(W)]
    dist.all_gather(ends, s_end, group=group)
    dist.all_gather(gams, gamma, group=group)
    s_in = incoming_carries(torch.stack(ends), torch.stack(gams))[r]
    return seg.pass2(s_in if r > 0 else None)


def segmented_on_one_device(q, k, v, g, scales, nseg, *, eta=1.0, scale=None, chunk_size=64, bits=8, rot=None, dqk=None,
                            out_dtype=None):
    """The same two passes with all ``nseg`` segments on one GPU (what ``nseg`` ranks would do, minus the all_gather)."""
    T = q.shape[1]
    assert T % (nseg * chunk_size) == 0
    L = T // nseg
    cut = lambda t, i: None if t is None else t[:, i * L:(i + 1) * L]  # noqa: E731
    segs = [_Segment(cut(q, i), cut(k, i), cut(v, i), cut(g, i), scales, eta=eta, scale=scale, chunk_size=chunk_size,
                     bits=bits, rot=rot, dqk=dqk, out_dtype=out_dtype) for i in range(nseg)]
    firsts = [s.pass1() for s in segs]
    s_in = incoming_carries(torch.stack([f[0] for f in firsts]), torch.stack([f[1] for f in firsts]))
    return torch.cat([s.pass2(s_in[i] if i > 0 else None) for i, s in enumerate(segs)], dim=1)
