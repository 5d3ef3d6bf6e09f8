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


# ----------------------------------------------------------------------------------------------------------------
# Mamba-2 SSD (SSDi8 lineage): the carry of the inter-chunk recurrence is an unclamped INT32 tensor, so handing THAT
# from the GPU that holds segment r to the GPU that holds segment r+1 reproduces the one-GPU result bit for bit.
# Every rank runs cumsum / chunk state / C.B^T of its own segment at once; the fixed-point state passing then forms a
# chain: rank r's kernel waits (bounded) for its local flags, runs its chunks, and stores its final carry and the
# flags straight into rank r+1's receive buffer over NVLink (plain stores into a CUDA-IPC mapping of memory that
# lives on the consumer GPU); the chunk scans run at once again.
import ctypes as _C


def _flag_count(B, H, D):
    return B * H * ((D // 8 + 255) // 256)


class _DevArray:
    """A raw device allocation seen as a tensor (``torch.as_tensor`` reads ``__cuda_array_interface__``)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SsdLink:
    """One rank's end of the hand-off chain for a fixed (B, H, P*N): a receive buffer in this GPU's memory (int32 carry
    followed by one flag per state-passing CTA) and, unless this is the last rank, the mapping of the next rank's
    buffer. Construction is collective over ``group`` (the IPC handles travel by ``all_gather_object``); ``local=True``
    builds the chain inside one process on one GPU instead (every segment's buffer is a local tensor), which is how a
    single device runs all segments one after the other."""

    def __init__(self, B, H, D, device, group=None, wait_ns=0, _local_next=None, _local_first=False, local=False):
        import torch.distributed as dist

        self.B, self.H, self.D = B, H, D
        self.device = torch.device(device)
        self.wait_ns = int(wait_ns)
        self.epoch = 0
        self.carry_bytes = B * H * D * 4
        self.nbytes = self.carry_bytes + _flag_count(B, H, D) * 4
        self._own_ptr = self._next_ptr = None
        self._lib = _cabi.lib()
        if local:
            self.rank, self.world = (0 if _local_first else 1), 2
            self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.recv_ptr = self.buf.data_ptr()
            self.next_ptr = None if _local_next is None else _local_next.recv_ptr
            self.is_first, self.is_last = _local_first, _local_next is None
            return
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.is_first, self.is_last = self.rank == 0, self.rank == self.world - 1
        handle = (_C.c_ubyte * 64)()
        ptr = _C.c_void_p()
        fn = self._lib.lq_peer_buffer_create
        fn.argtypes = [_C.c_size_t, _C.POINTER(_C.c_void_p), _C.POINTER(_C.c_ubyte)]
        with torch.cuda.device(self.device):
            _cabi.check(fn(self.nbytes, _C.byref(ptr), handle), "lq_peer_buffer_create")
        self._own_ptr = self.recv_ptr = ptr.value
        self.buf = torch.as_tensor(_DevArray(self.recv_ptr, self.nbytes), device=self.device)
        handles = [None] * self.world
        dist.all_gather_object(handles, (bytes(handle), self.device.index), group=group)
        self.next_ptr = None
        if not self.is_last:
            h, owner = handles[self.rank + 1]
            nxt = _C.c_void_p()
            op = self._lib.lq_peer_buffer_open
            op.argtypes = [_C.POINTER(_C.c_ubyte), _C.c_int, _C.POINTER(_C.c_void_p)]
            with torch.cuda.device(self.device):
                _cabi.check(op((_C.c_ubyte * 64).from_buffer_copy(h), owner, _C.byref(nxt)), "lq_peer_buffer_open")
            self._next_ptr = self.next_ptr = nxt.value
        dist.barrier(group)

    def next_call(self):
        """A new forward pass: the flags of the previous one stay where they are and simply become stale."""
        self.epoch += 1

    def apply(self, call, B, H, dim):
        assert (B, H, dim) == (self.B, self.H, self.D), "the link was built for another problem shape"
        assert self.epoch >= 1, "call next_call() once per forward pass before the state passing"
        p = call.p
        call.keep.append(self.buf)
        if not self.is_first:
            p.carry_in = self.recv_ptr
            p.wait_flags = self.recv_ptr + self.carry_bytes
        if self.next_ptr is not None:
            p.carry_out = self.next_ptr
            p.post_flags = self.next_ptr + self.carry_bytes
        p.epoch = self.epoch
        p.wait_ns = self.wait_ns

    def close(self):
        if self._next_ptr:
            fn = self._lib.lq_peer_buffer_close
            fn.argtypes = [_C.c_void_p]
            fn(self._next_ptr)
            self._next_ptr = None
        if self._own_ptr:
            torch.cuda.synchronize(self.device)
            self.buf = None
            fn = self._lib.lq_peer_buffer_destroy
            fn.argtypes = [_C.c_void_p]
            fn(self._own_ptr)
            self._own_ptr = None


def ssd_combined_seqpar(link, x_fp, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale, chunk_size, q_D, D_scale,
                        **kw):
    """``_quant_mamba_chunk_scan_combined_fwd`` on this rank's segment of the sequence (tokens
    [rank*L/W, (rank+1)*L/W) of every tensor with a token axis; L/W a multiple of the chunk size). The only exchange is
    the INT32 carry of the state passing, written by the previous rank's kernel into this rank's receive buffer. Returns
    (out segment, None); equal, bit for bit, to the same rows of the single-GPU result."""
    from .kernels.mamba2 import ssd_combined as sc

    link.next_call()
    return sc._quant_mamba_chunk_scan_combined_fwd(x_fp, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale,
                                                   chunk_size, q_D, D_scale, _link=link, **kw)


def ssd_segmented_on_one_device(nseg, x_fp, q_dt, dt_scale, q_A_log, A_log_scale, q_B, B_scale, q_C, C_scale, chunk_size, q_D,
                                D_scale, **kw):
    """All ``nseg`` segments on one GPU, one after the other on the current stream: the same kernels and the same
    carry / flag traffic as ``nseg`` ranks, with local buffers in place of the peer mappings."""
    B, L, H, P = x_fp.shape
    N = q_B.shape[-1]
    assert L % (nseg * chunk_size) == 0
    S = L // nseg
    links, nxt = [], None
    for i in reversed(range(nseg)):
        nxt = SsdLink(B, H, P * N, x_fp.device, local=True, _local_next=nxt, _local_first=(i == 0))
        links.append(nxt)
    links.reverse()
    cut = lambda t, i: t[:, i * S:(i + 1) * S]  # noqa: E731
    outs = []
    for i, link in enumerate(links):
        kws = dict(kw)
        if kws.get("b_fp") is not None:
            kws["b_fp"] = cut(kws["b_fp"], i)
        o, _ = ssd_combined_seqpar(link, cut(x_fp, i), cut(q_dt, i), dt_scale, q_A_log, A_log_scale, cut(q_B, i), B_scale,
                                   cut(q_C, i), C_scale, chunk_size, q_D, D_scale, **kws)
        outs.append(o)
    return torch.cat(outs, dim=1)
