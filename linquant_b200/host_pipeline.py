"""Host-buffer entry for the chunk prefill: pinned host tensors in, pinned host tensor out, with the copies of one
batch element overlapped with the kernels of another.

Static scales make batch elements independent (every scale is indexed by head), so the batch is cut into single
elements that flow through a two-deep pipeline on two CUDA streams: while element i computes, element i+1 is being
copied host->device and the output of element i-1 device->host. The result is bit-identical to one call on the
whole batch."""

from __future__ import annotations

import torch

from .kernels.zoo.simple_gla import chunk_simple_gla_int8


class SimpleGlaHostPipeline:
    """Reusable device staging for ``chunk_simple_gla_int8`` on host tensors of a fixed shape."""

    def __init__(self, B, T, H, K, V, dtype, device, depth=2):
        self.shape = (B, T, H, K, V)
        self.device = torch.device(device)
        self.depth = min(depth, B)
        mk = lambda *s, dt=dtype: torch.empty(*s, dtype=dt, device=self.device)  # noqa: E731
        self.slots = [dict(q=mk(1, T, H, K), k=mk(1, T, H, K), v=mk(1, T, H, V), g=mk(1, T, H, dt=torch.float32))
                      for _ in range(self.depth)]
        self.copy_stream = torch.cuda.Stream(self.device)
        self.out_stream = torch.cuda.Stream(self.device)
        self.loaded = [torch.cuda.Event() for _ in range(self.depth)]
        self.consumed = [torch.cuda.Event() for _ in range(self.depth)]

    def __call__(self, hq, hk, hv, hg, scales, ho, **kw):
        """hq, hk [B,T,H,K], hv [B,T,H,V], hg [B,T,H] pinned host tensors; ho [B,T,H,V] pinned host output."""
        B = self.shape[0]
        main = torch.cuda.current_stream(self.device)
        self.copy_stream.wait_stream(main)
        self.out_stream.wait_stream(main)
        done = []
        for i in range(B):
            s = i % self.depth
            slot = self.slots[s]
            with torch.cuda.stream(self.copy_stream):
                if i >= self.depth:
                    self.copy_stream.wait_event(self.consumed[s])
                slot["q"].copy_(hq[i:i + 1], non_blocking=True)
                slot["k"].copy_(hk[i:i + 1], non_blocking=True)
                slot["v"].copy_(hv[i:i + 1], non_blocking=True)
                slot["g"].copy_(hg[i:i + 1], non_blocking=True)
                self.loaded[s].record(self.copy_stream)
            main.wait_event(self.loaded[s])
            out, _ = chunk_simple_gla_int8(slot["q"], slot["k"], slot["v"], slot["g"], scales, **kw)
            self.consumed[s].record(main)
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.out_stream):
                self.out_stream.wait_event(ev)
                ho[i:i + 1].copy_(out, non_blocking=True)
                out.record_stream(self.out_stream)
            done.append(out)
        main.wait_stream(self.out_stream)
        return ho
