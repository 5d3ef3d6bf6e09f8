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


class SsdStackHostPipeline:
    """Host-buffer entry for a stack of Mamba-2 SSD layers: every layer's xBC and dt arrive in pinned host memory and its
    output leaves to pinned host memory, with the copies of neighbouring layers overlapped with the kernels of the
    current one (copy-in stream, compute on the caller's stream, copy-out stream; two device slots each way).

    ``run(layers)`` takes objects with the per-layer constants (``A_log``, ``D``, ``signs``, ``B_inv``, ``C_inv``,
    ``scales``) and uses the pipeline's own pinned ring as the host side of every layer: layer i reads host slot i % 2 and
    writes host output slot i % 2. ``forward`` is the per-layer product path (prologue + combined SSD forward)."""

    def __init__(self, B, L, dims, device, depth=2):
        H, P, N, G = dims["H"], dims["P"], dims["N"], dims["G"]
        self.dims, self.device, self.depth = dims, torch.device(device), depth
        width = H * P + 2 * G * N
        self.h_xBC = [torch.randn(B, L, width).to(torch.bfloat16).pin_memory() for _ in range(depth)]
        self.h_dt = [(torch.randn(B, L, H) * 0.5 - 2.0).pin_memory() for _ in range(depth)]
        self.h_out = [torch.empty(B, L, H, P, dtype=torch.float16).pin_memory() for _ in range(depth)]
        self.d_xBC = [torch.empty(B, L, width, dtype=torch.bfloat16, device=self.device) for _ in range(depth)]
        self.d_dt = [torch.empty(B, L, H, dtype=torch.float32, device=self.device) for _ in range(depth)]
        self.copy_stream, self.out_stream = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.loaded = [torch.cuda.Event() for _ in range(depth)]
        self.consumed = [torch.cuda.Event() for _ in range(depth)]
        self.stored = [torch.cuda.Event() for _ in range(depth)]
        self.h2d_bytes_per_layer = self.h_xBC[0].numel() * 2 + self.h_dt[0].numel() * 4
        self.d2h_bytes_per_layer = self.h_out[0].numel() * 2

    def forward(self, layer, xBC, dt_raw):
        from .kernels.mamba2 import ssd_combined as sc
        from .kernels.mamba2.fused_split_rotate_xBC import fused_split_rotate_quant_xBC

        d, S = self.dims, layer.scales
        x, qB, qC = fused_split_rotate_quant_xBC(xBC, layer.signs, d["H"], d["G"], d["N"], d["P"], layer.B_inv, layer.C_inv)
        out, _ = sc._quant_mamba_chunk_scan_combined_fwd(
            x, dt_raw, 1.0, layer.A_log, 1.0, qB, S["B_scale"], qC, S["C_scale"], d["C"], layer.D, 1.0, dt_softplus=True,
            static_state_scale=S["state_scale"], static_cb_scale=S["cb_scale"], alpha_hp=S["alpha_hp"], bscale_g=S["B_scale"])
        return out

    def run(self, layers):
        main = torch.cuda.current_stream(self.device)
        self.copy_stream.wait_stream(main)
        self.out_stream.wait_stream(main)
        for i, layer in enumerate(layers):
            s = i % self.depth
            with torch.cuda.stream(self.copy_stream):
                if i >= self.depth:
                    self.copy_stream.wait_event(self.consumed[s])
                self.d_xBC[s].copy_(self.h_xBC[s], non_blocking=True)
                self.d_dt[s].copy_(self.h_dt[s], non_blocking=True)
                self.loaded[s].record(self.copy_stream)
            main.wait_event(self.loaded[s])
            out = self.forward(layer, self.d_xBC[s], self.d_dt[s])
            self.consumed[s].record(main)
            with torch.cuda.stream(self.out_stream):
                self.out_stream.wait_event(self.consumed[s])
                if i >= self.depth:
                    self.out_stream.wait_event(self.stored[s])
                self.h_out[s].copy_(out, non_blocking=True)
                out.record_stream(self.out_stream)
                self.stored[s].record(self.out_stream)
        main.wait_stream(self.out_stream)
        return self.h_out
