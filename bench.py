#!/usr/bin/env python
"""INT8 chunk-prefill benchmark: Mtokens/s through the Mamba-2 2.7B-shaped SSD stack on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the largest single-GPU configuration): 64 layers of random-init Mamba-2 mixers' SSD region, nheads 80,
headdim 64, d_state 128, one group, chunk 256, batch 8, L 16384, bf16 operands with 1 % heavy channels (x20), INT8
operands and INT8 inter-chunk states, value-side absorption. One step = the 64 layers back to back, each layer being
the fused split / rotate / quantise prologue on xBC followed by the combined SSD forward (chunk cumsum, chunk state,
fixed-point state passing, C.B^T, chunk scan): 7 kernels per layer, 448 per step. Inputs are synthetic (seeded per
layer and batch element) and resident in HBM; scales come from absmax observers on four further seeded batches.

With N GPUs the SAME problem is sharded over batch x heads (whole batch elements per rank up to 8 ranks), no data-path
collective: strong scaling. Rank 0 prints one JSON line. The line also carries `per_config`: the other benchmark
configurations (Simple GLA, Gated DeltaNet, KDA, and the key-side variant of the Mamba-2 layer) at full size, each with
its stage times and roofline fractions, sharded the same way.

`--impl reference` times the reference's own CPU implementation of the path (the float64 recurrence, from oracle/_ref
when that was built, else its restatement oracle/zoo_oracle.py) on the host cores, on a bounded sample of the workload.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M2 = dict(layers=64, B=8, L=16384, H=80, P=64, N=128, G=1, C=256)
WORKLOAD = ("mamba2_2.7b_ssd_stack 64 layers x (B=8 L=16384 H=80 P=64 N=128 G=1 chunk=256) bf16 x/B/C, 1% heavy channels x20, "
            "INT8 operands + INT8 states, value-side absorption")

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per head-token of the two largest Mamba-2 layer kernels, from
# one ncu capture of each at B=2, L=8192 (1 310 720 head-tokens per launch: 354.78 MB and 206.56 MB). The traffic of these
# kernels grows in proportion to the (batch, chunk, head) items they walk, so a launch of the bench moves this figure
# times its head-tokens.
NCU_DRAM_BYTES_PER_HEAD_TOKEN = {"chunk_scan": 354.78e6 / 1310720, "chunk_state": 206.56e6 / 1310720}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 20 ms from the warm-up to the end of the timed regions
    (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self, ngpus):
        if self.p is None:
            return None
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                if int(parts[0]) >= ngpus:
                    continue
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        if not sm:
            return None
        busy = [s for s in sm if s >= 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------------
# Mamba-2 stack: synthetic layers, calibration, the step
def m2_algorithmic_bytes(keyside=False):
    """Per head-token, each kernel's own inputs read once and outputs written once; `path` = a layer's inputs and
    output only (x, dt, B and C lanes shared by the 80 heads, out)."""
    H, P, N, C = M2["H"], M2["P"], M2["N"], M2["C"]
    st = P * N / C
    b = {
        "path": 2 * P + 2 * P + 4 + 2 * (2 * N) / H,
        "prologue": (2 * 2 * N + 2 * N) / H,
        "chunk_cumsum": 4 + 8,
        "chunk_state": 2 * P + N / H + 8 + st + (0 if keyside else 2 * N / H),  # + the transposed copy of q_B (written, read)
        "state_passing": 2 * st,
        "bmm_chunk": (2 * N + C) / H,
        "chunk_scan": 2 * P + 2 * P + st + 8 + (N + C) / H,
    }
    if keyside:
        b["chunk_state"] = 2 * P + 2 * N / H + 8 + st  # b_fp (bf16) instead of the INT8 codes
        b["hadamard_B"] = (2 * N + 2 * N) / H
    return b


M2_INT8_OPS = {"chunk_state": 2 * 64 * 128, "chunk_scan": 2 * 128 * 64, "bmm_chunk": 2 * 256 * 128 / 80}  # per head-token


def m2_draw(seed, L, heavy, dev):
    """One batch element of a layer's post-conv operands: xBC ~ N(0,1) bf16 with the `heavy` channels x20, raw dt ~
    N(-2, 0.5) (the softplus is part of the op)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    width = M2["H"] * M2["P"] + 2 * M2["G"] * M2["N"]
    t = torch.randn(L, width, generator=g, device=dev)
    t[:, heavy] *= 20.0
    return t.to(torch.bfloat16), torch.randn(L, M2["H"], generator=g, device=dev) * 0.5 - 2.0


class M2Layer:
    """One layer's operands on the device: xBC (x | B | C lanes, bf16), raw dt, A_log, D, rotation signs, scales. Seeds
    are per (layer, batch element), so a batch shard holds the same data on any number of GPUs."""

    def __init__(self, layer, batch_ids, dev, L=None, segment=None):
        """segment = (r, W): keep only tokens [r L/W, (r+1) L/W) of every batch element (sequence-parallel mode)."""
        H, P, N, G = M2["H"], M2["P"], M2["N"], M2["G"]
        L = L or M2["L"]
        width = H * P + 2 * G * N
        self.layer = layer
        gl = torch.Generator(device=dev).manual_seed(7_000_000 + layer)
        self.A_log = torch.rand(H, generator=gl, device=dev) * math.log(16.0)
        self.D = torch.randn(H, generator=gl, device=dev)
        self.signs = (torch.randint(0, 2, (G, N), generator=gl, device=dev).float() * 2 - 1)
        self.heavy = torch.randperm(width, generator=gl, device=dev)[: max(1, round(0.01 * width))]
        lo, hi = (0, L) if segment is None else (segment[0] * (L // segment[1]), (segment[0] + 1) * (L // segment[1]))
        self.xBC = torch.empty(len(batch_ids), hi - lo, width, dtype=torch.bfloat16, device=dev)
        self.dt_raw = torch.empty(len(batch_ids), hi - lo, H, dtype=torch.float32, device=dev)
        for i, b in enumerate(batch_ids):
            xb, db = m2_draw(1_000_003 * layer + b, L, self.heavy, dev)
            self.xBC[i], self.dt_raw[i] = xb[lo:hi], db[lo:hi]
        self.scales = None

    def calibrate(self, dev, batches=4, Lc=1024):
        """absmax scales from `batches` further seeded batches of the same distribution (one element of Lc tokens each)."""
        from linquant_b200.kernels.hadamard import kronecker_hadamard_fwd
        from linquant_b200.kernels.mamba2.calibration import SsdObservers

        H, P, N, G, C = M2["H"], M2["P"], M2["N"], M2["G"], M2["C"]
        obs = SsdObservers()
        for s in range(batches):
            xBC, dt_raw = m2_draw(900_000_000 + 1000 * self.layer + s, Lc, self.heavy, dev)
            xBC, dt_raw = xBC.unsqueeze(0), dt_raw.unsqueeze(0)
            x = xBC[..., : H * P].reshape(1, Lc, H, P)
            Bf = kronecker_hadamard_fwd(xBC[..., H * P: H * P + G * N].reshape(1, Lc, G, N).contiguous(), self.signs, G)
            Cf = kronecker_hadamard_fwd(xBC[..., H * P + G * N:].reshape(1, Lc, G, N).contiguous(), self.signs, G)
            obs.observe(x, dt_raw, self.A_log, Bf, Cf, C)
        self.scales = {k: v.contiguous() for k, v in obs.scales().items()}
        self.B_inv = (1.0 / self.scales["B_scale"]).contiguous()
        self.C_inv = (1.0 / self.scales["C_scale"]).contiguous()
        return self


def m2_layer_forward(Lr, keyside=False, link=None):
    """The product path of one layer: prologue on xBC, then the combined SSD forward. Returns out [B,L,H,P] fp16.
    With `link` the layer is one rank's segment of the sequence and the state passing hands its carry to the next rank."""
    from linquant_b200.kernels.hadamard import kronecker_hadamard_fwd
    from linquant_b200.kernels.mamba2 import ssd_combined as sc
    from linquant_b200.kernels.mamba2.fused_split_rotate_xBC import fused_split_rotate_quant_xBC

    H, P, N, G, C = M2["H"], M2["P"], M2["N"], M2["G"], M2["C"]
    S = Lr.scales
    x, qB, qC = fused_split_rotate_quant_xBC(Lr.xBC, Lr.signs, H, G, N, P, Lr.B_inv, Lr.C_inv)
    b_fp = None
    if keyside:  # the key side quantises the gate-weighted, rotated B inside the chunk-state kernel
        Bl = Lr.xBC[..., H * P: H * P + G * N].unflatten(-1, (G, N))
        b_fp = kronecker_hadamard_fwd(Bl, Lr.signs, G)
    if link is not None:
        link.next_call()
    out, _ = sc._quant_mamba_chunk_scan_combined_fwd(
        x, Lr.dt_raw, 1.0, Lr.A_log, 1.0, qB, S["B_scale"], qC, S["C_scale"], C, Lr.D, 1.0, dt_softplus=True,
        static_state_scale=S["state_scale"], static_cb_scale=S["cb_scale"], alpha_hp=S["alpha_hp"], bscale_g=S["B_scale"],
        keyside=keyside, x_scale_hp=S["x_scale_hp"], b_fp=b_fp, b_gate_scale=S["b_gate_scale"], _link=link)
    return out


class StageTimer:
    """CUDA-event time of every sub-op of the combined forward, by wrapping the module attributes of `ssd_combined`
    (and the prologue) with event-recording shims on the launching stream."""

    NAMES = {"_quant_chunk_cumsum_fwd": "chunk_cumsum", "_quant_chunk_state_fwd_xfp_static_int8": "chunk_state",
             "_chunk_state_keyside_fwd": "chunk_state", "_fixedpoint_state_passing_fwd": "state_passing",
             "_quant_bmm_chunk_fwd": "bmm_chunk", "_chunk_scan_v2": "chunk_scan"}

    def __init__(self):
        self.pairs = []
        self.saved = {}

    def wrap(self, fn, name):
        def shim(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **kw)
            e1.record()
            self.pairs.append((name, e0, e1))
            return r
        return shim

    def __enter__(self):
        import linquant_b200.kernels.hadamard as hd
        import linquant_b200.kernels.mamba2.fused_split_rotate_xBC as fs
        from linquant_b200.kernels.mamba2 import ssd_combined as sc

        self.mods = [(sc, n, lab) for n, lab in self.NAMES.items()] + [(fs, "fused_split_rotate_quant_xBC", "prologue"),
                                                                        (hd, "kronecker_hadamard_fwd", "hadamard_B")]
        for mod, n, lab in self.mods:
            self.saved[(mod, n)] = getattr(mod, n)
            setattr(mod, n, self.wrap(getattr(mod, n), lab))
        return self

    def __exit__(self, *exc):
        for (mod, n), fn in self.saved.items():
            setattr(mod, n, fn)

    def totals_ms(self):
        torch.cuda.synchronize()
        out, cnt = {}, {}
        for name, e0, e1 in self.pairs:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
            cnt[name] = cnt.get(name, 0) + 1
        return out, cnt


def int8_tensor_peak(dev):
    """Dense INT8 tensor throughput of this GPU as cuBLAS delivers it: best of 10 torch._int_mm 8192^3 (TOP/s)."""
    try:
        a = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=dev)
        torch._int_mm(a, b)
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192**3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def dist_env():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


_ALL_CORES = None  # the affinity the process started with (the CPU baseline takes every core back)


def pin_host_threads(local, world):
    """Pins this rank's host threads to the CPU cores NVML reports as local to its GPU (its share of them when the ranks
    of the box report the same set), before any pinned host buffer is allocated. Returns a one-line record."""
    global _ALL_CORES
    try:
        import pynvml

        _ALL_CORES = os.sched_getaffinity(0)
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(local).uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cores = [64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1]
        allowed = sorted(set(cores) & os.sched_getaffinity(0))
        if not allowed:
            return "unchanged (NVML reports no usable local cores)"
        per = len(allowed) // world
        mine = allowed[local * per:(local + 1) * per] if per >= 2 else allowed
        os.sched_setaffinity(0, mine)
        torch.set_num_threads(max(1, min(len(mine), 8)))
        return f"cores {mine[0]}-{mine[-1]} ({len(mine)} of the {len(allowed)} NVML-local cores)"
    except Exception as e:  # no NVML, no permission: leave the affinity as it is
        return f"unchanged ({type(e).__name__})"


def run_ours(args):
    import torch.distributed as dist

    from linquant_b200 import _cabi, sharding
    from linquant_b200.host_pipeline import SsdStackHostPipeline

    world, rank, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    affinity = "unchanged (--no-pin)" if args.no_pin else pin_host_threads(local, world)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _cabi.lib()  # fail loudly when the CUDA library is missing

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    B, L, H = args.batch, M2["L"], M2["H"]
    n_layers = args.layers
    assert world <= B and B % world == 0, "the stack shards whole batch elements: --gpus must divide the batch"
    shard = sharding.plan(B, H, world, rank)
    bids = list(range(shard.b0, shard.b1))

    # distinct layer inputs resident in HBM: all of them when memory allows, else a ring (every layer is far larger than L2)
    per_layer = len(bids) * L * ((H * M2["P"] + 2 * M2["G"] * M2["N"]) * 2 + H * 4)
    free = torch.cuda.mem_get_info(dev)[0]
    distinct = max(1, min(n_layers, int((free - 24e9) // per_layer)))
    layers = [M2Layer(i, bids, dev).calibrate(dev) for i in range(distinct)]
    stack = [layers[i % distinct] for i in range(n_layers)]
    peak_i8 = int8_tensor_peak(dev) if rank == 0 else None

    def eager_step(keyside=False):
        for Lr in stack:
            m2_layer_forward(Lr, keyside)

    sampler = ClockSampler() if rank == 0 else None
    if sampler:
        sampler.start()
    eager_step()  # loads the kernels and sizes torch's pools before any capture
    torch.cuda.synchronize()
    _cabi.check_status(dev)
    graph, mode = None, "eager"
    if not args.eager:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                eager_step()
            mode = "cuda_graph"
        except Exception as e:  # the same kernels launched one by one from Python
            graph, mode = None, f"eager (graph capture failed: {type(e).__name__})"
            torch.cuda.synchronize()
    step = graph.replay if graph is not None else eager_step

    warm, t_w = 0, time.time()
    while warm < max(args.warmup, 3) or time.time() - t_w < 0.3:
        step()
        torch.cuda.synchronize()  # a graph replay returns at once: without this the loop would queue hundreds of steps
        warm += 1
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    _cabi.check_status(dev)

    # per-kernel durations of the same stack, CUDA events on the launching stream around every sub-op
    with StageTimer() as st:
        eager_step()
        stage_ms, stage_cnt = st.totals_ms()
    if args.kernels_only:
        if sampler:
            sampler.stop(world)
        if rank == 0:
            print(json.dumps({"kernels_only": True, "mode": mode, "ms_per_step": ms / args.steps,
                              "stage_us_per_layer": {k: round(1e3 * v / stage_cnt[k], 1) for k, v in stage_ms.items()}}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # end to end through the host-buffer call: per layer H2D of xBC and dt from pinned memory, the layer, D2H of out
    pipe = SsdStackHostPipeline(len(bids), L, M2, dev)
    e2e_steps = max(1, min(args.steps, 2))
    pipe.run(stack[: min(2, n_layers)])  # warm-up on two layers
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        pipe.run(stack)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    _cabi.check_status(dev)
    h2d, d2h = pipe.h2d_bytes_per_layer * n_layers, pipe.d2h_bytes_per_layer * n_layers
    del pipe
    clocks = sampler.stop(world) if sampler else None

    side = {}
    if not args.no_side:
        del stack, layers, graph
        torch.cuda.empty_cache()
        side = side_configs(dev, world, rank, barrier)

    tm = torch.tensor([ms, e2e_ms] + [stage_ms.get(k, 0.0) for k in sorted(stage_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    vals = tm.tolist()
    ms, e2e_ms = vals[0], vals[1]
    stage_ms = dict(zip(sorted(stage_ms), vals[2:]))
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    tokens = B * L
    ht_rank = len(bids) * L * H  # head-tokens one rank processes per layer
    peak, peak_kind = measured_peak()
    ab = m2_algorithmic_bytes()
    per_layer_us = {k: 1e3 * v / n_layers for k, v in stage_ms.items()}
    dom = max(per_layer_us, key=per_layer_us.get)
    achieved = ab[dom] * ht_rank / (per_layer_us[dom] * 1e-6) / 1e9
    path_gbs = ab["path"] * ht_rank * n_layers / (ms / args.steps * 1e-3) / 1e9
    traffic = NCU_DRAM_BYTES_PER_HEAD_TOKEN.get(dom)
    kernels = {}
    for k, us in per_layer_us.items():
        rec = {"us_per_layer": round(us, 1), "hbm_frac": round(ab[k] * ht_rank / (us * 1e-6) / 1e9 / peak, 3)}
        if peak_i8 and k in M2_INT8_OPS:
            rec["int8_tensor_frac"] = round(M2_INT8_OPS[k] * ht_rank / (us * 1e-6) / 1e12 / peak_i8, 4)
        kernels[k] = rec
    reduced = (n_layers, B, L) != (M2["layers"], M2["B"], 16384)
    line = {
        "metric": "INT8 chunk-prefill Mtokens/s", "value": tokens * args.steps / (ms * 1e-3) / 1e6, "unit": "Mtokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD if not reduced else f"REDUCED ({n_layers} layers, batch {B}, L {L}): not a bench value; " + WORKLOAD,
                   "sharding": f"batch x heads over {world} GPU(s): {len(bids)} batch element(s) per rank, no collective",
                   "launch": mode, "distinct_layer_inputs_in_hbm": distinct,
                   "l2": f"each layer reads {per_layer / 1e6:.0f} MB of fresh inputs per rank (L2 is 126 MB); no flush",
                   "calibration": "absmax observers on 4 further seeded batches per layer", "warmup_steps_run": warm},
        "e2e": {"value": tokens * e2e_steps / (e2e_ms * 1e-3) / 1e6, "unit": "Mtokens/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world, "steps": e2e_steps, "h2d_gbs_per_rank": h2d * e2e_steps / (e2e_ms * 1e-3) / 1e9,
                "host_buffers": "pinned ring of 2 layer inputs and 2 layer outputs per rank", "host_affinity_rank0": affinity},
        "gpu_launches": 7 * n_layers * args.steps,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": None if traffic is None else traffic * ht_rank,
                     "algorithmic_bytes": ab[dom] * ht_rank, "kernels": kernels,
                     "stage_sum_ms_per_step": round(sum(stage_ms.values()), 3),
                     "path_achieved": path_gbs, "path_frac": path_gbs / peak,
                     "int8_tensor_peak_tops": peak_i8, "int8_peak_how": "best of 10 torch._int_mm 8192^3, CUDA events"},
        "clocks": clocks,
        "per_config": side,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(reps=2)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------------------
# the other configurations, full size, as side records
ZOO = {
    # name: (synthetic config, delta, diagonal, stage entry points, path bytes per head-token)
    "simple_gla": ("simple_gla", False, False, ("lq_zoo_prologue_linear", "lq_zoo_state_linear", "lq_zoo_output_scalar"), 1028),
    "gated_deltanet": ("gated_deltanet", True, False, ("lq_zoo_prologue_delta", "lq_zoo_state_delta", "lq_zoo_output_scalar"), 1032),
    "kda": ("kda", True, True, ("lq_zoo_diag_rows", "lq_zoo_diag_amat", "lq_zoo_kda_wy", "lq_zoo_state_delta", "lq_zoo_output_scalar"), 1544),
}
ZOO_STAGE_BYTES = {  # per head-token, K = V = 128, chunk 64: own inputs once + own outputs once
    "lq_zoo_prologue_linear": 768 + 4 + 5 * 128 + 4,
    "lq_zoo_state_linear": 2 * 128 + 4.0 / 64 + 128 * 128 / 64,
    "lq_zoo_output_scalar": 3 * 128 + 128 * 128 / 64 + 4 + 256,
    "lq_zoo_prologue_delta": 768 + 8 + 3 * 128 + 256 + 8,
    "lq_zoo_state_delta": 128 + 256 + 128 + 256 + 128,
    "lq_zoo_diag_rows": 768 + 512 + 4 * 128 + 512 + 8,
    "lq_zoo_diag_amat": 2 * 128 + 512 + 128,
    "lq_zoo_kda_wy": 512 + 512 + 4 + 128 + 256 + 4,
}


def _gen_zoo(name, seed, B, T, dev):
    """The configuration's distribution drawn on the device (same recipe as linquant_b200.synthetic, one seed per batch
    element so that a shard of the batch is the same data on any number of GPUs)."""
    from linquant_b200.synthetic import CONFIGS

    c = CONFIGS[name]
    H, K, V = c["H"], c["K"], c["V"]
    F = torch.nn.functional
    out = {n: [] for n in ("q", "k", "v", "g", "beta")}
    for b in range(B[0], B[1]):
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + b)
        q = torch.randn(T, H, K, generator=g, device=dev)
        k = torch.randn(T, H, K, generator=g, device=dev)
        if c["op"] == "delta":
            q = F.normalize(q, dim=-1)
        if c.get("outliers"):
            go = torch.Generator(device=dev).manual_seed(seed)
            k[..., torch.randperm(K, generator=go, device=dev)[: max(1, round(c["outliers"] * K))]] *= 20.0
        k = F.normalize(k, dim=-1)
        out["q"].append(q.bfloat16())
        out["k"].append(k.bfloat16())
        out["v"].append(torch.randn(T, H, V, generator=g, device=dev).bfloat16())
        gs = (T, H, K) if c["op"] == "kda" else (T, H)
        out["g"].append(F.logsigmoid(torch.randn(*gs, generator=g, device=dev) + c["gmean"]))
        if c["op"] in ("delta", "kda"):
            out["beta"].append(torch.sigmoid(torch.randn(T, H, generator=g, device=dev)))
    return {n: (torch.stack(v) if v else None) for n, v in out.items()}


def _time_stages(fns, reps):
    for f in fns.values():
        f()
    torch.cuda.synchronize()
    ev = {n: [] for n in fns}
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        for n, f in fns.items():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            ev[n].append((e0, e1))
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps, {n: sum(x.elapsed_time(y) for x, y in p) / reps for n, p in ev.items()}


def zoo_config(name, dev, world, rank, reps=10, batch=None):
    from linquant_b200 import _cabi, sharding
    from linquant_b200 import invariances as inv
    from linquant_b200.kernels.zoo import _common
    from linquant_b200.synthetic import CONFIGS

    syn, delta, diag, stages, path_bytes = ZOO[name]
    c = CONFIGS[syn]
    B, T, H, K, V = batch or c["B"], c["T"], c["H"], c["K"], c["V"]
    sh = sharding.plan(B, H, world, rank)
    signs = inv.hadamard_signs(K, 0).to(dev)
    # scales (and D_QK) from four further seeded batches of one element, 1024 tokens each
    sc = inv.StaticScales(c["policy"], 8, 8)
    cal = [_gen_zoo(syn, 50 + i, (0, 1), 1024, dev) for i in range(4)]
    dqk = inv.dqk_from_stats(torch.cat([x["q"] for x in cal]), torch.cat([x["k"] for x in cal]), c["sqk"]).to(dev) if c.get("sqk") else None
    for x in cal:
        if diag:
            inv.calibrate_diagonal(sc, x["q"], x["k"], x["v"], x["g"], x["beta"], eta=c["eta"], sigma=c.get("sigma", 1.0),
                                   tau=c.get("tau", 1.0), chunk_size=64, rot_signs=signs)
        elif delta:
            inv.calibrate_delta(sc, x["q"], x["k"], x["v"], x["g"], x["beta"], eta=c["eta"], sigma=c["sigma"], tau=c["tau"],
                                chunk_size=64, rot_signs=signs, dqk=dqk)
        else:
            inv.calibrate_linear(sc, x["q"], x["k"], x["v"], x["g"], eta=c["eta"], chunk_size=64, rot_signs=signs)
    scales = sharding.take_scales(sh, sc.finalize().kernel_scales(H, K, V, dev))
    del cal
    x = _gen_zoo(syn, 7, (sh.b0, sh.b1), T, dev)
    q, k, v, g, beta = (None if x[n] is None else x[n][:, :, sh.h0:sh.h1].contiguous() for n in ("q", "k", "v", "g", "beta"))
    o, keep = torch.empty_like(v), []
    P = _common.make_problem(q, k, v, g, beta, scales, decay=2 if diag else 1, eta=c["eta"], sigma=c.get("sigma", 1.0), tau=c.get("tau", 1.0),
                             scale=K**-0.5, chunk_size=64, bits=8, out=o, final_state=None, rot_signs=signs,
                             dqk=None if dqk is None else dqk[sh.h0:sh.h1].contiguous(), keep=keep)
    ws = _cabi.Workspace(P, delta, dev)
    fns = {s: (lambda s=s: _common.run_stage(s, P, ws, q)) for s in stages}
    total_ms, st_ms = _time_stages(fns, reps)
    ws.check_status()
    return dict(total_ms=total_ms, stage_ms=st_ms, tokens=B * T, ht_rank=sh.units * T, path_bytes=path_bytes,
                stage_bytes={s: ZOO_STAGE_BYTES.get(s) for s in stages}, shape=f"B={B} H={H} K=V={K} L={T} chunk=64 bf16 {c['policy']}")


def m2_keyside_config(dev, world, rank, reps=3):
    from linquant_b200 import sharding

    sh = sharding.plan(M2["B"], M2["H"], world, rank)
    Lr = M2Layer(0, list(range(sh.b0, sh.b1)), dev).calibrate(dev)
    m2_layer_forward(Lr, True)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with StageTimer() as st:
        a.record()
        for _ in range(reps):
            m2_layer_forward(Lr, True)
        b.record()
        stage_ms, _ = st.totals_ms()
    ab = m2_algorithmic_bytes(True)
    return dict(total_ms=a.elapsed_time(b) / reps, stage_ms={k: v / reps for k, v in stage_ms.items()}, tokens=M2["B"] * M2["L"],
                ht_rank=sh.units * M2["L"], path_bytes=ab["path"], stage_bytes={k: ab.get(k) for k in stage_ms},
                shape="one layer of the stack, key-side absorption (INT8 x against gate-weighted B quantised in-kernel)")


def m2_seqpar_config(dev, world, rank, barrier, reps=3):
    """One layer of the stack with the SEQUENCE split over the ranks (every rank holds all 8 batch elements and 80 heads of
    its L / world tokens): cumsum, chunk state and C.B^T run at once on all ranks, the fixed-point state passing forms a
    chain in which each rank's kernel stores its INT32 carry straight into the next rank's memory over NVLink, the chunk
    scans run at once again."""
    from linquant_b200 import _cabi, seqpar

    Lr = M2Layer(0, list(range(M2["B"])), dev, segment=(rank, world)).calibrate(dev)
    link = seqpar.SsdLink(M2["B"], M2["H"], M2["P"] * M2["N"], dev, wait_ns=5_000_000_000)
    m2_layer_forward(Lr, link=link)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with StageTimer() as st:
        a.record()
        for _ in range(reps):
            m2_layer_forward(Lr, link=link)
        b.record()
        stage_ms, _ = st.totals_ms()
    _cabi.check_status(dev)
    barrier()
    link.close()
    ab = m2_algorithmic_bytes()
    return dict(total_ms=a.elapsed_time(b) / reps, stage_ms={k: v / reps for k, v in stage_ms.items()}, tokens=M2["B"] * M2["L"],
                ht_rank=M2["B"] * M2["H"] * M2["L"] // world, path_bytes=ab["path"], stage_bytes={k: ab.get(k) for k in stage_ms},
                shape=f"one layer of the stack, sequence split over {world} GPUs, INT32 carry stored into the next GPU's memory by the state-passing kernel")


def side_configs(dev, world, rank, barrier):
    import torch.distributed as dist

    peak, _ = measured_peak()
    out = {}
    names = list(ZOO) + ["mamba2_layer_keyside"] + (["mamba2_layer_seqpar"] if world > 1 and M2["L"] % (world * M2["C"]) == 0 else [])
    for name in names:
        try:
            if name == "mamba2_layer_seqpar":
                r = m2_seqpar_config(dev, world, rank, barrier)
            else:
                r = m2_keyside_config(dev, world, rank) if name == "mamba2_layer_keyside" else zoo_config(name, dev, world, rank)
            err = None
        except Exception as e:  # a side record must not take the headline down
            err = f"{type(e).__name__}: {e}"[:200]
        if world > 1:  # every rank learns whether any rank failed, so that all skip the reductions below together
            flag = torch.tensor([0 if err is None else 1], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            if int(flag.item()) and err is None:
                err = "another rank failed"
        if err is not None:
            out[name] = {"error": err}
            torch.cuda.empty_cache()
            continue
        keys = sorted(r["stage_ms"])
        tm = torch.tensor([r["total_ms"]] + [r["stage_ms"][k] for k in keys], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        vals = tm.tolist()
        rec = {"shape": r["shape"], "ms": round(vals[0], 4), "Mtokens_per_s": round(r["tokens"] / (vals[0] * 1e-3) / 1e6, 2),
               "path_frac": round(r["path_bytes"] * r["ht_rank"] / (vals[0] * 1e-3) / 1e9 / peak, 4), "stage_us": {}, "stage_hbm_frac": {}}
        for k, msv in zip(keys, vals[1:]):
            rec["stage_us"][k] = round(1e3 * msv, 1)
            if r["stage_bytes"].get(k):
                rec["stage_hbm_frac"][k] = round(r["stage_bytes"][k] * r["ht_rank"] / (msv * 1e-3) / 1e9 / peak, 3)
        out[name] = rec
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------------------------
# CPU arm: the reference recurrence on the host cores, bounded sample of the workload
def cpu_sample(threads, Ls=2048):
    """One layer x one batch element x the first Ls tokens of the stack, as the reference's float64 recurrence sees it:
    the linear / scalar-decay cell with q = C, k = B, v = x dt, g = dt A, scale 1 (the SSD's D x skip is a trivial
    epilogue and is left out), kernel_static, rotation on the state axis, INT8 state, chunk 256. Returns
    (callable, tokens, kind)."""
    from oracle import make_ref

    H, P, N, C = M2["H"], M2["P"], M2["N"], M2["C"]
    torch.set_num_threads(threads)

    def draw(seed, L):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(1, L, H, P, generator=g)
        Bm = torch.randn(1, L, 1, N, generator=g).expand(1, L, H, N)
        Cm = torch.randn(1, L, 1, N, generator=g).expand(1, L, H, N)
        dt = torch.nn.functional.softplus(torch.randn(1, L, H, generator=g) * 0.5 - 2.0)
        A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
        return Cm.contiguous(), Bm.contiguous(), x * dt.unsqueeze(-1), (dt * A).float()

    q, k, v, g = draw(1, Ls)
    ref = make_ref.load()
    if ref is not None:
        chunk_core, hadamard_rotation, FakeQuant, POLICIES = ref
        qz = FakeQuant("none", 8, ["ALL"], dict(POLICIES["kernel_static"]), state_bits=8, round_away=True)
        qz.tie_roles = qz.local_fp16 = qz.kernel_arith = True
        qz.layer = 0
        R = hadamard_rotation(N, 0)
        fn = lambda q, k, v, g: chunk_core(q, k, v, g, None, family="linear", decay="scalar", scale=1.0, qz=qz, rot_qk=R,  # noqa: E731
                                           eta=1.0, read_post=True, C=C, out_dtype=torch.float32)
        qz.calibrating = True
        for s in range(4):
            fn(*draw(10 + s, 512))
        qz.finalize()
        return (lambda: fn(q, k, v, g)), Ls, "reference"
    from oracle import zoo_oracle as zo

    R, _ = zo.signed_hadamard(N, 0)
    qz = zo.RoleQuantizer("kernel_static", 8, 8, True)
    fn = lambda q, k, v, g: zo.chunk_prefill(q, k, v, g, None, family="linear", decay="scalar", scale=1.0, qz=qz, rot_qk=R,  # noqa: E731
                                             eta=1.0, chunk=C, read_post=True)
    qz.start_calibration()
    for s in range(4):
        fn(*draw(10 + s, 512))
    qz.finish_calibration()
    return (lambda: fn(q, k, v, g)), Ls, "port"


CPU_SAMPLE = "1 of 64 layers x 1 of 8 batch elements x 2048 of 16384 tokens, all 80 heads; time scaled by 64 layers per token"


def cpu_baseline(reps):
    if _ALL_CORES:
        os.sched_setaffinity(0, _ALL_CORES)
    threads = os.cpu_count() or 1
    run, tokens, kind = cpu_sample(threads)
    run()
    t = time.perf_counter()
    for _ in range(reps):
        run()
    dt = (time.perf_counter() - t) / reps
    return {"value": tokens / (dt * M2["layers"]) / 1e6, "unit": "Mtokens/s", "cores": threads, "kind": kind, "sample": CPU_SAMPLE,
            "what": "the reference's float64 chunk_core on CPU torch" if kind == "reference" else "float64 torch port of chunk_core"}


def run_reference(args):
    world, rank, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    run, tokens, kind = cpu_sample(threads)
    warm = max(args.warmup, 3)  # the same count the measured arm reports
    for _ in range(warm):
        run()
    t = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t
    val = tokens * args.steps / (dt * M2["layers"]) / 1e6
    print(json.dumps({
        "impl": "reference", "metric": "INT8 chunk-prefill Mtokens/s", "value": val, "unit": "Mtokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": val, "unit": "Mtokens/s", "cores": threads, "kind": kind, "sample": CPU_SAMPLE + " (each step)"},
        "e2e": {"value": val, "unit": "Mtokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_stages(args):
    """`--stages NAME`: per-kernel CUDA-event times of one configuration at full size on one GPU (a development aid;
    the same records the bench line carries in `per_config`)."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if args.stages == "mamba2_layer":
        Lr = M2Layer(0, list(range(args.batch)), dev).calibrate(dev)
        m2_layer_forward(Lr)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with StageTimer() as st:
            a.record()
            for _ in range(args.steps):
                m2_layer_forward(Lr)
            b.record()
            stage_ms, _ = st.totals_ms()
        print(json.dumps({"stages": "mamba2_layer", "batch": args.batch, "layer_us": round(1e3 * a.elapsed_time(b) / args.steps, 1),
                          "stage_us": {k: round(1e3 * v / args.steps, 1) for k, v in stage_ms.items()}}), flush=True)
        return
    if args.stages == "mamba2_layer_keyside":
        r = m2_keyside_config(dev, 1, 0)
    elif args.stages in ZOO:
        r = zoo_config(args.stages, dev, 1, 0, reps=args.steps, batch=args.zoo_batch)
    else:
        raise SystemExit(f"--stages: one of {sorted(ZOO) + ['mamba2_layer', 'mamba2_layer_keyside']}")
    print(json.dumps({"stages": args.stages, "total_us": round(1e3 * r["total_ms"], 1),
                      "stage_us": {k: round(1e3 * v, 1) for k, v in r["stage_ms"].items()}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="skip the per_config side records")
    ap.add_argument("--no-pin", action="store_true", help="leave the host threads' CPU affinity as it is")
    ap.add_argument("--eager", action="store_true", help="launch the step kernel by kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--layers", type=int, default=M2["layers"], help="fewer layers: a reduced run for profiling, not a bench value")
    ap.add_argument("--batch", type=int, default=M2["B"], help="smaller batch: a reduced run for profiling, not a bench value")
    ap.add_argument("--seqlen", type=int, default=M2["L"], help="shorter sequences: a reduced run for profiling, not a bench value")
    ap.add_argument("--zoo-batch", type=int, default=None, help="with --stages: fewer batch elements of a zoo configuration (profiling)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="device-resident loop and per-kernel times only (no host-buffer leg, no side records, no CPU baseline)")
    ap.add_argument("--stages", default=None, metavar="CONFIG",
                    help="per-kernel times of one configuration (simple_gla, gated_deltanet, kda, mamba2_layer, mamba2_layer_keyside)")
    args = ap.parse_args()
    M2["L"] = args.seqlen
    if args.stages:
        return run_stages(args)
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:  # plain `python bench.py --gpus N`: become N ranks
        os.execv(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                                  "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__),
                                  *sys.argv[1:]])
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
