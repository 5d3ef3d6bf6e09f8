#!/usr/bin/env python
"""INT8 chunk-prefill benchmark: Mtokens/s of the chunk_simple_gla_int8 path on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the hot path (fused rotate/quantise prologue -> INT8 state pass -> output kernel) over one
batch of the Simple-GLA configuration (B=4, H=16, d_k=d_v=128, L=4096, chunk 64, bf16, kernel_pt scales, fused
R_QK Hadamard rotation, INT8 state). Batch x head units are independent, so N ranks each run one such batch
(weak scaling, no data-path collective). Rank 0 prints one JSON line.

`--impl reference` times the CPU port of the reference recurrence (oracle/zoo_oracle.py, float64 torch on the
host cores) on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "simple_gla"
ALGO_BYTES_PER_HEAD_TOKEN = {
    # each input read once, each output written once (q,k,v bf16 + g fp32 in, o bf16 out)
    "path": 128 * 2 * 3 + 4 + 128 * 2,
    # per kernel: its own inputs once + its own outputs once
    "prologue": 128 * 2 * 3 + 4 + 5 * 128 + 4,
    "state": 2 * 128 + 4.0 / 64 + 128 * 128 / 64,
    "output": 3 * 128 + 128 * 128 / 64 + 4 + 128 * 2,
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel at this workload, from ncu captures of
# `python bench.py --kernels-only --steps 1 --warmup 3` (profiles/simple_gla_cfg1_tc_kernels.md). Outputs that are still in the
# 126 MB L2 when the kernel ends are not counted by those counters, which is why traffic can sit below the
# algorithmic bytes.
NCU_DRAM_BYTES_PER_LAUNCH = {"prologue": 326.1e6, "state": 97.1e6, "output": 210.8e6}


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


def build_workload(device, seed):
    from linquant_b200 import invariances as inv
    from linquant_b200.synthetic import CONFIGS, make_inputs

    cfg = CONFIGS[WORKLOAD]
    x = make_inputs(WORKLOAD, seed=seed)
    signs = inv.hadamard_signs(cfg["K"], 0)
    return cfg, x, signs


def calibrated_scales(cfg, x, signs, device):
    """kernel_pt static scales from an absmax pass over the batch itself (torch ops on the GPU)."""
    from linquant_b200 import invariances as inv

    sc = inv.StaticScales(cfg["policy"], 8, 8)
    inv.calibrate_linear(sc, x["q"].to(device), x["k"].to(device), x["v"].to(device), x["g"].to(device), eta=cfg["eta"],
                         chunk_size=cfg["chunk"], rot_signs=signs)
    sc.finalize()
    return sc.kernel_scales(cfg["H"], cfg["K"], cfg["V"], device)


def run_ours(args):
    import torch.distributed as dist

    from linquant_b200 import _cabi
    from linquant_b200.kernels.zoo import _common
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _cabi.lib()  # fail loudly when the CUDA library is missing

    cfg, x, signs = build_workload(dev, seed=1000 + rank)
    B, T, H, K, V = cfg["B"], cfg["T"], cfg["H"], cfg["K"], cfg["V"]
    scales = calibrated_scales(cfg, x, signs, dev)
    q, k, v, g = (x[n].to(dev) for n in ("q", "k", "v", "g"))
    signs_d = signs.to(dev)

    # stage-level launches (the same three kernels lq_simple_gla_fwd enqueues) so each can be timed by events
    o = torch.empty_like(v)
    keep = []
    P = _common.make_problem(q, k, v, g, None, scales, decay=_cabi.DECAY_SCALAR, eta=cfg["eta"], sigma=1.0, tau=1.0,
                             scale=K**-0.5, chunk_size=cfg["chunk"], bits=8, out=o, final_state=None, rot_signs=signs_d,
                             dqk=None, keep=keep)
    ws = _cabi.Workspace(P, False, dev)
    stages = ("lq_zoo_prologue_linear", "lq_zoo_state_linear", "lq_zoo_output_scalar")

    def step(events=None):
        for i, s in enumerate(stages):
            if events is not None:
                events[i].record()
            _common.run_stage(s, P, ws, q)
        if events is not None:
            events[3].record()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler needs ~0.1 s to come up: it is started first and the warm-up keeps the GPU under load for at
    # least 0.3 s, so that samples exist from before the timed region to its end
    sampler = ClockSampler() if rank == 0 else None
    if sampler:
        sampler.start()
    warm, t_w = 0, time.time()
    while warm < max(args.warmup, 3) or time.time() - t_w < 0.3:
        step()
        warm += 1
        if warm % 16 == 0:
            torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        step(evs[i])
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    stage_ms = [sum(e[i].elapsed_time(e[i + 1]) for e in evs) / args.steps for i in range(3)]

    if args.kernels_only:
        if sampler:
            sampler.stop(world)
        if rank == 0:
            print(json.dumps({"kernels_only": True, "ms_per_step": ms / args.steps,
                              "stage_us": [round(1e3 * t, 2) for t in stage_ms]}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # end to end through the public call with host buffers: H2D of q,k,v,g from pinned memory, the op, D2H of o
    hq, hk, hv, hg = (x[n].pin_memory() for n in ("q", "k", "v", "g"))
    ho = torch.empty(v.shape, dtype=v.dtype).pin_memory()
    dq, dk, dv, dg = (torch.empty_like(t, device=dev) for t in (hq, hk, hv, hg))

    from linquant_b200.host_pipeline import SimpleGlaHostPipeline

    pipe = SimpleGlaHostPipeline(B, T, H, K, V, q.dtype, dev)
    del dq, dk, dv, dg

    def e2e_step():
        # public host-buffer call: per batch element H2D -> prologue/state/output -> D2H, copies overlapped with kernels
        pipe(hq, hk, hv, hg, scales, ho, eta=cfg["eta"], chunk_size=cfg["chunk"], rot=signs_d)

    for _ in range(2):
        e2e_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop(world) if sampler else None

    tm = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    ms, e2e_ms = tm.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    tokens = B * T * world
    head_tokens = B * T * H
    peak, peak_kind = measured_peak()
    names = ("prologue", "state", "output")
    dom = max(range(3), key=lambda i: stage_ms[i])
    achieved = ALGO_BYTES_PER_HEAD_TOKEN[names[dom]] * head_tokens / (stage_ms[dom] * 1e-3) / 1e9
    path_gbs = ALGO_BYTES_PER_HEAD_TOKEN["path"] * head_tokens / (ms / args.steps * 1e-3) / 1e9
    line = {
        "metric": "INT8 chunk-prefill Mtokens/s", "value": tokens * args.steps / (ms * 1e-3) / 1e6, "unit": "Mtokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "simple_gla_int8 B=4 H=16 dk=dv=128 L=4096 chunk=64 bf16 kernel_pt R_QK int8-state",
                   "per_gpu_batch": B, "sharding": f"batchxhead x{world}", "l2": "inputs (201 MB) exceed L2; no flush",
                   "warmup_steps_run": warm},
        "e2e": {"value": tokens * args.steps / (e2e_ms * 1e-3) / 1e6, "unit": "Mtokens/s",
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg)),
                "d2h_bytes_per_step": ho.numel() * ho.element_size()},
        "gpu_launches": 3 * args.steps,
        "roofline": {"bound": "hbm", "kernel": names[dom], "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind, "traffic": NCU_DRAM_BYTES_PER_LAUNCH[names[dom]],
                     "algorithmic_bytes": ALGO_BYTES_PER_HEAD_TOKEN[names[dom]] * head_tokens,
                     "stage_us": {n: round(1e3 * t, 2) for n, t in zip(names, stage_ms)},
                     "path_achieved": path_gbs, "path_frac": path_gbs / peak},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(reps=3)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_sample(threads):
    """One batch element of the workload, calibrated oracle ready to run. Returns (callable, tokens)."""
    from linquant_b200.synthetic import CONFIGS, make_inputs
    from oracle import zoo_oracle as zo

    cfg = CONFIGS[WORKLOAD]
    torch.set_num_threads(threads)
    x = make_inputs(WORKLOAD, seed=1000, B=1)
    R, _ = zo.signed_hadamard(cfg["K"], 0)
    qz = zo.RoleQuantizer(cfg["policy"], 8, 8, True)
    run = lambda: zo.chunk_prefill(x["q"], x["k"], x["v"], x["g"], None, family="linear", decay="scalar",  # noqa: E731
                                   scale=cfg["K"] ** -0.5, qz=qz, rot_qk=R, eta=cfg["eta"], chunk=cfg["chunk"], read_post=True)
    zo.calibrate(qz, run)
    return run, cfg["T"]


def cpu_baseline(reps):
    threads = os.cpu_count() or 1
    run, tokens = cpu_sample(threads)
    run()
    t = time.perf_counter()
    for _ in range(reps):
        run()
    dt = (time.perf_counter() - t) / reps
    return {"value": tokens / dt / 1e6, "unit": "Mtokens/s", "cores": threads, "kind": "port",
            "sample": "1 of 4 batch elements (H=16, L=4096), float64 torch port of the reference recurrence"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    run, tokens = cpu_sample(threads)
    for _ in range(min(args.warmup, 3)):
        run()
    t = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t
    val = tokens * args.steps / dt / 1e6
    sample = "1 of 4 batch elements (H=16, L=4096) per step, float64 torch port of the reference recurrence"
    print(json.dumps({
        "impl": "reference", "metric": "INT8 chunk-prefill Mtokens/s", "value": val, "unit": "Mtokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": min(args.warmup, 3),
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic",
        "config": {"workload": "simple_gla_int8 B=4 H=16 dk=dv=128 L=4096 chunk=64 bf16 kernel_pt R_QK int8-state"},
        "cpu_baseline": {"value": val, "unit": "Mtokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "Mtokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


STAGE_WORKLOADS = {
    # name: (B, T, H, K, V, delta, diagonal, stage entry points); per-GPU slices of the benchmark configurations
    "simple_gla": (4, 4096, 16, 128, 128, False, False, ("lq_zoo_prologue_linear", "lq_zoo_state_linear", "lq_zoo_output_scalar")),
    "gated_deltanet": (4, 8192, 16, 128, 128, True, False, ("lq_zoo_prologue_delta", "lq_zoo_state_delta", "lq_zoo_output_scalar")),
    "kda_b2": (2, 8192, 32, 128, 128, True, True,
               ("lq_zoo_diag_rows", "lq_zoo_diag_amat", "lq_zoo_kda_wy", "lq_zoo_state_delta", "lq_zoo_output_scalar")),
    "gla_b2": (2, 8192, 32, 128, 128, False, True, ("lq_zoo_diag_rows", "lq_zoo_diag_amat", "lq_zoo_state_linear", "lq_zoo_output_scalar")),
}


def _time_us(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def run_stages(args):
    """Per-kernel CUDA-event times of one workload (`--stages NAME`), device-resident inputs, constant scales (timing
    does not depend on their values). `mamba2_b2` = one layer of the Mamba-2 2.7B-shaped SSD stack at B=2 of 8."""
    from linquant_b200 import _cabi
    from linquant_b200.kernels.zoo import _common

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    f = lambda *s, val=1.0: torch.full(s, val, device=dev)  # noqa: E731
    res = {}
    if args.stages in STAGE_WORKLOADS:
        B, T, H, K, V, delta, diag, stages = STAGE_WORKLOADS[args.stages]
        nrm = torch.nn.functional.normalize
        q = nrm(torch.randn(B, T, H, K, device=dev), dim=-1).bfloat16()
        k = nrm(torch.randn(B, T, H, K, device=dev), dim=-1).bfloat16()
        v = torch.randn(B, T, H, V, device=dev, dtype=torch.bfloat16)
        g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, *((K,) if diag else ()), device=dev) + 3)
        beta = torch.sigmoid(torch.randn(B, T, H, device=dev)) if delta else None
        sc = {"q": f(H, val=K**-0.5 / 127), "k": f(H, val=1 / 127), "kw": f(H, K, val=1 / 127), "vw": f(H, V, val=4 / 127),
              "vl": f(H, V, val=4 / 127), "state": f(H, V, val=2 / 127), "w": f(H, val=1 / 127), "el": f(H, V, val=4 / 127),
              "ew": f(H, V, val=4 / 127)}
        o, keep = torch.empty_like(v), []
        P = _common.make_problem(q, k, v, g, beta, sc, decay=2 if diag else 1, eta=0.0 if diag else 1.0, sigma=0.5 if delta else 1.0,
                                 tau=1.0, scale=K**-0.5, chunk_size=64, bits=8, out=o, final_state=None,
                                 rot_signs=torch.ones(K, device=dev), dqk=(f(H, K) if (delta and not diag) else None), keep=keep)
        ws = _cabi.Workspace(P, delta, dev)
        for st in stages:
            res[st] = _time_us(lambda: _common.run_stage(st, P, ws, q), args.steps)
        ws.check_status()
        tokens = B * T
    elif args.stages == "mamba2_b2":
        from linquant_b200.kernels.mamba2 import _ssd
        from linquant_b200.kernels.mamba2 import ssd_combined as sc2

        B, L, H, Pd, G, N, C = 2, 16384, 80, 64, 1, 128, 256
        x = torch.randn(B, L, H, Pd, device=dev).half()
        qB = torch.randint(-127, 128, (B, L, G, N), device=dev, dtype=torch.int8)
        qC = torch.randint(-127, 128, (B, L, G, N), device=dev, dtype=torch.int8)
        dtr, A_log = torch.randn(B, L, H, device=dev) * 0.5 - 2, torch.rand(H, device=dev) * 2.7
        a_hp, s_g, s_hp, cbs, Dv = f(H, Pd, val=0.01), f(G, val=0.03), f(H, Pd, val=0.5), f(G, val=0.3), f(H)
        dA, dt = sc2._quant_chunk_cumsum_fwd(dtr, 1.0, A_log, 1.0, C, None, True)
        st = sc2._quant_chunk_state_fwd_xfp_static_int8(x, qB, dt, dA, a_hp, s_g, s_hp)
        sp, _ = sc2._fixedpoint_state_passing_fwd(st.reshape(B, -1, H, Pd * N), dA[..., -1])
        cb = sc2._quant_bmm_chunk_fwd(qC, s_g, qB, s_g, C, cbs)
        spv = sp.reshape(B, -1, H, Pd, N)
        ops = {
            "chunk_cumsum": lambda: sc2._quant_chunk_cumsum_fwd(dtr, 1.0, A_log, 1.0, C, None, True),
            "chunk_state (transpose + tcgen05)": lambda: sc2._quant_chunk_state_fwd_xfp_static_int8(x, qB, dt, dA, a_hp, s_g, s_hp),
            "state_passing": lambda: sc2._fixedpoint_state_passing_fwd(st.reshape(B, -1, H, Pd * N), dA[..., -1]),
            "bmm_chunk": lambda: sc2._quant_bmm_chunk_fwd(qC, s_g, qB, s_g, C, cbs),
            "chunk_scan (warp_mma, default)": lambda: sc2._chunk_scan_v2(cb, x, dt, dA, qC, s_g, spv, Dv, 1.0, s_hp, cbs),
            "chunk_scan (tcgen05)": lambda: sc2._chunk_scan_v2(cb, x, dt, dA, qC, s_g, spv, Dv, 1.0, s_hp, cbs, kernel="tcgen05"),
        }
        for name, fn in ops.items():
            res[name] = _time_us(fn, args.steps)
        # the ops above are timed one at a time, so the short ones include the host's launch path; the whole forward,
        # queued back to back as a layer runs it, is the figure that counts
        layer = _time_us(lambda: sc2._quant_mamba_chunk_scan_combined_fwd(
            x, dtr, 1.0, A_log, 1.0, qB, s_g, qC, s_g, C, Dv, 1.0, dt_softplus=True, static_state_scale=s_hp,
            static_cb_scale=cbs, alpha_hp=a_hp, bscale_g=s_g), args.steps)
        _ssd.check_status(dev)
        tokens = B * L
    else:
        raise SystemExit(f"--stages: unknown workload {args.stages}; one of {sorted(STAGE_WORKLOADS) + ['mamba2_b2']}")
    total = sum(v for n, v in res.items() if "tcgen05)" not in n or "chunk_state" in n)
    line = {"stages": args.stages, "stage_us": {n: round(v, 1) for n, v in res.items()}, "default_path_us": round(total, 1),
            "Mtokens_per_s": round(tokens / total, 2)}
    if args.stages == "mamba2_b2":
        line["combined_forward_us"] = round(layer, 1)
        line["Mtokens_per_s"] = round(tokens / layer, 2)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernels-only", action="store_true",
                    help="device-resident stage loop only (no host-buffer leg, no CPU baseline): the command profiled by ncu")
    ap.add_argument("--stages", default=None, metavar="WORKLOAD",
                    help="per-kernel times of another workload (simple_gla, gated_deltanet, kda_b2, gla_b2, mamba2_b2) instead of the bench line")
    args = ap.parse_args()
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
