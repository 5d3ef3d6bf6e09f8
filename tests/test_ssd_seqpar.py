"""Sequence-parallel Mamba-2 SSD: the INT32 carry of the fixed-point state passing crosses the cut, so the segments
reproduce the one-call result bit for bit. One GPU runs all segments in turn (same kernels, same carry / flag traffic,
local buffers); two GPUs run one segment each, rank 0's kernel storing its carry into rank 1's memory over NVLink."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B=2, L=2048, H=8, seed=2):
    from tests.test_ssd_ops import make_case

    return make_case(B=B, L=L, H=H, chunk=256, seed=seed)


def _kw(k, keyside, dev):
    kw = dict(dt_softplus=True, static_state_scale=k["state_scale"], static_cb_scale=k["cb_scale"], alpha_hp=k["alpha"],
              bscale_g=k["sB"], keyside=keyside, x_scale_hp=k["x_scale"], b_fp=k["Bm"], b_gate_scale=k["b_gate"])
    return {n: (v.to(dev) if torch.is_tensor(v) else v) for n, v in kw.items()}


def test_state_passing_carry_chains_calls_bit_for_bit():
    from linquant_b200.kernels.mamba2.state_passing import _fixedpoint_state_passing_fwd as sp

    g = torch.Generator().manual_seed(4)
    B, NC, H, D = 2, 12, 3, 8192
    states = torch.randint(-127, 128, (B, NC, H, D), generator=g, dtype=torch.int8).cuda()
    dA = (-torch.rand(B, H, NC, generator=g) * 2).cuda()
    whole, fin, carry = sp(states, dA, return_carry=True)
    a, _, ca = sp(states[:, :5], dA[..., :5].contiguous(), return_carry=True)
    b, finb, cb = sp(states[:, 5:], dA[..., 5:].contiguous(), initial_carry=ca, return_carry=True)
    torch.cuda.synchronize()
    assert torch.equal(torch.cat([a, b], 1), whole) and torch.equal(finb, fin) and torch.equal(cb, carry)
    assert int(carry.abs().max()) > 127  # the carry is the unclamped INT32 state, not its INT8 copy


@pytest.mark.parametrize("keyside", [False, True])
@pytest.mark.parametrize("nseg", [2, 4])
def test_segments_on_one_device_equal_the_single_call(nseg, keyside):
    import linquant_b200
    from linquant_b200 import seqpar
    from linquant_b200.kernels.mamba2.ssd_combined import _quant_mamba_chunk_scan_combined_fwd as fwd

    k = _case()
    d = "cuda"
    args = (k["x"].to(d), k["dt_raw"].to(d), 1.0, k["A_log"].to(d), 1.0, k["qB"].to(d), k["sB"].to(d), k["qC"].to(d), k["sC"].to(d),
            256, k["D"].to(d), 1.0)
    whole, _ = fwd(*args, **_kw(k, keyside, d))
    seg = seqpar.ssd_segmented_on_one_device(nseg, *args, **_kw(k, keyside, d))
    torch.cuda.synchronize()
    linquant_b200.check_status(d)
    assert torch.equal(seg, whole), f"{(seg != whole).sum().item()} outputs differ"


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import linquant_b200
    from linquant_b200 import seqpar
    from linquant_b200.kernels.mamba2.ssd_combined import _quant_mamba_chunk_scan_combined_fwd as fwd

    k = _case()
    B, L, H, P = k["x"].shape
    N = k["qB"].shape[-1]
    S = L // world
    sl = slice(rank * S, (rank + 1) * S)
    link = seqpar.SsdLink(B, H, P * N, dev, wait_ns=5_000_000_000)
    kw = _kw(k, False, dev)
    kw["b_fp"] = kw["b_fp"][:, sl]
    worst = 0
    for it in range(3):  # several forward passes through the same link: the epoch advances, flags are never reset
        out, _ = seqpar.ssd_combined_seqpar(link, k["x"][:, sl].to(dev), k["dt_raw"][:, sl].to(dev), 1.0, k["A_log"].to(dev), 1.0,
                                            k["qB"][:, sl].to(dev), k["sB"].to(dev), k["qC"][:, sl].to(dev), k["sC"].to(dev), 256,
                                            k["D"].to(dev), 1.0, **kw)
        torch.cuda.synchronize()
        linquant_b200.check_status(dev)
        whole, _ = fwd(k["x"].to(dev), k["dt_raw"].to(dev), 1.0, k["A_log"].to(dev), 1.0, k["qB"].to(dev), k["sB"].to(dev),
                       k["qC"].to(dev), k["sC"].to(dev), 256, k["D"].to(dev), 1.0, **_kw(k, False, dev))
        torch.cuda.synchronize()
        worst = max(worst, int((out != whole[:, sl]).sum().item()))
        dist.barrier()
    ret[rank] = worst
    dist.barrier()
    link.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_segments_on_several_gpus_equal_the_single_gpu_result(world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret[r] == 0 for r in range(world)), dict(ret)
