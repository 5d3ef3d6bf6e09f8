"""Sequence-parallel Mamba-2 SSD, host logic on two CPU ranks over gloo: each rank evaluates its segment with the CPU
restatement of the ops, rank 0 sends the unclamped INT32 carry of its state passing to rank 1 (the message the GPU
kernels store into the next GPU's memory), and the two segments reproduce the unsplit output bit for bit."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import ssd_oracle as so
    from tests.test_ssd_ops import make_case

    k = make_case(B=1, L=512, H=2, N=64, chunk=64, seed=6)
    kw = dict(dt_softplus=True, static_state_scale=k["state_scale"], static_cb_scale=k["cb_scale"], alpha_hp=k["alpha"], bscale_g=k["sB"])
    args = lambda sl: (k["x"][:, sl], k["dt_raw"][:, sl], 1.0, k["A_log"], 1.0, k["qB"][:, sl], k["sB"], k["qC"][:, sl], k["sC"], 64,  # noqa: E731
                       k["D"], 1.0)
    want, _ = so.ssd_combined(*args(slice(None)), **kw)
    S = 512 // world
    sl = slice(rank * S, (rank + 1) * S)
    carry_in = None
    if rank > 0:
        carry_in = torch.empty(1, 2, 64 * 64, dtype=torch.int32)
        dist.recv(carry_in, src=rank - 1)
    out, aux = so.ssd_combined(*args(sl), **kw, initial_carry=carry_in)
    if rank < world - 1:
        dist.send(aux["carry"].contiguous(), dst=rank + 1)
    ret[rank] = bool(torch.equal(out, want[:, sl]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsplit_output_bit_for_bit():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0] and ret[1], dict(ret)
