"""Batch x head sharding on two CPU ranks over gloo: each rank runs its shard of the recurrence (the CPU oracle stands
in for the device work), the gathered output must equal the unsharded run bit for bit."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from linquant_b200 import sharding


def test_plan_covers_every_unit_once():
    for B, H, world in ((4, 16, 1), (4, 16, 2), (4, 16, 4), (4, 16, 8), (8, 32, 8), (3, 5, 2), (1, 8, 8)):
        seen = torch.zeros(B, H, dtype=torch.int32)
        for r in range(world):
            s = sharding.plan(B, H, world, r)
            seen[s.b0:s.b1, s.h0:s.h1] += 1
        assert bool((seen == 1).all()), (B, H, world)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import zoo_oracle as zo
    from tests.helpers import OracleRun, zoo_inputs

    q, k, v, g, _ = zoo_inputs(B, 128, H, 64, 64, decay="scalar")
    full = OracleRun(q, k, v, g, None, family="linear", decay="scalar", policy="kernel_static")
    want = full.run().float()
    scales = full.qz.scales  # calibrated once on the whole batch, then sliced by head
    sh = sharding.plan(B, H, world, rank)
    ql, kl, vl, gl = sharding.take(sh, q, k, v, g)
    qz = zo.RoleQuantizer("kernel_static", 8, 8, True)
    qz.scales = {r: (s[sh.h0:sh.h1] if s.dim() > 0 else s) for r, s in scales.items()}
    local = zo.chunk_prefill(ql, kl, vl, gl, None, family="linear", decay="scalar", scale=64**-0.5, qz=qz, eta=1.0, chunk=64,
                             read_post=True, out_dtype=torch.float32)
    got = sharding.gather_output(local, sh, B, H)
    ks = sharding.take_scales(sh, full.scales("cpu"))
    assert ks["kw"].shape == (sh.h1 - sh.h0, 64) and ks["q"].shape == (sh.h1 - sh.h0,)
    ret[rank] = bool(torch.equal(got, want))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_output():
    for B, H in ((2, 4), (1, 4)):  # batch split, then head split
        port = _free_port()
        ret = mp.Manager().dict()
        mp.spawn(_worker, args=(2, port, B, H, ret), nprocs=2, join=True)
        assert ret[0] and ret[1], (B, H, dict(ret))
