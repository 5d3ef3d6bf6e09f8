"""Sequence-parallel host logic on two CPU ranks over gloo: segment end carries and decays are all-gathered, every rank
forms its incoming carry by the exclusive scan, and the segment outputs (the CPU oracle stands in for the device work)
reproduce the unsplit run."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from linquant_b200 import seqpar


def test_exclusive_scan_of_carries():
    torch.manual_seed(0)
    W, B, H, K, V = 4, 2, 3, 4, 5
    S_end, gam = torch.randn(W, B, H, K, V), torch.rand(W, B, H)
    got = seqpar.incoming_carries(S_end, gam)
    run = torch.zeros(B, H, K, V)
    for r in range(W):
        assert torch.allclose(got[r], run)
        run = gam[r][..., None, None] * run + S_end[r]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import zoo_oracle as zo
    from tests.helpers import OracleRun, zoo_inputs

    q, k, v, g, _ = zoo_inputs(1, 256, 2, 64, 64, decay="scalar")
    full = OracleRun(q, k, v, g, None, family="linear", decay="scalar")
    want = full.run()
    L = 256 // world
    sl = slice(rank * L, (rank + 1) * L)
    kw = dict(full.kw)
    _, s_end = zo.chunk_prefill(q[:, sl], k[:, sl], v[:, sl], g[:, sl], None, **{**kw, "return_final_state": True})
    gamma = seqpar.segment_gamma(g[:, sl], 1, 2, "cpu")
    ends = [torch.empty_like(s_end) for _ in range(world)]
    gams = [torch.empty_like(gamma) for _ in range(world)]
    dist.all_gather(ends, s_end.contiguous())
    dist.all_gather(gams, gamma)
    s_in = seqpar.incoming_carries(torch.stack(ends).float(), torch.stack(gams))[rank]
    out = zo.chunk_prefill(q[:, sl], k[:, sl], v[:, sl], g[:, sl], None, **{**kw, "initial_state": s_in if rank else None})
    err = ((out - want[:, sl]).norm() / want[:, sl].norm()).item()
    ret[rank] = err
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsplit_output():
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0] < 1e-12 and ret[1] < 2e-3, dict(ret)
