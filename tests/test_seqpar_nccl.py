"""Sequence-parallel prefill on two GPUs over NCCL (skipped with fewer than two devices)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from linquant_b200 import seqpar
    from linquant_b200.kernels.zoo.simple_gla import chunk_simple_gla_int8
    from tests.helpers import OracleRun, rel_l2, zoo_inputs

    q, k, v, g, _ = zoo_inputs(2, 512, 2, 128, 128, decay="scalar", dtype=torch.bfloat16, seed=9)
    orc = OracleRun(q, k, v, g, None, family="linear", decay="scalar", policy="kernel_pt")
    sc = orc.scales("cuda")
    L = 512 // world
    sl = slice(rank * L, (rank + 1) * L)
    out = seqpar.chunk_simple_gla_int8_seqpar(q[:, sl].cuda(), k[:, sl].cuda(), v[:, sl].cuda(), g[:, sl].cuda(), sc)
    whole, _ = chunk_simple_gla_int8(q.cuda(), k.cuda(), v.cuda(), g.cuda(), sc)
    torch.cuda.synchronize()
    ret[rank] = rel_l2(out, whole[:, sl])
    dist.barrier()
    dist.destroy_process_group()


def test_seqpar_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0] == 0.0 and ret[1] <= 1e-3, dict(ret)
