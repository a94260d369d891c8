"""Row-sharded forward on two GPUs against the single-GPU forward, with both transports: NCCL collectives between
the kernels, and the kernels storing to / loading from the peer GPU's memory. Skipped with fewer than two GPUs.

Child processes, one per GPU; NVLS is switched off for the library, the peer accesses are plain (non-multicast)
TMA stores and 16-byte loads, and no kernel waits on another GPU.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.helpers import rand_params

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, outgoing, incoming, transport, contraction, N, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import miniworld_b200 as mw
        from miniworld_b200 import sharded

        p = rand_params(61)
        g = torch.Generator().manual_seed(62)
        z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
        mask = torch.rand(1, N, generator=g) > 0.15
        begin, rows = sharded.row_range(N, world, rank)
        full = mw.TriangleMultiplication(128, outgoing=outgoing, check_status=True)
        full.load_state_dict(p)
        full = full.to(dev).to(torch.bfloat16).eval()
        shard = sharded.RowShardedTriangleMultiplication(128, outgoing=outgoing, incoming=incoming, transport=transport,
                                                         contraction=contraction, check_status=True)
        shard.load_state_dict(p)
        shard = shard.to(dev).to(torch.bfloat16).eval()
        with torch.no_grad():
            want = full(z.to(dev), mask.to(dev))[:, begin : begin + rows]
            for _ in range(3):  # later calls reuse the buffers (the p2p transport alternates between two)
                got = shard(z[:, begin : begin + rows].contiguous().to(dev), mask.to(dev))
        assert shard.transport == transport and shard.contraction == contraction
        torch.cuda.synchronize()
        ret[rank] = (bool(torch.equal(got, want)), float((got.float() - want.float()).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize(
    "outgoing,incoming,transport,contraction",
    [(True, "reduce", "nccl", "rows"), (False, "gather", "nccl", "rows"), (False, "reduce", "nccl", "rows"),
     (True, "reduce", "p2p", "rows"), (False, "reduce", "p2p", "rows"), (True, "reduce", "p2p", "channels"),
     (False, "reduce", "p2p", "channels")],
)
def test_row_sharded_equals_single_gpu(outgoing, incoming, transport, contraction):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, N = 2, 256
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, outgoing, incoming, transport, contraction, N, ret), nprocs=world, join=True)
        assert len(ret) == world
        for rank, (same, err) in ret.items():
            if outgoing or incoming == "gather" or contraction == "channels":
                # same kernels, same k order: the rows a rank computes are bit-identical to the unsharded forward
                assert same, (rank, err)
            else:
                # partial sums rounded to fp16 per rank: a few bf16 output roundings may differ
                assert err <= 0.0625, (rank, err)
