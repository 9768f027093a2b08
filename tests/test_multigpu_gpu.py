"""Multi-GPU parity on real GPUs (needs at least two; skipped otherwise): one process per GPU over NCCL.

* Ulysses: the output shard is BITWISE the single-GPU operator's output for the same tokens, when that operator is
  given the gathered full sequence of exactly the heads each Ulysses call attends.
* Ring: within the operator's own accuracy against fp32 SDPA (every shard is smoothed and quantised on its own).
* Head sharding: bitwise equal to the single-GPU operator (nothing is exchanged but the outputs).
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    import sageattention_b200 as sa
    from sageattention_b200 import distributed as sd
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        res = bench._ulysses_parity(sa, sd, dist, dev, world, rank)
        # head sharding: every rank holds the full tensors, attends its heads, gathers
        g = torch.Generator(device=dev).manual_seed(5)
        q = torch.randn((1, 4 * world, 300, 128), generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn((1, 2 * world, 300, 128), generator=g, device=dev).to(torch.bfloat16)
        v = torch.randn((1, 2 * world, 300, 128), generator=g, device=dev).to(torch.bfloat16)
        hk = 2
        want = torch.cat([sa.sageattn(q[:, r * hk * 2:(r + 1) * hk * 2].contiguous(), k[:, r * hk:(r + 1) * hk].contiguous(),
                                      v[:, r * hk:(r + 1) * hk].contiguous(), is_causal=True) for r in range(world)], dim=1)
        got = sd.sageattn_head_parallel(q, k, v, is_causal=True)
        res["head_parallel_bitwise"] = bool(torch.equal(got, want))
        ret[rank] = res
    finally:
        dist.destroy_process_group()


def test_ulysses_ring_and_head_sharding_on_gpus():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        for r in range(world):
            assert ret[r]["ulysses_parity"] == "bitwise", ret[r]
            assert ret[r]["ring_parity"]["ok"], ret[r]
            assert ret[r]["head_parallel_bitwise"], ret[r]
