"""Host-side logic of the multi-GPU layer on CPU ranks (gloo, world_size 2): the Ulysses exchange
and the head sharding must reproduce single-process attention exactly when the same attention
function is used on both sides (fp32 SDPA here, so no GPU is needed)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sage3
from sageattention_b200 import distributed as sd


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _sdpa_fn(q, k, v, tensor_layout="HND", is_causal=False, **kw):
    if tensor_layout == "NHD":
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
    o = sage3.sdpa_fp32(q, k, v, is_causal=is_causal)
    return o.transpose(1, 2).contiguous() if tensor_layout == "NHD" else o


def _worker(rank, world, port, chunks, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        B, N, H, D = 2, 64, 8, 16
        q, k, v = (torch.randn(B, N, H, D, generator=g) for _ in range(3))
        n = N // world
        sl = slice(rank * n, (rank + 1) * n)
        out = sd.ulysses_attention(q[:, sl], k[:, sl], v[:, sl], head_chunks=chunks, attn_fn=_sdpa_fn, is_causal=True)
        want = _sdpa_fn(q, k, v, tensor_layout="NHD", is_causal=True)[:, sl]
        ok1 = torch.allclose(out, want, atol=1e-6)
        qh, kh, vh = (t.transpose(1, 2).contiguous() for t in (q, k[:, :, :4], v[:, :, :4]))      # GQA 8 / 4
        out2 = sd.sageattn_head_parallel(qh, kh, vh, attn_fn=_sdpa_fn)
        ok2 = torch.allclose(out2, _sdpa_fn(qh, kh, vh), atol=1e-6)
        ret[rank] = (bool(ok1), bool(ok2))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 2])
def test_ulysses_and_head_sharding_match_single_process(chunks):
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, chunks, ret), nprocs=world, join=True)
        assert dict(ret) == {0: (True, True), 1: (True, True)}


def test_ulysses_rejects_indivisible_heads():
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        x = torch.randn(1, 8, 3, 16)
        with pytest.raises(ValueError):
            sd.ulysses_attention(x, x, x, head_chunks=2, attn_fn=_sdpa_fn)
    finally:
        dist.destroy_process_group()


def test_shard_units_cover_every_unit_once():
    for B, H, W in [(1, 40, 8), (4, 8, 8), (1, 40, 3), (2, 3, 4)]:
        parts = sd.shard_units(B, H, W)
        flat = [u for p in parts for u in p]
        assert sorted(flat) == [(b, h) for b in range(B) for h in range(H)]
        sizes = [len(p) for p in parts]
        assert max(sizes) - min(sizes) <= 1
