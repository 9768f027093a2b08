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


def _sdpa_lse_fn(q, k, v, tensor_layout="NHD", is_causal=False, return_lse=True, **kw):
    """fp32 attention with log-sum-exp, NHD, GQA, top-left = bottom-right causal (equal lengths)."""
    qh, kh, vh = (t.transpose(1, 2).float() for t in (q, k, v))
    g = qh.shape[1] // kh.shape[1]
    kh, vh = kh.repeat_interleave(g, dim=1), vh.repeat_interleave(g, dim=1)
    s = torch.matmul(qh, kh.transpose(-1, -2)) * qh.shape[-1] ** -0.5
    if is_causal:
        n = s.shape[-1]
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vh)
    return o.transpose(1, 2).contiguous(), lse


def _ring_worker(rank, world, port, causal, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        B, N, Hq, Hkv, D = 2, 96, 4, 2, 16
        q = torch.randn(B, N, Hq, D, generator=g)
        k, v = (torch.randn(B, N, Hkv, D, generator=g) for _ in range(2))
        n = N // world
        sl = slice(rank * n, (rank + 1) * n)
        out = sd.ring_attention(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(),
                                is_causal=causal, attn_fn=_sdpa_lse_fn)
        want, _ = _sdpa_lse_fn(q, k, v, is_causal=causal)
        ret[rank] = bool(torch.allclose(out, want[:, sl], atol=1e-5))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,causal", [(2, False), (2, True), (3, True)])
def test_ring_attention_matches_single_process(world, causal):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_ring_worker, args=(world, port, causal, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def test_merge_partial_ignores_rows_without_keys():
    o1, o2 = torch.randn(1, 4, 2, 8), torch.randn(1, 4, 2, 8)
    l1 = torch.randn(1, 2, 4)
    l2 = torch.full((1, 2, 4), float("inf"))                   # non-finite either way counts as "no key"
    out, lse = sd.merge_partial(o1, l1, o2, l2)
    assert torch.allclose(out, o1) and torch.allclose(lse, l1)
    out, lse = sd.merge_partial(o1, torch.full_like(l1, -float("inf")), o2, l2)
    assert torch.equal(out, torch.zeros_like(out))


@pytest.mark.parametrize("chunks", [1, 2, [1, 2, 1]])
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
