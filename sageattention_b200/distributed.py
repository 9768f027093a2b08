"""Multi-GPU layer of the FP4 attention path: one process per GPU, ``torch.distributed`` (NCCL over
NVLink / NVSwitch on the GPUs, gloo in the CPU tests).

The reference has no communication code (its one multi-GPU example delegates to the external xDiT
package, ``example/parallel_sageattn_cogvideo.py:8-14,89-95``, whose Ulysses degree must divide the
head count, ``:31-36``).  Two schemes are provided:

* **head sharding** - smoothing, quantisation and attention are independent per (batch, kv head), so
  ranks take disjoint sets of (batch, kv-head group) units and nothing is exchanged on the data path
  (:func:`shard_units`, :func:`sageattn_head_parallel`).
* **Ulysses sequence parallelism** for sequences held sequence-sharded ``[B, N/P, H, D]``: one
  all-to-all turns the sequence shards of all heads into all tokens of ``H/P`` heads, the single-GPU
  operator runs unchanged (K means and Q block means see the whole sequence, so no further
  collective is needed), and one all-to-all brings the output back (:func:`ulysses_attention`).
  Heads are processed in chunks so that the exchange of chunk ``i+1`` overlaps the attention of
  chunk ``i``.  Every exchanged tile lands in local HBM first; the kernels only ever read local
  memory.
* **ring (context-parallel) attention** for sequences too long for the all-to-all scheme (or head
  counts that the world size does not divide): K/V shards travel round a ring of point-to-point
  copies while every rank attends its own queries to the shard it currently holds; the partial
  outputs are merged with their log-sum-exp (:func:`ring_attention`, :func:`merge_partial`).  Each
  step quantises and smooths its K shard on its own, which is exact for the merge because the
  operator's LSE output already carries the K-mean correction.
"""
from __future__ import annotations

import os
import time
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_units(batch: int, kv_heads: int, world_size: int) -> List[List[Tuple[int, int]]]:
    """Split the ``batch x kv_heads`` independent units over ranks as evenly as possible, keeping
    each rank's units contiguous (query heads follow their kv head, so GQA groups are never split)."""
    units = [(b, h) for b in range(batch) for h in range(kv_heads)]
    base, extra = divmod(len(units), world_size)
    out, pos = [], 0
    for r in range(world_size):
        n = base + (1 if r < extra else 0)
        out.append(units[pos:pos + n])
        pos += n
    return out


def sageattn_head_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, gather: bool = True,
                           attn_fn: Optional[Callable] = None, **kwargs) -> torch.Tensor:
    """Every rank holds the full HND tensors, computes the heads of its share of kv heads and
    (optionally) all-gathers the outputs.  Requires ``Hkv % world_size == 0``."""
    if attn_fn is None:
        from .api import sageattn as attn_fn
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    if Hkv % world != 0:
        raise ValueError("head sharding needs the number of kv heads to be a multiple of the world size")
    hk = Hkv // world
    g = Hq // Hkv
    qs = q[:, rank * hk * g:(rank + 1) * hk * g]
    ks, vs = k[:, rank * hk:(rank + 1) * hk], v[:, rank * hk:(rank + 1) * hk]
    out = attn_fn(qs.contiguous(), ks.contiguous(), vs.contiguous(), tensor_layout="HND", **kwargs)
    if not gather:
        return out
    parts = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(parts, out.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def _seq_to_head(x: torch.Tensor, world: int, group, async_op: bool = False):
    """[B, n, H, D] sequence shard -> [B, world*n, H/world, D] (all tokens, this rank's heads)."""
    B, n, H, D = x.shape
    send = x.reshape(B, n, world, H // world, D).permute(2, 0, 1, 3, 4).contiguous()   # [P, B, n, h, D]
    recv = torch.empty_like(send)
    work = dist.all_to_all_single(recv, send, group=group, async_op=async_op)

    def finish():
        # recv[p] = tokens of rank p's sequence shard for my heads
        return recv.permute(1, 0, 2, 3, 4).reshape(B, world * n, H // world, D)
    return work, finish


def _head_to_seq(x: torch.Tensor, world: int, group, async_op: bool = False):
    """[B, world*n, h, D] (all tokens, my heads) -> [B, n, world*h, D] (my tokens, all heads)."""
    B, N, h, D = x.shape
    n = N // world
    send = x.reshape(B, world, n, h, D).permute(1, 0, 2, 3, 4).contiguous()            # [P, B, n, h, D]
    recv = torch.empty_like(send)
    work = dist.all_to_all_single(recv, send, group=group, async_op=async_op)

    def finish(out: Optional[torch.Tensor] = None):
        # recv[p] = my tokens for rank p's heads; written straight into `out` [B, n, world*h, D] (a view into the
        # caller's result is fine) when given, so that the chunks need no concatenation afterwards
        src = recv.permute(1, 2, 0, 3, 4)                                              # [B, n, P, h, D]
        if out is None:
            return src.reshape(B, n, world * h, D)
        out.unflatten(2, (world, h)).copy_(src)
        return out
    return work, finish


def _chunk_sizes(heads_per_rank: int, head_chunks) -> List[int]:
    """Heads per rank of every chunk: an int splits evenly, a sequence is taken as it is."""
    if isinstance(head_chunks, int):
        if head_chunks < 1 or heads_per_rank % head_chunks != 0:
            raise ValueError(f"heads per rank ({heads_per_rank}) must be a multiple of head_chunks ({head_chunks})")
        return [heads_per_rank // head_chunks] * head_chunks
    sizes = [int(n) for n in head_chunks]
    if any(n < 1 for n in sizes) or sum(sizes) != heads_per_rank:
        raise ValueError(f"head chunk sizes {sizes} must be positive and add up to the heads per rank ({heads_per_rank})")
    return sizes


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, head_chunks=1,
                      attn_fn: Optional[Callable] = None, exposed: Optional[list] = None, **kwargs) -> torch.Tensor:
    """Sequence-parallel attention.  q, k, v: this rank's sequence shard ``[B, N/P, H, D]`` ("NHD";
    shard r holds tokens ``r*N/P ... (r+1)*N/P - 1``).  Returns the output shard ``[B, N/P, H, D]``.

    Requires ``H % P == 0`` and the same head count for q, k, v (expand GQA first).  ``head_chunks``: the
    heads are exchanged and attended in chunks - an int for equal chunks, or a sequence of heads per rank
    per chunk, e.g. ``[1, 2, 2]`` for 5 heads per rank - so that the all-to-all of the next chunk and the
    return all-to-all of the previous one are in flight while the current chunk is attended; only the
    first exchange and the last return are exposed, so small first and last chunks expose the least.
    Chunk ``c`` with ``n_c`` heads per rank carries the global heads ``[P*o_c, P*(o_c + n_c))`` (``o_c`` = heads
    per rank of the chunks before it), rank ``p`` attending ``[P*o_c + p*n_c, P*o_c + (p+1)*n_c)``.
    ``exposed``: a list that receives ``(start, end)`` CUDA event pairs around every point where the compute
    stream waits for a collective (their elapsed times add up to the exposed communication time).
    """
    if attn_fn is None:
        from .api import sageattn as attn_fn
    world = dist.get_world_size(group)
    B, n, H, D = q.shape
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError("ulysses_attention expects q, k, v of identical shape [B, N/P, H, D]")
    if H % world != 0:
        raise ValueError(f"the head count {H} must be a multiple of the world size {world}")
    sizes = _chunk_sizes(H // world, head_chunks)
    starts = [world * sum(sizes[:c]) for c in range(len(sizes))]

    def waited(work):
        if exposed is not None and q.is_cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            work.wait()
            e1.record()
            exposed.append((e0, e1))
        else:
            work.wait()

    def launch(c):
        sl = slice(starts[c], starts[c] + world * sizes[c])
        return [_seq_to_head(t[:, :, sl], world, group, async_op=True) for t in (q, k, v)]

    pending = launch(0)
    back = []
    for c in range(len(sizes)):
        cur = pending
        if c + 1 < len(sizes):
            pending = launch(c + 1)
        full = []
        for work, finish in cur:
            waited(work)
            full.append(finish())
        o = attn_fn(full[0], full[1], full[2], tensor_layout="NHD", **kwargs)          # [B, N, n_c, D]
        back.append(_head_to_seq(o, world, group, async_op=True))
    out = torch.empty_like(q)
    for c, (work, finish) in enumerate(back):
        waited(work)
        finish(out[:, :, starts[c]:starts[c] + world * sizes[c]])                      # heads in rank order = global order
    return out


def merge_partial(out_a: torch.Tensor, lse_a: torch.Tensor, out_b: torch.Tensor, lse_b: torch.Tensor):
    """Merge two attention results over disjoint key sets.  ``out`` [B,N,H,D] (NHD), ``lse`` [B,H,N]
    natural-log sum of exp(scores); rows that saw no key carry ``lse = -inf`` (or ``+inf``, which the
    kernel writes for tiles without keys) and weight 0."""
    la = torch.where(torch.isfinite(lse_a), lse_a, torch.full_like(lse_a, -float("inf")))
    lb = torch.where(torch.isfinite(lse_b), lse_b, torch.full_like(lse_b, -float("inf")))
    lse = torch.logaddexp(la, lb)
    safe = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    wa = torch.exp(la - safe).transpose(1, 2).unsqueeze(-1)                 # [B,N,H,1]
    wb = torch.exp(lb - safe).transpose(1, 2).unsqueeze(-1)
    out = out_a.float() * wa + out_b.float() * wb
    return out, lse


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, is_causal: bool = False,
                   attn_fn: Optional[Callable] = None, **kwargs) -> torch.Tensor:
    """Context-parallel attention.  q, k, v: this rank's sequence shard ``[B, N/P, H(kv), D]`` ("NHD";
    shard r holds tokens ``r*N/P ... (r+1)*N/P - 1``; GQA allowed).  Returns the output shard.

    ``attn_fn(q, k, v, tensor_layout="NHD", is_causal=..., return_lse=True)`` must return
    ``(out, lse)`` like :func:`sageattention_b200.sageattn`.  Step ``s`` attends to the shard of rank
    ``r - s``; the shard for step ``s + 1`` is in flight (one send, one receive per rank over
    NVLink / NVSwitch, into local HBM) while step ``s`` computes.  Causal: the own shard is attended
    with the causal mask, shards of lower ranks in full, shards of higher ranks are skipped (they are
    still forwarded)."""
    if attn_fn is None:
        from .api import sageattn as attn_fn
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    send_to = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    recv_from = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    kv = torch.stack([k, v]).contiguous()                       # one message per step
    out, lse = None, None
    for s in range(world):
        nxt, reqs = None, []
        if s + 1 < world:
            nxt = torch.empty_like(kv)
            ops = [dist.P2POp(dist.isend, kv, send_to, group), dist.P2POp(dist.irecv, nxt, recv_from, group)]
            reqs = dist.batch_isend_irecv(ops)
        src = (rank - s) % world                                 # whose shard kv holds now
        if not (is_causal and src > rank):
            o, l = attn_fn(q, kv[0], kv[1], tensor_layout="NHD", is_causal=bool(is_causal and src == rank),
                           return_lse=True, **kwargs)
            if out is None:
                out, lse = o.float(), l
            else:
                out, lse = merge_partial(out, lse, o, l)
        for r in reqs:
            r.wait()
        if nxt is not None:
            kv = nxt
    return out.to(q.dtype)


# ----------------------------------------------------------------------------------------------------
# benchmark leg used by bench.py --workload ulysses / ring
# ----------------------------------------------------------------------------------------------------

def bench_ulysses(args, w, dist_mod, dev, ring: bool = False):
    import json
    import sageattention_b200 as sa
    rank, world = dist_mod.get_rank(), dist_mod.get_world_size()
    B, H, N, D = w["B"], w["Hq"], w["N"], w["D"]
    if N % world or (H % world and not ring):
        raise SystemExit("ulysses workload: heads and tokens must be multiples of the number of GPUs")
    n = N // world
    g = torch.Generator(device=dev).manual_seed(4321 + rank)
    q = torch.randn((B, n, H, D), generator=g, device=dev).to(torch.bfloat16)
    koff = torch.randn((B, 1, H, D), generator=torch.Generator(device=dev).manual_seed(99), device=dev) * w["k_off"]
    k = (torch.randn((B, n, H, D), generator=g, device=dev) + koff).to(torch.bfloat16)
    v = torch.randn((B, n, H, D), generator=g, device=dev).to(torch.bfloat16)
    chunks = 2 if (H // world) % 2 == 0 else 1

    def step():
        if ring:
            return ring_attention(q, k, v, is_causal=w["causal"])
        return ulysses_attention(q, k, v, head_chunks=chunks, is_causal=w["causal"])

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist_mod.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist_mod.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    dist_mod.all_reduce(t, op=dist_mod.ReduceOp.MAX)
    ms = t.item()
    flops = 4.0 * B * H * N * N * D / (2 if w["causal"] else 1)
    if rank == 0:
        print(json.dumps({
            "metric": "attention_tops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp4 (e2m1 x ue4m3 block-scaled, fp32 accumulate)",
            "data": "synthetic",
            "config": ({"workload": "ring", "B": B, "H": H, "N": N, "D": D, "causal": w["causal"],
                        "sharding": f"sequence-sharded input, {world} ring steps of {n} keys, K/V shards by point-to-point copies",
                        "step": f"{world} x (K mean + fused quant + delta_s + attention) + {world - 1} K/V exchanges + LSE merges"}
                       if ring else
                       {"workload": "ulysses", "B": B, "H": H, "N": N, "D": D, "causal": w["causal"],
                        "sharding": f"sequence-sharded input, all-to-all to {H // world} heads per GPU, {chunks} head chunk(s)",
                        "step": "3 all-to-all + K mean + fused quant + delta_s + attention + 1 all-to-all"}),
            "gpu_launches": 4 * (world if ring else chunks) * args.steps}), flush=True)
    dist_mod.destroy_process_group()
