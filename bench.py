#!/usr/bin/env python
"""Benchmark of the FP4 attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" = one pass of the whole operator (K channel means, fused smoothing + NVFP4 quantisation,
delta_s, FP4 attention) over one batch of seeded synthetic input.  The metric is the reference's
attention throughput ``4*B*Hq*Nq*Nk*D / t`` (halved for causal), sageattention3_blackwell/scripts/
bench.py:151-153.  Prints ONE JSON line (rank 0).

Workloads (value distributions of the benchmark configurations; synthetic stand-ins for the
reference's video-model activations):
  dit      B=1 H=40 N=32760 D=128 non-causal, K channel offsets ~N(0,4), 5% of V channels x8  (default)
  prefill  B=4 Hq=32 Hkv=8 N=8192 D=128 causal, K channel offsets ~N(0,2)
  ulysses  B=1 H=40 N=75600 D=128 non-causal, sequence-sharded input, all-to-all over NCCL (needs N>1)
  ring     the same problem, K/V shards passed round a ring of point-to-point copies, partial outputs merged
           by their log-sum-exp (needs N>1)
With N GPUs the `dit` / `prefill` workloads are sharded over batch x heads with no collective: every
rank processes the same per-GPU workload (weak scaling) and the value is the sum over ranks.

Every default run also carries a `"ulysses"` object: the long-sequence configuration (B=1 H=40 N=75600 D=128,
the one multi-GPU path that communicates) in strong scaling - at N=1 the plain operator on the whole problem, at
N>1 `ulysses_attention` on sequence-sharded inputs (all-to-all over NCCL), after a parity check on a reduced
shape against the single-GPU operator; rank 0 also times the whole problem on its own GPU so that the line
carries `efficiency = t_1 / (N * t_N)` measured in the same run.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    "dit": dict(B=1, Hq=40, Hkv=40, N=32760, D=128, causal=False, k_off=2.0, v_out=0.05),
    "prefill": dict(B=4, Hq=32, Hkv=8, N=8192, D=128, causal=True, k_off=math.sqrt(2.0), v_out=0.0),
    "ulysses": dict(B=1, Hq=40, Hkv=40, N=75600, D=128, causal=False, k_off=2.0, v_out=0.0),
    "ring": dict(B=1, Hq=40, Hkv=40, N=75600, D=128, causal=False, k_off=2.0, v_out=0.0),
    "profile": dict(B=1, Hq=10, Hkv=10, N=32760, D=128, causal=False, k_off=2.0, v_out=0.05),   # a quarter of dit
    "small": dict(B=1, Hq=8, Hkv=8, N=1024, D=128, causal=False, k_off=2.0, v_out=0.0),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch, per head, at N = 32760, D = 128 (ncu)
TRAFFIC_PER_HEAD_DIT = 30.05e6


def attn_flops(B, Hq, Nq, Nk, D, causal):
    f = 4.0 * B * Hq * Nq * Nk * D
    return f / 2 if causal else f


def gen_inputs(w, seed, device, pin=False):
    """Seeded N(0,1) bf16 Q, K, V with the configuration's outliers, generated on the device to keep
    start-up short (the parity tests use CPU-generated inputs)."""
    g = torch.Generator(device=device).manual_seed(seed)
    shp_q = (w["B"], w["Hq"], w["N"], w["D"])
    shp_k = (w["B"], w["Hkv"], w["N"], w["D"])
    q = torch.randn(shp_q, generator=g, device=device)
    k = torch.randn(shp_k, generator=g, device=device)
    v = torch.randn(shp_k, generator=g, device=device)
    k += w["k_off"] * torch.randn((w["B"], w["Hkv"], 1, w["D"]), generator=g, device=device)
    if w["v_out"] > 0:
        n = max(1, int(round(w["D"] * w["v_out"])))
        idx = torch.randperm(w["D"], generator=g, device=device)[:n]
        v[..., idx] *= 8
    return tuple(t.to(torch.bfloat16) for t in (q, k, v))


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = sorted(float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i] == "Active" for r in self.rows)]
        # under load = upper half of the samples (idle samples before/after the region pull the median down)
        load = sm[len(sm) // 2:] if sm else []
        return {"sm_mhz": load[len(load) // 2] if load else None, "sm_max_mhz": mx[0] if mx else None,
                "samples": len(sm), "reasons": reasons}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("hbm_gbs"), d.get("bf16_tflops"), d.get("bf16_tflops_sustained"), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


# --------------------------------------------------------------------------------------------------
# CPU arm: the reference semantics in PyTorch (oracle/sage3.py) on the host cores
# --------------------------------------------------------------------------------------------------

def cpu_sample(w, seed=0, rows=256):
    """A bounded sample of the workload: one head, the first `rows` queries against all keys."""
    from oracle import sage3
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    N, D = w["N"], w["D"]
    q = torch.randn(1, 1, rows, D, generator=g).to(torch.bfloat16)
    k = (torch.randn(1, 1, N, D, generator=g) + w["k_off"] * torch.randn(1, 1, 1, D, generator=g)).to(torch.bfloat16)
    v = torch.randn(1, 1, N, D, generator=g).to(torch.bfloat16)
    t0 = time.perf_counter()
    sage3.sageattn3_emulated(q, k, v, is_causal=False)
    dt = time.perf_counter() - t0
    flops = attn_flops(1, 1, rows, N, D, False)
    return flops / dt / 1e12, dt, threads, f"1 head, first {rows} queries x all {N} keys of the workload, non-causal"


def run_reference_arm(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        tops, dt, threads, sample = cpu_sample(w, seed=i, rows=512)
        if i >= args.warmup:
            vals.append((tops, dt))
    tops = sum(v[0] for v in vals) / len(vals)
    ms = 1e3 * sum(v[1] for v in vals) / len(vals)
    line = {"impl": "reference", "metric": "attention_tops", "value": tops, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp32 emulation of fp4 (e2m1 x ue4m3)",
            "data": "synthetic", "config": {"workload": name, **{k: w[k] for k in ("B", "Hq", "Hkv", "N", "D", "causal")}},
            "cpu_baseline": {"value": tops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                             "sample": "per step: " + sample},
            "e2e": {"value": tops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# kernel sweep (the reference's bench/bench_baseline.py:9-11,30-31 shape: B=4, H=32)
# --------------------------------------------------------------------------------------------------

def run_sweep(args):
    import sageattention_b200 as sa
    dev = torch.device("cuda", 0)
    for D in (128, 64):
        for causal in (False, True):
            for N in (1024, 2048, 4096, 8192, 16384, 32768):
                w = dict(B=4, Hq=32, Hkv=32, N=N, D=D, causal=causal, k_off=0.0, v_out=0.0)
                q, k, v = gen_inputs(w, 1000 + N, dev)
                z = sa.quantize_qkv(q, k, v)
                for _ in range(8):
                    sa.fp4_attention(z, is_causal=causal)
                # back-to-back launches between two events, as the reference's bench times its kernel
                # (flash_attn's benchmark_forward): the host's per-call cost hides behind the queue
                reps = 20 if N <= 8192 else 5
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    sa.fp4_attention(z, is_causal=causal)
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / reps
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(4):
                    sa.sageattn(q, k, v, is_causal=causal)
                e1.record()
                torch.cuda.synchronize()
                ms_full = e0.elapsed_time(e1) / 4
                fl = attn_flops(4, 32, N, N, D, causal)
                # K-packing mode: same logical flops (the reference's reports count it that way), 16/15 more keys
                kp, vp, lam, _ = sa.pack_kv(k, v)
                zp = sa.quantize_qkv(q, kp, vp, per_block_mean=True, smooth_k=False)
                zp.k_lambda, zp.nk_slots = lam, (N // 15) * 16 + (0 if N % 15 == 0 else N % 15 + 1)
                for _ in range(4):
                    sa.fp4_attention(zp, is_causal=causal)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    sa.fp4_attention(zp, is_causal=causal)
                e1.record()
                torch.cuda.synchronize()
                ms_p = e0.elapsed_time(e1) / reps
                print(json.dumps({"sweep": True, "D": D, "causal": causal, "N": N, "kernel_ms": ms,
                                  "kernel_tops": fl / ms / 1e9, "operator_ms": ms_full,
                                  "operator_tops": fl / ms_full / 1e9, "packed_kernel_ms": ms_p,
                                  "packed_kernel_tops": fl / ms_p / 1e9}), flush=True)
                del q, k, v, z, kp, vp, lam, zp


# --------------------------------------------------------------------------------------------------
# the reference's own quantisation kernels on the same tensors (oracle/_ref, built by oracle/build_ref.py)
# --------------------------------------------------------------------------------------------------

def time_reference_quant(q, k, v, reps=3):
    """Milliseconds of the reference preprocessing on this GPU: eager K smoothing + padding, its Triton-free parts
    of the Q block mean done in eager PyTorch, delta_s GEMM, and its three CUDA quantisation kernels
    (quantization/fp4_quantization_4d.cu: scaled_fp4_quant, _permute, _trans), timed with CUDA events outside
    the bench's timed region.  Returns None when the checker library is not built."""
    import importlib.util
    so = ROOT / "oracle" / "_ref" / "sage_ref_quant_cuda.so"
    if not so.exists():
        return None
    spec = importlib.util.spec_from_file_location("sage_ref_quant_cuda", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    B, H, N, D = q.shape
    Hk = k.shape[1]
    Np = (N + 127) // 128 * 128
    dev = q.device
    pad = lambda x: torch.nn.functional.pad(x, (0, 0, 0, Np - N)) if Np != N else x

    def kernels_only(qs, ks, vp, bufs):
        ref.scaled_fp4_quant(qs, bufs[0], bufs[1], 1)
        ref.scaled_fp4_quant_permute(ks, bufs[2], bufs[3], 1)
        ref.scaled_fp4_quant_trans(vp, bufs[4], bufs[5], 1)

    def whole(bufs):
        ks = pad(k - k.mean(dim=-2, keepdim=True))                                  # api.py:184, 196-203
        qp = pad(q)
        g = qp.float().reshape(B, H, Np // 128, 128, D)
        qm = g.mean(dim=-2)
        qs = (g - qm.unsqueeze(-2)).to(torch.bfloat16).reshape(B, H, Np, D)         # api.py:26-72 (Triton there)
        kr = ks if H == Hk else ks.repeat_interleave(H // Hk, dim=1)
        ds = torch.matmul(qm.to(torch.bfloat16), kr.transpose(-2, -1)).float()      # api.py:201
        kernels_only(qs, ks, pad(v), bufs)
        return qs, ks, ds

    u8 = dict(dtype=torch.uint8, device=dev)
    f8 = dict(dtype=torch.float8_e4m3fn, device=dev)
    bufs = [torch.empty((B, H, Np, D // 2), **u8), torch.empty((B, H, Np, D // 16), **f8),
            torch.empty((B, Hk, Np, D // 2), **u8), torch.empty((B, Hk, Np, D // 16), **f8),
            torch.empty((B, Hk, D, Np // 2), **u8), torch.empty((B, Hk, D, Np // 16), **f8)]
    qs, ks, _ = whole(bufs)
    vp = pad(v)
    out = {}
    for name, fn in (("kernels_ms", lambda: kernels_only(qs, ks, vp, bufs)), ("pipeline_ms", lambda: whole(bufs))):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / reps
    return out


# --------------------------------------------------------------------------------------------------
# the long-sequence configuration (Ulysses all-to-all), part of every default run
# --------------------------------------------------------------------------------------------------

def _ulysses_parity(sa, sd, dist, dev, world, rank):
    """Reduced shape, every rank: the Ulysses output shard must be BITWISE the single-GPU operator's output for the
    same tokens when that operator is given the gathered full sequence of exactly the heads each Ulysses call
    attends (the K channel means are fp32 sums whose chunking depends on the number of heads in a call).  The ring
    scheme quantises every K/V shard on its own, so it is compared within a tolerance and against fp32 SDPA."""
    from oracle import sage3
    B, n, D = 1, 333, 128
    sizes = [1, 2]
    H = world * sum(sizes)
    g = torch.Generator(device=dev).manual_seed(77 + rank)
    q, k, v = (torch.randn((B, n, H, D), generator=g, device=dev).to(torch.bfloat16) for _ in range(3))
    k = (k.float() + 1.5).to(torch.bfloat16)
    full = []
    for t in (q, k, v):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        full.append(torch.cat(parts, dim=1))                        # [B, N, H, D]
    got = sd.ulysses_attention(q, k, v, head_chunks=sizes)
    want = torch.empty_like(full[0])
    start = 0
    for n_c in sizes:
        for p in range(world):
            sl = slice(start + p * n_c, start + (p + 1) * n_c)
            want[:, :, sl] = sa.sageattn(full[0][:, :, sl].contiguous(), full[1][:, :, sl].contiguous(),
                                         full[2][:, :, sl].contiguous(), tensor_layout="NHD")
        start += world * n_c
    mine = slice(rank * n, (rank + 1) * n)
    bitwise = bool(torch.equal(got, want[:, mine]))
    ring = sd.ring_attention(q, k, v)
    ref = sage3.sdpa_fp32(*(t.cpu().transpose(1, 2) for t in full)).transpose(1, 2)[:, mine]
    cos_ring, l1_ring = sage3.accuracy(ring.float().cpu(), ref)
    cos_one, l1_one = sage3.accuracy(want[:, mine].float().cpu(), ref)
    flags = torch.tensor([int(bitwise), int(cos_ring >= cos_one - 5e-3)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    return {"ulysses_parity": "bitwise" if int(flags[0]) else "MISMATCH",
            "ring_parity": {"ok": bool(int(flags[1])), "cos_vs_fp32_sdpa": cos_ring, "single_gpu_cos_vs_fp32_sdpa": cos_one,
                            "tolerance": "cosine vs fp32 SDPA no more than 5e-3 below the single-GPU operator's"},
            "parity_shape": {"B": B, "H": H, "N": n * world, "D": D, "head_chunks": sizes}}


def ulysses_head_chunks(hpr):
    """Heads per rank of every exchange / attention chunk: one head first and last (only the first exchange and the
    last return are exposed), a short ramp, and the bulk in one large chunk in the middle (every chunk is a launch
    sequence of its own and a round of the persistent attention kernel with a partly filled tail)."""
    if hpr <= 3:
        return [1] * hpr
    ramp = min(3, (hpr - 2) // 3) if hpr >= 8 else 0
    mid = hpr - 2 - 2 * ramp
    return [1] + ([ramp] if ramp else []) + [mid] + ([ramp] if ramp else []) + [1]


ULYSSES_SM_MARGIN = 8


def run_ulysses_leg(sa, dist, dev, world, rank, steps):
    w = WORKLOADS["ulysses"]
    B, H, N, D = w["B"], w["Hq"], w["N"], w["D"]
    flops = attn_flops(B, H, N, N, D, False)
    out = {"config": {"workload": "ulysses", "B": B, "H": H, "N": N, "D": D, "causal": False}, "n_gpus": world,
           "scaling": "strong", "steps": steps, "warmup": 3}

    def time_single():
        q, k, v = gen_inputs(w, seed=4321, device=dev)
        for _ in range(3):
            sa.sageattn(q, k, v)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sa.sageattn(q, k, v)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    if world == 1:
        ms = time_single()
        out.update(ms_per_step=ms, tops=flops / (ms * 1e-3) / 1e12, single_gpu_ms=ms, efficiency=1.0,
                   step="the plain operator on the whole problem (nothing to exchange on one GPU)")
        return out
    from sageattention_b200 import distributed as sd
    if N % world or H % world:
        out["skipped"] = f"{world} GPUs divide neither {H} heads nor {N} tokens"
        return out
    out.update(_ulysses_parity(sa, sd, dist, dev, world, rank))
    n, hpr = N // world, H // world
    g = torch.Generator(device=dev).manual_seed(4321 + rank)
    q = torch.randn((B, n, H, D), generator=g, device=dev).to(torch.bfloat16)
    koff = torch.randn((B, 1, H, D), generator=torch.Generator(device=dev).manual_seed(99), device=dev) * w["k_off"]
    k = (torch.randn((B, n, H, D), generator=g, device=dev) + koff).to(torch.bfloat16)
    v = torch.randn((B, n, H, D), generator=g, device=dev).to(torch.bfloat16)
    def timed(sizes, margin, warm):
        # max over ranks of the step time and of the time the compute stream waited for a collective
        for _ in range(warm):
            sd.ulysses_attention(q, k, v, head_chunks=sizes, sm_margin=margin)
        torch.cuda.synchronize()
        dist.barrier()
        exposed = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sd.ulysses_attention(q, k, v, head_chunks=sizes, exposed=exposed, sm_margin=margin)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps, sum(a.elapsed_time(b) for a, b in exposed) / steps],
                         device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # Overlapping the exchange with the attention of other heads hides the transfer, but the collectives' kernels
    # take SMs from the persistent attention kernel while they run and every chunk has its own tail.  Which wins
    # depends on the number of GPUs, so the schedules are tried out: heads in ramp-shaped chunks (with all SMs, and
    # with some left to the collectives) and all heads at once.  The step is reported for the best one, all are listed.
    ramp = ulysses_head_chunks(hpr)
    schedules = {"chunks": (ramp, 0), f"chunks, sm_margin {ULYSSES_SM_MARGIN}": (ramp, ULYSSES_SM_MARGIN),
                 "one exchange": ([hpr], 0)}
    tried = {name: timed(sz, m, 3 if i == 0 else 1) for i, (name, (sz, m)) in enumerate(schedules.items())}
    best = min(tried, key=lambda n: tried[n][0])
    ms, exp_ms = tried[best]
    sizes, margin = schedules[best]
    del q, k, v
    torch.cuda.empty_cache()
    single = time_single() if rank == 0 else 0.0
    dist.barrier()
    out.update(ms_per_step=ms, tops=flops / (ms * 1e-3) / 1e12, exposed_all_to_all_ms=exp_ms, single_gpu_ms=single,
               efficiency=(single / (world * ms)) if single else None, head_chunks=sizes, sm_margin=margin,
               schedule=best, ms_by_schedule={n: round(v[0], 3) for n, v in tried.items()},
               step=f"3 all-to-all in + operator + 1 all-to-all out per head chunk, {hpr} heads per GPU, best of the "
                    "schedules tried; "
                    "exposed = time the compute stream waited for a collective (max over ranks)")
    return out


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dit", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the device-timed steps (for profiling): no end-to-end leg, copy rates, reference "
                         "quantisation timing, FP4 peak measurement, Ulysses leg or CPU baseline")
    ap.add_argument("--sweep", action="store_true",
                    help="kernel-only TOPS over B=4 H=32, D in {64,128}, N = 1K..32K, causal and not (one JSON line per point)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference_arm(args, w, args.workload)
    if args.sweep:
        return run_sweep(args)
    args.warmup = max(args.warmup, 3)

    import sageattention_b200 as sa
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    if args.workload in ("ulysses", "ring"):
        from sageattention_b200 import distributed as sd
        if world < 2:
            raise SystemExit("the ulysses and ring workloads need >= 2 GPUs (torchrun)")
        return sd.bench_ulysses(args, w, dist, dev, ring=(args.workload == "ring"))

    B, Hq, Hkv, N, D, causal = w["B"], w["Hq"], w["Hkv"], w["N"], w["D"], w["causal"]
    q, k, v = gen_inputs(w, seed=1234 + rank, device=dev)
    flops = attn_flops(B, Hq, N, N, D, causal)
    sm_scale = D ** -0.5

    def step_split(evs=None):
        if evs:
            evs[0].record()
        z = sa.quantize_qkv(q, k, v)
        if evs:
            evs[1].record()
        o = sa.fp4_attention(z, sm_scale=sm_scale, is_causal=causal)
        if evs:
            evs[2].record()
        return o

    for _ in range(args.warmup):
        step_split()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    torch.cuda.synchronize()
    for i in range(args.steps):
        step_split(evs[i])
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = evs[0][0].elapsed_time(evs[-1][2])
    quant_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    attn_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    t = torch.tensor([total_ms, quant_ms, attn_ms], device=dev, dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, quant_ms, attn_ms = t.tolist()
    ms_per_step = total_ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": "attention_tops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                              "config": {"workload": args.workload},
                              "kernel_only": {"attention_ms": attn_ms, "preprocess_ms": quant_ms,
                                              "attention_tops": flops / (attn_ms * 1e-3) / 1e12}}), flush=True)
        if dist:
            dist.destroy_process_group()
        return

    # end to end through the public operator with HOST buffers: pinned H2D of q,k,v and D2H of the output
    qh, kh, vh = (x.cpu().pin_memory() for x in (q, k, v))
    oh = torch.empty_like(qh).pin_memory()

    def step_e2e():
        # host tensors in, host tensor out; copies of one head group overlap the kernels of another
        sa.sageattn_from_host(qh, kh, vh, out=oh, device=dev, is_causal=causal)

    for _ in range(2):
        step_e2e()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if dist:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_val = world * flops / (e2e_ms.item() * 1e-3) / 1e12
    h2d = sum(x.numel() * 2 for x in (qh, kh, vh))
    d2h = oh.numel() * 2

    # what the copies alone take on this rank (all ranks copy at the same time, as in the e2e step): pinned host ->
    # device of Q, K, V and device -> host of the output, each on its own, then the e2e step is compared with the
    # slower of the two (they run in opposite directions and overlap)
    def copy_ms(fn):
        fn()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(3):
            fn()
        c1.record()
        torch.cuda.synchronize()
        return c0.elapsed_time(c1) / 3
    o_dev = torch.empty_like(q)
    h2d_ms = copy_ms(lambda: [d.copy_(h, non_blocking=True) for d, h in ((q, qh), (k, kh), (v, vh))])
    d2h_ms = copy_ms(lambda: oh.copy_(o_dev, non_blocking=True))
    # ... and both directions at once, as in the pipelined step (the two share the host's memory system)
    side = torch.cuda.Stream(dev)

    def both():
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            oh.copy_(o_dev, non_blocking=True)
        for d, h in ((q, qh), (k, kh), (v, vh)):
            d.copy_(h, non_blocking=True)
        torch.cuda.current_stream(dev).wait_stream(side)
    both_ms = copy_ms(both)
    cm = torch.tensor([h2d_ms, d2h_ms, both_ms], device=dev, dtype=torch.float64)
    if dist:
        dist.all_reduce(cm, op=dist.ReduceOp.MAX)
    h2d_ms, d2h_ms, both_ms = cm.tolist()
    del o_dev

    ref_quant = time_reference_quant(q, k, v) if rank == 0 else None
    peak_tf, peak_note = None, None
    if rank == 0:
        import ctypes as C
        lib = sa._lib.load()
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        best = 0.0
        for n_cols in (128, 256):
            val = C.c_double()
            rc = lib.sage3_fp4_mma_peak(n_cols, 256, 8, st.data_ptr(), torch.cuda.current_stream().cuda_stream, C.byref(val))
            if rc == 0 and val.value > best:
                best, peak_note = val.value, f"M=128 N={n_cols} K=64"
        peak_tf = best if best > 0 else None
    del qh, kh, vh, oh, q, k, v
    torch.cuda.empty_cache()
    uly = run_ulysses_leg(sa, dist, dev, world, rank, steps=3) if args.workload == "dit" else None

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return
    hbm, bf16_burst, bf16_sus, which = measured_peaks()
    # tensor roofline: the dense block-scaled FP4 MMA rate measured on this GPU a moment ago (back-to-back
    # tcgen05.mma kind::mxf4nvf4 on resident operands, one CTA per SM); 4 x the cuBLAS bf16 figure only if that failed
    peak_fp4 = peak_tf if peak_tf else 4.0 * bf16_sus
    achieved = flops / (attn_ms * 1e-3) / 1e12
    Tq = (N + 127) // 128
    quant_bytes = B * N * ((Hq + 2 * Hkv) * (2 * D + D // 2 + D // 16))          # one read of Q, K, V + codes + scales
    line = {
        "metric": "attention_tops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4 (e2m1 x ue4m3 block-scaled, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "N": N, "D": D, "causal": causal,
                   "sharding": f"batch x heads over {world} GPU(s), no collective",
                   "l2": "inputs (3 x %.0f MB bf16) exceed the 126 MB L2" % (B * Hq * N * D * 2 / 1e6),
                   "step": "K mean + fused quant + delta_s + attention, inputs resident in HBM"},
        "kernel_only": {"attention_ms": attn_ms, "attention_tops": achieved, "preprocess_ms": quant_ms,
                        "preprocess_gbs": quant_bytes / (quant_ms * 1e-3) / 1e9,
                        "preprocess_frac_of_hbm": quant_bytes / (quant_ms * 1e-3) / 1e9 / hbm,
                        "reference_quant": (None if ref_quant is None else {
                            **ref_quant, "vs_reference_quant": ref_quant["pipeline_ms"] / quant_ms,
                            "what": "the reference's preprocessing on the same tensors and GPU: pipeline_ms = eager "
                                    "smoothing, block means, delta_s GEMM and its three CUDA quantisation kernels; "
                                    "kernels_ms = those three kernels alone; ratio = pipeline_ms / preprocess_ms"})},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_fp4, "unit": "TFLOP/s",
                     "frac": achieved / peak_fp4,
                     # DRAM bytes per launch from the ncu capture of a quarter of this workload, proportional to the
                     # number of heads
                     "traffic": (B * Hq * TRAFFIC_PER_HEAD_DIT) if (N == 32760 and D == 128 and not causal) else None,
                     "note": (f"peak = dense FP4 MMA rate measured live on this GPU ({peak_note}, sage3_fp4_mma_peak)"
                              if peak_tf else f"peak = 4 x {which} sustained bf16 cuBLAS (FP4 MMA measurement failed)")
                             + f"; for context 4 x {which} sustained bf16 cuBLAS = {4 * bf16_sus:.0f}, "
                               f"achieved / bf16 sustained = {achieved / bf16_sus:.3f}"},
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms.item(),
                "h2d_gbs_per_rank": h2d / (h2d_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (d2h_ms * 1e-3) / 1e9,
                "copy_bound_ms": max(h2d_ms, d2h_ms), "copies_both_directions_ms": both_ms,
                "note": "copy rates measured with all ranks copying at once, each direction alone; the step cannot be "
                        "shorter than the slower direction (copy_bound_ms), than the operator (ms_per_step of the line) "
                        "or - when it overlaps them completely - than the two directions running at the same time "
                        "(copies_both_directions_ms)"},
        "gpu_launches": 4 * args.steps,
        "clocks": clocks,
    }
    if uly is not None:
        line["ulysses"] = uly
    if not args.no_cpu_baseline:
        tops, dt, threads, sample = cpu_sample(w, rows=2048)
        line["cpu_baseline"] = {"value": tops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": sample, "seconds": dt}
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
