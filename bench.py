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

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return
    hbm, bf16_burst, bf16_sus, which = measured_peaks()
    peak_fp4 = 4.0 * bf16_sus          # dense FP4 : dense bf16 = 9 : 2.25 nominal; bf16 figure is the sustained one
    achieved = flops / (attn_ms * 1e-3) / 1e12
    Tq = (N + 127) // 128
    quant_bytes = B * N * ((Hq + 2 * Hkv) * (2 * D + D // 2 + D // 16)) + B * Hkv * N * 2 * D   # + second K read
    line = {
        "metric": "attention_tops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4 (e2m1 x ue4m3 block-scaled, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "Hq": Hq, "Hkv": Hkv, "N": N, "D": D, "causal": causal,
                   "sharding": f"batch x heads over {world} GPU(s), no collective",
                   "l2": "inputs (3 x %.0f MB bf16) exceed the 126 MB L2" % (q.numel() * 2 / 1e6),
                   "step": "K mean + fused quant + delta_s + attention, inputs resident in HBM"},
        "kernel_only": {"attention_ms": attn_ms, "attention_tops": achieved, "preprocess_ms": quant_ms,
                        "preprocess_gbs": quant_bytes / (quant_ms * 1e-3) / 1e9},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_fp4, "unit": "TFLOP/s",
                     "frac": achieved / peak_fp4,
                     # ncu, quarter-size capture (profiles/attn_fwd_kernel_quarter_dit.md): 30.05 MB of DRAM traffic per
                     # head at N = 32760, D = 128, proportional to the number of heads
                     "traffic": (B * Hq * 30.05e6) if (N == 32760 and D == 128 and not causal) else None,
                     "note": f"peak = 4 x {which} sustained bf16 cuBLAS ({bf16_sus} TF/s): dense FP4 is 4x dense bf16 on "
                             f"B200; vs bf16 sustained itself: {achieved / bf16_sus:.3f}"},
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms.item()},
        "gpu_launches": 4 * args.steps,
        "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        tops, dt, threads, sample = cpu_sample(w, rows=2048)
        line["cpu_baseline"] = {"value": tops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": sample, "seconds": dt}
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
