"""GPU parity of the persistent attention kernel where one CTA walks SEVERAL work items, and at the sizes of
the benchmark configurations.

The kernel launches at most one CTA per SM (148 on B200); a work item is a pair of 128-row query tiles of one
head (``csrc/attn.cu``; the reference's persistent loop is ``blackwell/fwd_kernel.cu:133,173`` over
``tile_scheduler.h:181-239``).  Every case here has more work items than SMs, so barrier phases, the K/V ring,
the Q slots and the output staging are reused across items.

* ``test_multi_item_*``: a few hundred work items, EVERY output row compared with the CPU restatement fed with the
  very operands the kernel consumed.
* ``test_benchmark_size_sampled``: the benchmark configurations themselves (tens of rounds per CTA); the oracle
  checks a few heads x query tiles {first, second, middle, last (ragged)} against ALL keys.

Tolerance (floating point): cosine similarity >= 0.999 and relative L1 <= 2e-2, LSE within 2e-3.
"""
import pytest
import torch

import sageattention_b200 as sa
from oracle import nvfp4, sage3
from tests import _util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_L1_MAX = 0.999, 2e-2
SMS = 148


def _work_items(B, Hq, Nq):
    return B * Hq * (((Nq + 127) // 128 + 1) // 2)


def _oracle_tiles(z, b, h, tiles, sm_scale, causal):
    """CPU oracle for query tiles ``tiles`` of (batch b, query head h) against all keys, from the device operands."""
    B, Hq, Hkv, Nq, Nk, D = z.shape
    hk = h // (Hq // Hkv)
    idx = torch.as_tensor(tiles, device=z.q_codes.device)
    qc, qs = U.unpack_rows(z.q_codes[b:b + 1, h:h + 1].index_select(2, idx), z.q_sf[b:b + 1, h:h + 1].index_select(2, idx))
    kc, ks = U.unpack_rows(z.k_codes[b:b + 1, hk:hk + 1], z.k_sf[b:b + 1, hk:hk + 1])
    vc, vs = U.unpack_vt(z.vt_codes[b:b + 1, hk:hk + 1], z.vt_sf[b:b + 1, hk:hk + 1])
    qd = torch.from_numpy(nvfp4.dequantize_nvfp4(qc, qs))
    kd = torch.from_numpy(nvfp4.dequantize_nvfp4(kc, ks))
    vtd = torch.from_numpy(nvfp4.dequantize_nvfp4(vc, vs))
    ds = None
    if z.delta_s is not None:
        ds = z.delta_s[b:b + 1, h:h + 1]
        ds = (ds.index_select(2, idx) if z.delta_s_rows > 1 else ds.expand(-1, -1, len(tiles), -1)).float().cpu()
    lam = None
    len_k = Nk
    if z.k_lambda is not None:
        lam = z.k_lambda[b:b + 1, hk:hk + 1].float().cpu()
        len_k = int(z.nk_slots)
    return sage3.attention_quantised(qd, kd, vtd, ds, Nq, len_k, sm_scale, causal, return_lse=True, lamb=lam,
                                     q_tiles=list(tiles))


def _check_all(z, out, lse, sm_scale, causal):
    """Every row of every head against the oracle, in one oracle pass over the whole batch."""
    B, Hq, Hkv, Nq, Nk, D = z.shape
    qc, qs = U.unpack_rows(z.q_codes, z.q_sf)
    kc, ks = U.unpack_rows(z.k_codes, z.k_sf)
    vc, vs = U.unpack_vt(z.vt_codes, z.vt_sf)
    qd = torch.from_numpy(nvfp4.dequantize_nvfp4(qc, qs))
    kd = torch.from_numpy(nvfp4.dequantize_nvfp4(kc, ks))
    vtd = torch.from_numpy(nvfp4.dequantize_nvfp4(vc, vs))
    ds = z.delta_s.float().cpu() if z.delta_s is not None else None
    lam, len_k = None, Nk
    if z.k_lambda is not None:
        lam, len_k = z.k_lambda.float().cpu(), int(z.nk_slots)
    want, want_lse = sage3.attention_quantised(qd, kd, vtd, ds, Nq, len_k, sm_scale, causal, return_lse=True, lamb=lam)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    ref = want.to(torch.bfloat16).float()
    cos, l1 = sage3.accuracy(got, ref)
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)
    # ... and per work item (a pair of query tiles of one head), so that one bad item cannot hide in the average
    for b in range(B):
        for h in range(Hq):
            for r0 in range(0, Nq, 256):
                g_, r_ = got[b, h, r0:r0 + 256], ref[b, h, r0:r0 + 256]
                if float(r_.abs().max()) == 0.0:                  # causal rows that see no key: zeros on both sides
                    assert float(g_.abs().max()) == 0.0, (b, h, r0)
                    continue
                cos, l1 = sage3.accuracy(g_, r_)
                assert cos >= COS_MIN and l1 <= 2 * REL_L1_MAX, (b, h, r0, cos, l1)
    if lse is not None:
        fin = torch.isfinite(want_lse)
        assert torch.allclose(lse.cpu()[fin], want_lse[fin], atol=2e-3, rtol=1e-4)


def _check_tiles(z, out, lse, picks, tiles, sm_scale, causal):
    B, Hq, Hkv, Nq, Nk, D = z.shape
    for b, h in picks:
        want, want_lse = _oracle_tiles(z, b, h, tiles, sm_scale, causal)
        for i, t in enumerate(tiles):
            rows = min(128, Nq - t * 128)
            got = out[b, h, t * 128:t * 128 + rows].float().cpu()
            ref = want[0, 0, i * 128:i * 128 + rows].to(torch.bfloat16).float()
            assert torch.isfinite(got).all(), (b, h, t)
            cos, l1 = sage3.accuracy(got, ref)
            assert cos >= COS_MIN and l1 <= REL_L1_MAX, (b, h, t, cos, l1)
            if lse is not None:
                wl = want_lse[0, 0, i * 128:i * 128 + rows]
                fin = torch.isfinite(wl)
                gl = lse[b, h, t * 128:t * 128 + rows].cpu()
                assert torch.allclose(gl[fin], wl[fin], atol=2e-3, rtol=1e-4), (b, h, t)


MULTI = [
    # B, Hq, Hkv, Nq, Nk, D, causal                work items
    (1, 16, 16, 2560, 2560, 128, False),         # 160: one full round + a partial, reversed one
    (2, 16, 4, 2560, 2560, 128, True),           # 320: three rounds, causal cost order over all heads, GQA
    (1, 20, 20, 2500, 2500, 64, False),          # 200, ragged tail, D = 64
    (1, 12, 4, 3300, 2900, 128, True),           # 156, Nq != Nk, odd number of query tiles (a half-empty item)
    (3, 8, 8, 1920, 2048, 64, True),             # 192 = 3 x 8 x 8 pairs (Tq = 15, odd)
]


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nk,D,causal", MULTI)
def test_multi_item_all_rows_match_oracle(B, Hq, Hkv, Nq, Nk, D, causal):
    assert _work_items(B, Hq, Nq) > SMS
    q, k, v = U.make_qkv(B, Hq, Hkv, Nq, Nk, D, seed=Nq + D + B, device=DEV)
    sm_scale = D ** -0.5
    z = sa.quantize_qkv(q, k, v)
    out, lse = sa.fp4_attention(z, sm_scale=sm_scale, is_causal=causal, return_lse=True, check_status=True)
    _check_all(z, out, lse, sm_scale, causal)


def test_multi_item_k_packing_mode():
    B, Hq, Hkv, N, D = 1, 16, 8, 2560, 128
    assert _work_items(B, Hq, N) > SMS
    q, k, v = U.make_qkv(B, Hq, Hkv, N, N, D, seed=3, device=DEV)
    lib = sa._lib.load()
    for causal in (False, True):
        kp, vp, lam, _ = sa.pack_kv(k, v)
        z = sa.quantize_qkv(q, kp, vp, per_block_mean=True, smooth_k=False)
        z.k_lambda, z.nk_slots = lam, lib.sage3_packed_len(N)
        out = sa.fp4_attention(z, is_causal=causal, check_status=True)
        _check_all(z, out, None, D ** -0.5, causal)


def _v_outliers(v, frac, seed):
    g = torch.Generator().manual_seed(seed)
    B, H, _, D = v.shape
    n = max(1, int(round(D * frac)))
    for b in range(B):
        for h in range(H):
            idx = torch.randperm(D, generator=g)[:n].to(v.device)
            v[b, h, :, idx] *= 8
    return v


def _device_qkv(B, Hq, Hkv, N, D, seed, k_offset_std):
    """Benchmark-sized inputs are drawn on the device (seeded): the CPU generator would take minutes."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.randn(B, Hq, N, D, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(B, Hkv, N, D, generator=g, device=DEV, dtype=torch.float32)
    if k_offset_std > 0:
        k = k + k_offset_std * torch.randn(B, Hkv, 1, D, generator=g, device=DEV)
    k = k.to(torch.bfloat16)
    v = torch.randn(B, Hkv, N, D, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    return q, k, v


BENCH = [
    # name, B, Hq, Hkv, N, D, causal, k offset std, V outlier fraction, (batch, head) picks
    ("dit", 1, 40, 40, 32760, 128, False, 2.0, 0.05, [(0, 0), (0, 17), (0, 39)]),
    ("prefill", 4, 32, 8, 8192, 128, True, 2.0 ** 0.5, 0.0, [(0, 0), (1, 13), (3, 31)]),
    ("sweep_d64_32k_causal", 4, 32, 32, 32768, 64, True, 0.0, 0.0, [(0, 0), (3, 31)]),
    ("ulysses_shard_5_heads", 1, 5, 5, 75600, 128, False, 2.0, 0.0, [(0, 0), (0, 4)]),
]


@pytest.mark.parametrize("name,B,Hq,Hkv,N,D,causal,koff,vfrac,picks", BENCH)
def test_benchmark_size_sampled(name, B, Hq, Hkv, N, D, causal, koff, vfrac, picks):
    q, k, v = _device_qkv(B, Hq, Hkv, N, D, seed=len(name), k_offset_std=koff)
    if vfrac > 0:
        v = _v_outliers(v, vfrac, seed=1)
    sm_scale = D ** -0.5
    z = sa.quantize_qkv(q, k, v)
    out, lse = sa.fp4_attention(z, sm_scale=sm_scale, is_causal=causal, return_lse=True, check_status=True)
    Tq = (N + 127) // 128
    tiles = sorted({0, 1, Tq // 2, Tq - 1})
    _check_tiles(z, out, lse, picks, tiles, sm_scale, causal)
    # the whole operator (its own workspace carving) gives the same rows
    whole = sa.sageattn3_blackwell(q, k, v, is_causal=causal, check_status=True)
    for b, h in picks:
        for t in tiles:
            a, w = whole[b, h, t * 128:(t + 1) * 128], out[b, h, t * 128:(t + 1) * 128]
            cos, l1 = sage3.accuracy(a.float().cpu(), w.float().cpu())
            assert cos >= 0.9999 and l1 <= 5e-3, (name, b, h, t, cos, l1)
