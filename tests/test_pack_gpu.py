"""GPU parity of the K-packing mode ("SageAttention4" of the fork, sageattn4/api.py:122-177, 250-288;
kernel side fwd_mainloop.cu:273-324, 796-891): the packing kernel against the CPU restatement (which is
itself pinned to the reference's preprocessing by tests/golden/pack_emulation.npz), the packed attention
kernel against the oracle run on the very operands the GPU consumed, and the whole operator.

Tolerances.  Packed K residuals and V: bit-exact except where the fp32 summation order of lambda moves a
value across a bf16 rounding boundary (at most 0.5 % of the elements, each by one bf16 ulp); lambda:
rel 2e-5.  Attention: cosine >= 0.999 and relative L1 <= 2e-2 against the oracle."""
import numpy as np
import pytest
import torch

import sageattention_b200 as sa
from oracle import nvfp4, sage3
from tests import _util as U
from tests.test_attn_gpu import COS_MIN, REL_L1_MAX

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("B,H,N,D", [(1, 2, 100, 64), (1, 2, 128, 128), (2, 3, 333, 128), (1, 1, 15, 128),
                                     (1, 1, 16, 64), (1, 2, 1, 128), (1, 2, 2000, 128)])
def test_pack_kernel_matches_oracle(B, H, N, D):
    _, k, v = U.make_qkv(B, H, H, 8, N, D, seed=N + D, device=DEV)
    kp, vp, lam, km = sa.pack_kv(k, v)
    torch.cuda.synchronize()
    k_s = (k.cpu() - km.cpu().unsqueeze(-2))                       # the K means are checked elsewhere
    kp_o, lam_o = sage3.pack_k(k_s)
    vp_o = sage3.pack_v(v.cpu())
    rows = kp_o.shape[-2]
    assert kp.shape == (B, H, rows, D) and lam.shape[-1] == (rows + 127) // 128 * 128
    assert torch.equal(vp.cpu(), vp_o)
    assert torch.equal(kp.cpu()[:, :, 0::16], kp_o[:, :, 0::16])  # the FP4-rounded group means: exact
    np.testing.assert_allclose(lam.cpu()[..., :rows].numpy(), lam_o.numpy(), rtol=2e-5, atol=2e-6)
    assert float(lam.cpu()[..., rows:].abs().max()) == 0.0 if lam.shape[-1] > rows else True
    a, b = kp.cpu().view(torch.int16).int(), kp_o.view(torch.int16).int()
    diff = (a - b).abs()
    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) <= 5e-3


def oracle_on_packed_operands(z, sm_scale, causal, mean_slot="mask"):
    B, Hq, Hkv, Nq, Nk, D = z.shape
    qc, qs = U.unpack_rows(z.q_codes, z.q_sf)
    kc, ks = U.unpack_rows(z.k_codes, z.k_sf)
    vc, vs = U.unpack_vt(z.vt_codes, z.vt_sf)
    qd = torch.from_numpy(nvfp4.dequantize_nvfp4(qc, qs))
    kd = torch.from_numpy(nvfp4.dequantize_nvfp4(kc, ks))
    vtd = torch.from_numpy(nvfp4.dequantize_nvfp4(vc, vs))
    ds = z.delta_s.float().cpu()
    if z.delta_s_rows == 1:
        ds = ds.expand(-1, -1, qd.shape[2] // 128, -1)
    return sage3.attention_quantised(qd, kd, vtd, ds, Nq, z.nk_slots, sm_scale, causal, lamb=z.k_lambda.cpu(),
                                     mean_slot=mean_slot)


CASES = [
    # B, Hq, Hkv, Nq, Nk, D, causal
    (1, 2, 2, 128, 128, 128, False),
    (1, 2, 2, 256, 240, 128, False),        # exactly two key tiles after packing
    (1, 4, 4, 512, 512, 128, True),
    (1, 8, 2, 640, 640, 128, True),         # GQA
    (1, 2, 2, 200, 333, 128, False),        # ragged
    (1, 2, 2, 333, 200, 128, True),         # causal with more queries than keys
    (1, 2, 1, 200, 333, 128, True),
    (1, 4, 2, 300, 300, 64, True),
    (1, 4, 4, 512, 500, 64, False),
    (1, 1, 1, 1, 1, 128, False),
    (1, 1, 1, 17, 5, 64, True),
]


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nk,D,causal", CASES)
def test_packed_kernel_matches_oracle_on_same_operands(B, Hq, Hkv, Nq, Nk, D, causal):
    q, k, v = U.make_qkv(B, Hq, Hkv, Nq, Nk, D, seed=Nq + Nk + D + 1, device=DEV)
    kp, vp, lam, _ = sa.pack_kv(k, v)
    z = sa.quantize_qkv(q, kp, vp, per_block_mean=True, smooth_k=False)
    z.k_lambda, z.nk_slots = lam, sage3.logical_to_packed_len(Nk)
    out = sa.fp4_attention(z, is_causal=causal, check_status=True)
    ref = oracle_on_packed_operands(z, D ** -0.5, causal)
    cos, l1 = sage3.accuracy(out.float().cpu(), ref)
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("causal", [False, True])
def test_packed_operator_matches_emulation(layout, causal):
    B, Hq, Hkv, N, D = 1, 4, 2, 700, 128
    q, k, v = U.make_qkv(B, Hq, Hkv, N, N, D, seed=11, layout=layout, device=DEV)
    out = sa.sageattn4_blackwell(q, k, v, tensor_layout=layout, is_causal=causal, check_status=True)
    hnd = (lambda t: t.transpose(1, 2)) if layout == "NHD" else (lambda t: t)
    emu = sage3.sageattn4_emulated(hnd(q).cpu().contiguous(), hnd(k).cpu().contiguous(), hnd(v).cpu().contiguous(),
                                   is_causal=causal)
    cos, l1 = sage3.accuracy(hnd(out).float().cpu(), emu.float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)
    sd = sage3.sdpa_fp32(hnd(q).cpu(), hnd(k).cpu(), hnd(v).cpu(), is_causal=causal)
    cos_k, _ = sage3.accuracy(hnd(out).float().cpu(), sd)
    cos_e, _ = sage3.accuracy(emu.float(), sd)
    assert cos_k >= cos_e - 2e-3                                   # no worse than the emulation against fp32 SDPA


def test_packed_mode_rejects_unsupported_variants():
    q, k, v = U.make_qkv(1, 2, 2, 64, 64, 128, seed=1, device=DEV)
    with pytest.raises(AssertionError):
        sa.sageattn4_blackwell(q, k, v, quant_block=8)


@pytest.mark.parametrize("B,H,N,D", [(1, 2, 100, 64), (2, 3, 333, 128), (1, 1, 16, 64), (1, 2, 2000, 128)])
def test_split_first_v_layout_matches_oracle(B, H, N, D):
    """The V layout of the reference's v_trick (api.py:158-170): bit-exact against the restatement, which is pinned
    to the reference's own preprocess_qkv by tests/golden/pack_emulation.npz."""
    _, k, v = U.make_qkv(B, H, H, 8, N, D, seed=N + D, device=DEV)
    _, vp, _, _ = sa.pack_kv(k, v, split_first=True)
    assert torch.equal(vp.cpu(), sage3.pack_v(v.cpu(), split_first=True))


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nk,D,causal", CASES)
def test_mean_slot_first_kernel_matches_oracle_on_same_operands(B, Hq, Hkv, Nq, Nk, D, causal):
    """The kernel variant the reference builds for per_block_mean=False (fwd_mainloop.cu:847-891): whole-sequence Q
    mean (one delta_s row), split-first V, the mean slot takes the first token's score and stays out of the row sum."""
    q, k, v = U.make_qkv(B, Hq, Hkv, Nq, Nk, D, seed=Nq + Nk + D + 2, device=DEV)
    kp, vp, lam, _ = sa.pack_kv(k, v, split_first=True)
    z = sa.quantize_qkv(q, kp, vp, per_block_mean=False, smooth_k=False)
    z.k_lambda, z.nk_slots, z.mean_slot_first = lam, sage3.logical_to_packed_len(Nk), True
    out = sa.fp4_attention(z, is_causal=causal, check_status=True)
    ref = oracle_on_packed_operands(z, D ** -0.5, causal, mean_slot="first")
    cos, l1 = sage3.accuracy(out.float().cpu(), ref)
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)


@pytest.mark.parametrize("causal", [False, True])
def test_packed_operator_whole_sequence_mean_variant_matches_emulation(causal):
    B, Hq, Hkv, N, D = 1, 4, 2, 700, 128
    q, k, v = U.make_qkv(B, Hq, Hkv, N, N, D, seed=12, device=DEV)
    out = sa.sageattn4_blackwell(q, k, v, is_causal=causal, per_block_mean=False, check_status=True)
    emu = sage3.sageattn4_emulated(q.cpu(), k.cpu(), v.cpu(), is_causal=causal, per_block_mean=False)
    cos, l1 = sage3.accuracy(out.float().cpu(), emu.float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)
    # the two V layouts are interchangeable for the masked-slot kernel (the slot's V row is never used there)
    out2 = sa.sageattn4_blackwell(q, k, v, is_causal=causal, per_block_mean=True, v_trick=True, check_status=True)
    emu2 = sage3.sageattn4_emulated(q.cpu(), k.cpu(), v.cpu(), is_causal=causal, per_block_mean=True, v_trick=True)
    cos, l1 = sage3.accuracy(out2.float().cpu(), emu2.float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)


@pytest.mark.parametrize("tag", ["s128", "s256"])
def test_packed_operator_on_reference_fixtures(tag):
    """The reference's real-activation inputs (tests/fixtures/*.pt) with its own thresholds against fp32 SDPA
    (tests/test.py:36-47: 1 - cos < 0.01, L1 < 0.01), K-packing operator."""
    from pathlib import Path
    z = np.load(Path(__file__).resolve().parent / "golden" / "llama_fixture_qkv.npz")
    bf = lambda name: torch.from_numpy(nvfp4.from_bf16_bits(z[f"{tag}_{name}"])).to(torch.bfloat16).to(DEV)
    q, k, v = bf("q"), bf("k"), bf("v")
    out = sa.sageattn4_blackwell(q, k, v, is_causal=False, check_status=True).float().cpu()
    ref = torch.from_numpy(z[f"{tag}_sdpa"])
    cos = torch.nn.functional.cosine_similarity(out, ref, dim=-1).mean().item()
    l1 = torch.nn.functional.l1_loss(out, ref).item()
    assert 1 - cos < 0.01 and l1 < 0.01, (cos, l1)
