"""Pins the CPU oracle against vectors produced by the reference's own Python code
(tests/golden/make_golden.py): the NVFP4 quantiser emulation of
sageattention3_blackwell/sageattn4/api.py:77-110 and the reference's real-activation fixtures."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nvfp4, sage3

G = Path(__file__).resolve().parent / "golden"


def f32(bits):
    return nvfp4.from_bf16_bits(bits)


def test_e2m1_tie_points_match_reference_emulation():
    # api.py:100-103: {0.25,0.75,1.25,1.75,2.5,3.5,5} at scale 1 -> codes {0,1,1,2,2,4,4}
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    got = nvfp4.e2m1_decode(nvfp4.e2m1_encode(mids))
    assert got.tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]
    assert nvfp4.e2m1_encode(np.float32(-0.0)) == 8 and nvfp4.e2m1_encode(np.float32(-7.0)) == 15


def test_e4m3_matches_torch_cast_on_finite_range():
    x = np.concatenate([np.linspace(0, 448, 20001), nvfp4.E4M3_VALUES, nvfp4._E4M3_MID]).astype(np.float32)
    ours = nvfp4.e4m3_decode(nvfp4.e4m3_encode(x))
    theirs = torch.from_numpy(x).to(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(ours, theirs)
    assert nvfp4.e4m3_encode(np.float32(1e9)) == 126      # satfinite


def test_rowwise_quant_matches_reference_emulation():
    z = np.load(G / "quant_emulation.npz")
    x, y = f32(z["x"]), f32(z["y"])
    got = nvfp4.from_bf16_bits(nvfp4.to_bf16_bits(nvfp4.fake_quant(x, "exact")))
    assert np.array_equal(got.view(np.uint32), y.view(np.uint32))


def test_tokenwise_quant_matches_reference_emulation():
    z = np.load(G / "quant_emulation.npz")
    xt, yt = f32(z["xt"]), f32(z["yt"])
    xt_t = np.ascontiguousarray(np.swapaxes(xt, -1, -2))
    got = np.swapaxes(nvfp4.fake_quant(xt_t, "exact"), -1, -2)
    got = nvfp4.from_bf16_bits(nvfp4.to_bf16_bits(got))
    assert np.array_equal(got, yt)


@pytest.mark.parametrize("tag", ["s128", "s256"])
def test_llama_fixture_smoothing_and_quant(tag):
    z = np.load(G / "llama_fixture_qkv.npz")
    k = torch.from_numpy(f32(z[f"{tag}_k"])).to(torch.bfloat16)
    v = torch.from_numpy(f32(z[f"{tag}_v"])).to(torch.bfloat16)
    ks, _ = sage3.smooth_k(k)
    assert np.array_equal(nvfp4.to_bf16_bits(ks.float().numpy()), z[f"{tag}_ks"])
    got = nvfp4.to_bf16_bits(nvfp4.fake_quant(ks.float().numpy()))
    assert np.array_equal(got, z[f"{tag}_ks_fq"])
    codes, sf = sage3.quant_v_transposed(v)
    vfq = sage3.dequant(codes, sf).transpose(-1, -2).contiguous().numpy()
    assert np.array_equal(nvfp4.to_bf16_bits(vfq), z[f"{tag}_v_fq"])


@pytest.mark.parametrize("tag", ["s128", "s256"])
def test_llama_fixture_attention_within_reference_thresholds(tag):
    # sageattention3_blackwell/tests/test.py:36-47: 1 - cos < 0.01 and L1 < 0.01 against SDPA
    z = np.load(G / "llama_fixture_qkv.npz")
    q, k, v = (torch.from_numpy(f32(z[f"{tag}_{n}"])).to(torch.bfloat16) for n in "qkv")
    out = sage3.sageattn3_emulated(q, k, v).float()
    ref = torch.from_numpy(z[f"{tag}_sdpa"])
    cos = torch.nn.functional.cosine_similarity(out, ref, dim=-1).mean().item()
    l1 = torch.nn.functional.l1_loss(out, ref).item()
    assert 1 - cos < 0.01 and l1 < 0.01, (cos, l1)
    assert torch.allclose(sage3.sdpa_fp32(q, k, v), ref, atol=2e-5)


def test_ref_sf_swizzle_roundtrip():
    rows, cols = 128, 8
    r, c = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    off = nvfp4.ref_sf_offset(r, c, cols)
    assert sorted(off.flatten().tolist()) == list(range(rows * cols))
    perm = nvfp4.ref_k_row_permutation()
    assert sorted(perm.tolist()) == list(range(128))
    assert perm[:10].tolist() == [0, 1, 8, 9, 16, 17, 24, 25, 2, 3]


@pytest.mark.parametrize("tag", ["rand", "s128"])
def test_k_packing_matches_reference_preprocessing(tag):
    """oracle.sage3.pack_k / pack_v / delta_s against the fork's own preprocess_qkv (api.py:112-205,
    per_block_mean=True), run unchanged on CPU by tests/golden/make_golden.py."""
    z = np.load(G / "pack_emulation.npz")
    bf = lambda name: torch.from_numpy(f32(z[f"{tag}_{name}"])).to(torch.bfloat16)
    q, k, v = bf("q"), bf("k"), bf("v")
    k_s, _ = sage3.smooth_k(k)
    kp, lam = sage3.pack_k(k_s)
    kp, lam = sage3.pad_tokens(kp), sage3.pad_tokens(lam.unsqueeze(-1)).squeeze(-1)
    vp = sage3.pad_tokens(sage3.pack_v(v))
    assert kp.shape == tuple(z[f"{tag}_kp"].shape) and sage3.logical_to_packed_len(k.shape[-2]) <= kp.shape[-2]
    assert torch.equal(vp, bf("vp"))
    assert torch.equal(kp, bf("kp"))
    np.testing.assert_allclose(lam.numpy(), z[f"{tag}_lam"], rtol=1e-6, atol=1e-7)
    _, qm = sage3.q_block_mean(sage3.pad_tokens(q))
    ds = torch.matmul(qm, kp.transpose(-2, -1)).float()
    np.testing.assert_allclose(ds.numpy(), z[f"{tag}_ds"], rtol=1e-6, atol=1e-6)
    for n in (0, 1, 14, 15, 16, 29, 30, 100, 32760):
        assert sage3.packed_len_to_logical(sage3.logical_to_packed_len(n)) == n
    # the other kernel variant (per_block_mean=False): whole-sequence Q mean, split-first V, one delta_s row
    vp0 = sage3.pad_tokens(sage3.pack_v(v, split_first=True))
    assert torch.equal(vp0, bf("vp0"))
    q_pad = sage3.pad_tokens(q)
    qm0 = q_pad.mean(dim=-2, keepdim=True)
    assert torch.equal(q_pad - qm0, bf("qs0"))
    ds0 = torch.matmul(qm0, kp.transpose(-2, -1)).float()
    np.testing.assert_allclose(ds0.numpy(), z[f"{tag}_ds0"], rtol=1e-6, atol=1e-6)


def test_sampled_query_tiles_equal_the_full_evaluation():
    """attention_quantised(q_tiles=...) - used to check a few tiles of a benchmark-sized problem - gives exactly the
    rows of the full evaluation."""
    torch.manual_seed(0)
    B, H, N, D = 1, 2, 512, 64
    q, k, v = (torch.randn(B, H, N, D).to(torch.bfloat16) for _ in range(3))
    qs, ks, vp, ds, _ = sage3.preprocess(q, k, v)
    qd = sage3.dequant(*sage3.quant_rows(qs)); kd = sage3.dequant(*sage3.quant_rows(ks))
    vtd = sage3.dequant(*sage3.quant_v_transposed(vp))
    for causal in (False, True):
        full, lse = sage3.attention_quantised(qd, kd, vtd, ds, 500, 500, D ** -0.5, causal, True)
        tiles = [1, 3]
        qsel = torch.cat([qd[:, :, t * 128:(t + 1) * 128] for t in tiles], 2)
        part, lp = sage3.attention_quantised(qsel, kd, vtd, ds[:, :, tiles], 500, 500, D ** -0.5, causal, True, q_tiles=tiles)
        assert torch.equal(part[:, :, :128], full[:, :, 128:256]) and torch.equal(part[:, :, 128:244], full[:, :, 384:500])
        assert torch.equal(lp[:, :, :128], lse[:, :, 128:256])


@pytest.mark.parametrize("causal", [False, True])
def test_k_packing_variants_agree_with_fp32_attention(causal):
    """Both K-packing kernel variants of the restatement (masked mean slot / mean slot takes the first score with the
    split-first V layout) stay within the reference test's thresholds of fp32 attention on the reference's fixture."""
    z = np.load(G / "llama_fixture_qkv.npz")
    q, k, v = (torch.from_numpy(f32(z[f"s256_{n}"])).to(torch.bfloat16) for n in "qkv")
    ref = sage3.sdpa_fp32(q, k, v, is_causal=causal)
    for pbm in (True, False):
        out = sage3.sageattn4_emulated(q, k, v, is_causal=causal, per_block_mean=pbm).float()
        cos = torch.nn.functional.cosine_similarity(out, ref, dim=-1).mean().item()
        l1 = torch.nn.functional.l1_loss(out, ref).item()
        assert 1 - cos < 0.01 and l1 < 0.01, (pbm, cos, l1)
