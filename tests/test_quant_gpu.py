"""GPU parity of the fused smoothing + NVFP4 quantisation kernel.

Bit-exact bar: FP4 codes and E4M3 scale bytes must equal (a) the reference's own CUDA kernels
(quantization/fp4_quantization_4d.cu, compiled for sm_100a into oracle/_ref) and (b) the CPU oracle
in "device" mode, on the same smoothed bf16 values.  The means used for smoothing are floating-point
reductions whose summation order differs between implementations; tests that let the kernel compute
its own means therefore state a mismatch budget instead of demanding equality.
"""
import numpy as np
import pytest
import torch

import sageattention_b200 as sa
from oracle import nvfp4, sage3
from tests import _util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    mod = U.load_reference_quant()
    if mod is None:
        pytest.skip("oracle/_ref/sage_ref_quant_cuda.so not built")
    return mod


def ref_quant_rows(ref, x, permute=False):
    """x [B,H,Np,D] bf16 cuda (Np multiple of 128) -> logical codes/sf via the reference kernels."""
    B, H, N, D = x.shape
    codes = torch.zeros((B, H, N, D // 2), dtype=torch.uint8, device=x.device)
    sf = torch.zeros((B, H, N, D // 16), dtype=torch.float8_e4m3fn, device=x.device)
    (ref.scaled_fp4_quant_permute if permute else ref.scaled_fp4_quant)(x, codes, sf, 1)
    torch.cuda.synchronize()
    c = codes.cpu().numpy()
    s = nvfp4.ref_sf_unswizzle(sf.view(torch.uint8).cpu().numpy())
    if permute:   # output row p of each 128-block holds input token perm[p]
        perm = nvfp4.ref_k_row_permutation()
        inv = np.argsort(perm)
        c = c.reshape(B, H, N // 128, 128, -1)[:, :, :, inv].reshape(B, H, N, -1)
        s = s.reshape(B, H, N // 128, 128, -1)[:, :, :, inv].reshape(B, H, N, -1)
    return c, s


def ref_quant_trans(ref, v):
    B, H, N, D = v.shape
    codes = torch.zeros((B, H, D, N // 2), dtype=torch.uint8, device=v.device)
    sf = torch.zeros((B, H, D, N // 16), dtype=torch.float8_e4m3fn, device=v.device)
    ref.scaled_fp4_quant_trans(v, codes, sf, 1)
    torch.cuda.synchronize()
    return codes.cpu().numpy(), nvfp4.ref_sf_unswizzle(sf.view(torch.uint8).cpu().numpy())


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("N", [128, 1024, 1000, 1])
def test_plain_quant_matches_reference_kernels(ref, D, N):
    q, k, v = U.make_qkv(2, 3, 3, N, N, D, seed=N + D, device=DEV)
    z = sa.quantize_qkv(q, k, v, per_block_mean=None, smooth_k=False, with_delta_s=False)
    qp, kp, vp = (sage3.pad_tokens(t) for t in (q, k, v))
    for mine, theirs in [(U.unpack_rows(z.q_codes, z.q_sf), ref_quant_rows(ref, qp)),
                         (U.unpack_rows(z.k_codes, z.k_sf), ref_quant_rows(ref, kp, permute=True)),
                         (U.unpack_vt(z.vt_codes, z.vt_sf), ref_quant_trans(ref, vp))]:
        assert np.array_equal(mine[1], theirs[1]), "scale bytes differ"
        assert np.array_equal(mine[0], theirs[0]), "fp4 codes differ"


def test_quant_matches_cpu_oracle_device_mode():
    if nvfp4.device_tables() is None:
        pytest.skip("tests/golden/device_tables.npz not generated yet")
    q, k, v = U.make_qkv(1, 2, 2, 384, 384, 128, seed=5, device=DEV)
    z = sa.quantize_qkv(q, k, v, per_block_mean=None, smooth_k=False, with_delta_s=False)
    c, s = U.unpack_rows(z.q_codes, z.q_sf)
    oc, os_ = nvfp4.quantize_nvfp4(U.bf16_np(q), "device")
    assert np.array_equal(s, os_) and np.array_equal(c, oc)
    cv, sv = U.unpack_vt(z.vt_codes, z.vt_sf)
    ocv, osv = nvfp4.quantize_nvfp4(U.bf16_np(v.transpose(-1, -2).contiguous()), "device")
    assert np.array_equal(sv, osv) and np.array_equal(cv, ocv)


def test_quant_vs_cpu_oracle_exact_mode_differs_only_rarely():
    # IEEE division (the reference's Python emulation) vs the GPU's approximate division: a code may
    # differ only where x/scale falls within an ulp of a rounding boundary.  Budget: 0.5 % of codes.
    q, k, v = U.make_qkv(1, 2, 2, 512, 512, 128, seed=6, device=DEV)
    z = sa.quantize_qkv(q, k, v, per_block_mean=None, smooth_k=False, with_delta_s=False)
    c, s = U.unpack_rows(z.q_codes, z.q_sf)
    oc, os_ = nvfp4.quantize_nvfp4(U.bf16_np(q), "exact")
    assert (s != os_).mean() < 5e-3
    lo, hi = (c & 15) != (oc & 15), (c >> 4) != (oc >> 4)
    assert (lo.mean() + hi.mean()) / 2 < 5e-3


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("N", [1024, 777])
def test_smoothed_quant_with_given_means_matches_reference(ref, layout, N):
    """With the means taken from PyTorch (what the reference's eager preprocessing computes) the whole
    preprocessing + quantisation result is bit-identical to the reference pipeline."""
    B, Hq, Hkv, D = 2, 4, 2, 128
    q, k, v = U.make_qkv(B, Hq, Hkv, N, N, D, seed=N, layout=layout, device=DEV)
    qh, kh, vh = (t if layout == "HND" else t.transpose(1, 2) for t in (q, k, v))
    km = kh.mean(dim=-2, keepdim=True)                                      # api.py:184
    ks = sage3.pad_tokens(kh - km)
    qpad = sage3.pad_tokens(qh)
    g = qpad.float().reshape(B, Hq, -1, 128, D)
    qm32 = g.sum(dim=-2) / 128                                              # api.py:46
    qs = (g - qm32.unsqueeze(-2)).to(torch.bfloat16).reshape(qpad.shape)    # api.py:48-49
    z = sa.quantize_qkv(q, k, v, tensor_layout=layout, per_block_mean=True, smooth_k=True,
                        km=km.squeeze(-2), qm_fp32=qm32)
    for mine, theirs in [(U.unpack_rows(z.q_codes, z.q_sf), ref_quant_rows(ref, qs)),
                         (U.unpack_rows(z.k_codes, z.k_sf), ref_quant_rows(ref, ks, permute=True)),
                         (U.unpack_vt(z.vt_codes, z.vt_sf), ref_quant_trans(ref, sage3.pad_tokens(vh)))]:
        assert np.array_equal(mine[1], theirs[1]) and np.array_equal(mine[0], theirs[0])
    assert torch.equal(z.qm, qm32.to(torch.bfloat16))
    # delta_s = bf16(qm @ ks^T) widened to fp32 (api.py:201); fp32 accumulation order may differ from
    # cuBLAS, so allow one bf16 ulp on a few entries
    ks_rep = ks.repeat_interleave(Hq // Hkv, dim=1)
    want = torch.matmul(qm32.to(torch.bfloat16), ks_rep.transpose(-2, -1)).float()
    got = z.delta_s.float()
    close = (got - want).abs() <= want.abs() * 2.0 ** -7 + 1e-6
    assert close.all() and (got != want).float().mean() < 0.02


def test_self_computed_means_are_close_to_torch():
    """The kernel's own means (fp32 sums in its own order) vs PyTorch's: equal up to rounding of the
    bf16 result; the budget is 2 % of mean entries off by at most one bf16 ulp, and < 0.5 % of codes."""
    B, Hq, Hkv, N, D = 1, 4, 4, 2048, 128
    q, k, v = U.make_qkv(B, Hq, Hkv, N, N, D, seed=11, k_offset_std=2.0, device=DEV)
    z = sa.quantize_qkv(q, k, v)
    km = k.mean(dim=-2)
    diff = (z.km.float() - km.float()).abs()
    assert (diff <= km.float().abs() * 2.0 ** -7 + 1e-30).all()
    assert (diff > 0).float().mean() < 0.02
    z2 = sa.quantize_qkv(q, k, v, km=km)
    assert ((z.k_codes != z2.k_codes).float().mean()) < 5e-3


def test_whole_sequence_q_mean_mode():
    B, H, N, D = 1, 2, 300, 128
    q, k, v = U.make_qkv(B, H, H, N, N, D, seed=3, device=DEV)
    z = sa.quantize_qkv(q, k, v, per_block_mean=False)
    qpad = sage3.pad_tokens(q)
    qm = qpad.mean(dim=-2, keepdim=True)                                    # api.py:190
    assert (z.qm.float() - qm.float()).abs().max() <= qm.float().abs().max() * 2.0 ** -7
    qs = (qpad - z.qm)                                                      # with the kernel's own mean
    oc, os_ = nvfp4.quantize_nvfp4(U.bf16_np(qs), "device" if nvfp4.device_tables() else "exact")
    c, s = U.unpack_rows(z.q_codes, z.q_sf)
    assert (s != os_).mean() < 5e-3
    assert z.delta_s.shape == (B, H, 1, 384)


def test_bad_arguments_are_rejected():
    q, k, v = U.make_qkv(1, 2, 2, 128, 128, 128, device=DEV)
    with pytest.raises(AssertionError):
        sa.quantize_qkv(q.half(), k.half(), v.half())
    big = torch.zeros(1, 2, 128, 136, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        sa.sageattn3_blackwell(big, big, big)                   # head dims above 128: core.py:937
    with pytest.raises(ValueError):
        sa.sageattn3_blackwell(q, k, v, tensor_layout="XYZ")
    q3 = torch.cat([q, q], dim=1)[:, :3].contiguous()      # 3 query heads over 2 kv heads
    with pytest.raises(ValueError):
        sa.sageattn3_blackwell(q3, k, v)
