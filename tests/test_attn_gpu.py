"""GPU parity of the FP4 attention kernel and of the whole operator.

Tolerance (floating point): cosine similarity >= 0.999 and relative L1 <= 2e-2 against the CPU
restatement of the reference arithmetic (oracle/sage3.py); both numbers are also checked, with the
reference test's own thresholds (tests/test.py:36-47: 1 - cos < 0.01), against fp32 SDPA.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import sageattention_b200 as sa
from oracle import nvfp4, sage3
from tests import _util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_L1_MAX = 0.999, 2e-2
LOG2E = 1.4426950408889634


def oracle_on_device_operands(z, sm_scale, causal, return_lse=False):
    """CPU oracle fed with the very codes / scales / delta_s the GPU kernel consumes."""
    B, Hq, Hkv, Nq, Nk, D = z.shape
    qc, qs = U.unpack_rows(z.q_codes, z.q_sf)
    kc, ks = U.unpack_rows(z.k_codes, z.k_sf)
    vc, vs = U.unpack_vt(z.vt_codes, z.vt_sf)
    qd = torch.from_numpy(nvfp4.dequantize_nvfp4(qc, qs))
    kd = torch.from_numpy(nvfp4.dequantize_nvfp4(kc, ks))
    vtd = torch.from_numpy(nvfp4.dequantize_nvfp4(vc, vs))
    ds = None
    if z.delta_s is not None:
        ds = z.delta_s.float().cpu()
        if z.delta_s_rows == 1:
            ds = ds.expand(-1, -1, qd.shape[2] // 128, -1)
    return sage3.attention_quantised(qd, kd, vtd, ds, Nq, Nk, sm_scale, causal, return_lse)


CASES = [
    # B, Hq, Hkv, Nq, Nk, D, causal
    (1, 2, 2, 128, 128, 128, False),
    (1, 2, 2, 256, 256, 128, False),
    (1, 8, 8, 1024, 1024, 128, False),      # benchmark config 1 shape
    (2, 4, 4, 512, 512, 128, True),
    (1, 8, 2, 640, 640, 128, True),         # GQA
    (1, 2, 2, 200, 333, 128, False),        # ragged, Nq != Nk
    (1, 2, 2, 333, 200, 128, True),         # causal with more queries than keys (rows without keys)
    (1, 2, 1, 200, 333, 128, True),
    (1, 4, 4, 512, 512, 64, False),
    (1, 4, 2, 300, 300, 64, True),
    (1, 1, 1, 1, 1, 128, False),
    (1, 1, 1, 17, 5, 64, False),
]


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nk,D,causal", CASES)
def test_kernel_matches_oracle_on_same_operands(B, Hq, Hkv, Nq, Nk, D, causal):
    q, k, v = U.make_qkv(B, Hq, Hkv, Nq, Nk, D, seed=Nq + Nk + D, device=DEV)
    sm_scale = D ** -0.5
    z = sa.quantize_qkv(q, k, v)
    out, lse = sa.fp4_attention(z, sm_scale=sm_scale, is_causal=causal, return_lse=True, check_status=True)
    want, want_lse = oracle_on_device_operands(z, sm_scale, causal, return_lse=True)
    assert torch.isfinite(out).all()
    cos, l1 = sage3.accuracy(out.float().cpu(), want.to(torch.bfloat16).float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)
    fin = torch.isfinite(want_lse)
    assert torch.allclose(lse.cpu()[fin], want_lse[fin], atol=2e-3, rtol=1e-4)
    # rows that see no key (causal, more queries than keys): one sentinel, -inf, whether the whole query tile or only
    # the row is without keys - what an LSE merge over key shards expects
    assert bool(torch.isneginf(lse.cpu()[~fin]).all())
    if causal and Nq > Nk:
        assert int((~fin).sum()) == B * Hq * (Nq - Nk)


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nk,D,causal", CASES[:10])
@pytest.mark.parametrize("layout", ["HND", "NHD"])
def test_operator_matches_emulation_and_sdpa(B, Hq, Hkv, Nq, Nk, D, causal, layout):
    q, k, v = U.make_qkv(B, Hq, Hkv, Nq, Nk, D, seed=7 + Nq, k_offset_std=2.0, layout=layout, device=DEV)
    out = sa.sageattn(q, k, v, tensor_layout=layout, is_causal=causal, check_status=True)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    qh, kh, vh = (t.cpu() if layout == "HND" else t.cpu().transpose(1, 2) for t in (q, k, v))
    oh = out.cpu() if layout == "HND" else out.cpu().transpose(1, 2)
    mode = "device" if nvfp4.device_tables() is not None else "exact"
    emu = sage3.sageattn3_emulated(qh, kh, vh, is_causal=causal, mode=mode)
    cos, l1 = sage3.accuracy(oh.float(), emu.float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, ("vs emulation", cos, l1)
    # against fp32 SDPA the FP4 operator is only as accurate as the reference arithmetic allows on
    # this data; it must not be less accurate than the emulation of that arithmetic
    ref = sage3.sdpa_fp32(qh, kh, vh, is_causal=causal)
    cos2, l12 = sage3.accuracy(oh.float(), ref)
    cos3, l13 = sage3.accuracy(emu.float(), ref)
    assert cos2 >= cos3 - 3e-3 and l12 <= l13 + 1e-2, ("vs sdpa", cos2, l12, "emulation", cos3, l13)
    assert cos2 > 0.95


def test_sm_scale_and_lse_against_sdpa():
    B, H, N, D = 1, 4, 384, 128
    q, k, v = U.make_qkv(B, H, H, N, N, D, seed=21, device=DEV)
    sm = 0.05
    out, lse = sa.sageattn3_blackwell(q, k, v, sm_scale=sm, return_lse=True, check_status=True)
    s = torch.matmul(q.float().cpu(), k.float().cpu().transpose(-2, -1)) * sm
    want_lse = torch.logsumexp(s, dim=-1)
    assert (lse.cpu() - want_lse).abs().max() < 0.05
    emu = sage3.sageattn3_emulated(q.cpu(), k.cpu(), v.cpu(), sm_scale=sm)
    cos, l1 = sage3.accuracy(out.float().cpu(), emu.float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)


def test_whole_sequence_mean_and_no_smoothing_variants():
    q, k, v = U.make_qkv(1, 2, 2, 384, 384, 128, seed=4, device=DEV)
    for kw, okw in ((dict(per_block_mean=False), dict(per_block_mean=False)),
                    (dict(smooth_k=False), dict(smooth=False))):
        emu = sage3.sageattn3_emulated(q.cpu(), k.cpu(), v.cpu(), **okw)
        out = sa.sageattn3_blackwell(q, k, v, check_status=True, **kw)
        cos, l1 = sage3.accuracy(out.float().cpu(), emu.float())
        assert cos >= COS_MIN and l1 <= REL_L1_MAX, (kw, cos, l1)


@pytest.mark.parametrize("tag", ["s128", "s256"])
def test_reference_llama_fixtures(tag):
    # the reference's only test (tests/test.py): real activations, thresholds vs SDPA
    z = np.load(Path(__file__).parent / "golden" / "llama_fixture_qkv.npz")
    q, k, v = (torch.from_numpy(nvfp4.from_bf16_bits(z[f"{tag}_{n}"])).to(torch.bfloat16).to(DEV) for n in "qkv")
    out = sa.sageattn3_blackwell(q, k, v, is_causal=False, per_block_mean=True, check_status=True).float().cpu()
    ref = torch.from_numpy(z[f"{tag}_sdpa"])
    cos = torch.nn.functional.cosine_similarity(out, ref, dim=-1).mean().item()
    l1 = torch.nn.functional.l1_loss(out, ref).item()
    assert 1 - cos < 0.01 and l1 < 0.01, (cos, l1)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D", [128, 64])
def test_varlen_matches_per_sequence_calls(causal, D):
    """One pass over a packed variable-length batch (sage3_attention_varlen) against one dense call per
    sequence and against fp32 SDPA.  Not bit-identical to the dense calls: the K channel means are fp32
    sums whose chunking depends on the batch shape, so a mean can differ in its last bf16 bit."""
    Hq, Hkv = 4, 2
    # equal neighbours, ragged ones, a single token, a sequence without keys, one without queries
    lens_q, lens_k = [100, 257, 200, 200, 200, 1, 64, 5, 0, 300], [130, 257, 300, 300, 300, 40, 64, 0, 17, 300]
    g = torch.Generator().manual_seed(0)
    q = torch.randn(sum(lens_q), Hq, D, generator=g).to(torch.bfloat16).to(DEV)
    k = (torch.randn(sum(lens_k), Hkv, D, generator=g) + 1.5).to(torch.bfloat16).to(DEV)
    v = torch.randn(sum(lens_k), Hkv, D, generator=g).to(torch.bfloat16).to(DEV)
    cq = torch.tensor([0] + np.cumsum(lens_q).tolist(), dtype=torch.int32, device=DEV)
    ck = torch.tensor([0] + np.cumsum(lens_k).tolist(), dtype=torch.int32, device=DEV)
    out = sa.sageattn_varlen(q, k, v, cq, ck, max(lens_q), max(lens_k) + 50, is_causal=causal, check_status=True)
    assert out.shape == q.shape
    for i in range(len(lens_q)):
        qs, ks = slice(int(cq[i]), int(cq[i + 1])), slice(int(ck[i]), int(ck[i + 1]))
        if lens_q[i] == 0:
            continue
        if lens_k[i] == 0:
            assert float(out[qs].float().abs().max()) == 0.0
            continue
        one = sa.sageattn(q[qs][None], k[ks][None], v[ks][None], tensor_layout="NHD", is_causal=causal)[0]
        cos, l1 = sage3.accuracy(out[qs].float().cpu(), one.float().cpu())
        assert cos >= 0.9995 and l1 <= 2e-2, (i, cos, l1)
        if causal and lens_q[i] > lens_k[i]:
            continue            # rows without any key: SDPA gives NaN there, the kernels zeros (checked above)
        ref = sage3.sdpa_fp32(q[qs].cpu().transpose(0, 1)[None], k[ks].cpu().transpose(0, 1)[None],
                              v[ks].cpu().transpose(0, 1)[None], is_causal=causal)[0].transpose(0, 1)
        cos, _ = sage3.accuracy(out[qs].float().cpu(), ref)
        assert 1 - cos < 0.03, (i, cos)


def test_full_size_properties():
    """Size-independent checks at a benchmark-sized problem (too large for the CPU oracle):
    (1) rows of V all equal -> output equals that row up to the FP4 rounding of V (a few percent);
    (2) permuting the keys (and values) changes the output only by quantisation noise; (3) attention
    over keys [A | B] equals the LSE-weighted merge of attention over A and over B, again up to
    quantisation noise.  The noise floor on this N(0,1) data is the operator's own accuracy against
    fp32 attention (cosine about 0.985), so two FP4 evaluations agree to about 0.97."""
    B, H, N, D = 1, 4, 8192, 128
    q, k, v = U.make_qkv(B, H, H, N, N, D, seed=99, device=DEV)
    vc = v[:, :, :1].expand(-1, -1, N, -1).contiguous()
    out = sa.sageattn3_blackwell(q, k, vc, check_status=True)
    cos, l1 = sage3.accuracy(out.float().cpu(), vc.float().cpu())
    assert cos > 0.999 and l1 < 5e-2, (cos, l1)
    base, lse = sa.sageattn3_blackwell(q, k, v, return_lse=True, check_status=True)
    perm = torch.randperm(N, device=DEV)
    outp = sa.sageattn3_blackwell(q, k[:, :, perm].contiguous(), v[:, :, perm].contiguous(), check_status=True)
    cos, l1 = sage3.accuracy(outp.float().cpu(), base.float().cpu())
    assert cos > 0.96, (cos, l1)
    h = N // 2
    oa, la = sa.sageattn3_blackwell(q, k[:, :, :h].contiguous(), v[:, :, :h].contiguous(), return_lse=True)
    ob, lb = sa.sageattn3_blackwell(q, k[:, :, h:].contiguous(), v[:, :, h:].contiguous(), return_lse=True)
    lm = torch.logaddexp(la, lb)
    merged = oa.float() * (la - lm).exp()[..., None] + ob.float() * (lb - lm).exp()[..., None]
    cos, l1 = sage3.accuracy(merged.cpu(), base.float().cpu())
    assert cos > 0.96, (cos, l1)
    assert (lm - lse).abs().max() < 0.05


def test_host_tensor_entry_point_matches_device_operator():
    q, k, v = U.make_qkv(2, 8, 4, 300, 300, 128, seed=12)
    want = sa.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=True).cpu()
    for chunks in (1, 3, 8):
        got = sa.sageattn_from_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), head_chunks=chunks, is_causal=True)
        torch.cuda.synchronize()
        assert torch.equal(got, want), chunks


def test_custom_op_runs_and_matches_direct_call():
    from sageattention_b200 import compile_ops
    q, k, v = U.make_qkv(1, 4, 2, 300, 300, 128, seed=5, device=DEV)
    for packing in (False, True):
        direct = (sa.sageattn4_blackwell if packing else sa.sageattn3_blackwell)(q, k, v, is_causal=True)
        via_op = compile_ops.sageattn_compilable(q, k, v, is_causal=True, k_packing=packing)
        assert torch.equal(direct, via_op)
    torch.library.opcheck(compile_ops.fp4_attention_op, (q, k, v, "HND", False, 0.0, True, False),
                          test_utils=("test_schema", "test_faketensor"))


def test_operator_can_be_captured_in_a_cuda_graph():
    """The whole operator (memsets + four kernels, no allocation or synchronisation inside the library) is
    captured once and replayed on new input values."""
    q, k, v = U.make_qkv(2, 4, 2, 700, 700, 128, seed=21, device=DEV)
    for _ in range(2):
        sa.sageattn(q, k, v, is_causal=True)                   # warm up (lazy driver look-ups, allocator)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = sa.sageattn(q, k, v, is_causal=True)
    q2, k2, v2 = U.make_qkv(2, 4, 2, 700, 700, 128, seed=22, device=DEV)
    q.copy_(q2); k.copy_(k2); v.copy_(v2)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, sa.sageattn(q2, k2, v2, is_causal=True))


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier nothing completes runs out after its (short) poll limit: the kernel returns normally, the
    status word carries its code, the host call maps it to SAGE3_ERR_DEVICE_WAIT and the context stays usable."""
    import ctypes as C
    from sageattention_b200 import _lib
    lib = _lib.load()
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sage3_selftest_bounded_wait(st.data_ptr(), stream) == _lib.OK
    code = C.c_int32(0)
    assert lib.sage3_read_device_status(st.data_ptr(), stream, C.byref(code)) == _lib.ERR_DEVICE_WAIT
    assert code.value == 77
    # the device is still fine: a real operator call right after it succeeds
    q, k, v = U.make_qkv(1, 2, 2, 256, 256, 128, seed=1, device=DEV)
    out = sa.sageattn(q, k, v, check_status=True)
    assert torch.isfinite(out).all()


def test_varlen_sequences_longer_than_max_seqlen_are_cut_not_overrun():
    """A caller that passes max_seqlen smaller than its longest sequence gets that sequence cut at max_seqlen (the
    operand layouts and the workspace are sized by it): no tile index beyond the layouts is ever formed."""
    Hq, Hkv, D = 2, 2, 128
    lens = [300, 700, 128]
    g = torch.Generator().manual_seed(5)
    q = torch.randn(sum(lens), Hq, D, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(sum(lens), Hkv, D, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(sum(lens), Hkv, D, generator=g).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0] + np.cumsum(lens).tolist(), dtype=torch.int32, device=DEV)
    cap = 384
    out = sa.sageattn_varlen(q, k, v, cu, cu, cap, cap, is_causal=False, check_status=True)
    for i, n in enumerate(lens):
        s0 = int(cu[i])
        m = min(n, cap)
        one = sa.sageattn(q[s0:s0 + m][None], k[s0:s0 + m][None], v[s0:s0 + m][None], tensor_layout="NHD")[0]
        cos, l1 = sage3.accuracy(out[s0:s0 + m].float().cpu(), one.float().cpu())
        assert cos >= 0.9995 and l1 <= 2e-2, (i, cos, l1)


def test_host_tensor_entry_point_batched_is_copy_bound_not_stride_bound():
    """B > 1: the head groups of a [B,H,N,D] host tensor are not contiguous across the batch; the entry point copies
    them batch entry by batch entry.  Same values as the device operator."""
    q, k, v = U.make_qkv(3, 8, 4, 500, 500, 128, seed=13)
    want = sa.sageattn(q.cuda(), k.cuda(), v.cuda(), is_causal=False).cpu()
    got = sa.sageattn_from_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), head_chunks=4)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


@pytest.mark.parametrize("D,layout,causal", [(96, "HND", False), (40, "NHD", True), (72, "HND", True), (100, "HND", False)])
def test_head_dims_other_than_64_and_128_are_zero_padded(D, layout, causal):
    """sageattention/core.py:925-937, :990: D < 64 -> 64, 64 < D < 128 -> 128 with zero channels, default scale from
    the original D, output cut back.  Multiples of 8 are padded inside the kernels (no copy), others in PyTorch."""
    B, Hq, Hkv, N = 1, 4, 2, 300
    q, k, v = U.make_qkv(B, Hq, Hkv, N, N, D, seed=D, layout=layout, device=DEV)
    out, lse = sa.sageattn(q, k, v, tensor_layout=layout, is_causal=causal, return_lse=True, check_status=True)
    assert out.shape == q.shape
    Dp = 64 if D < 64 else 128
    hnd = (lambda t: t.transpose(1, 2)) if layout == "NHD" else (lambda t: t)
    qp, kp, vp = (torch.nn.functional.pad(hnd(t).cpu(), (0, Dp - D)).contiguous() for t in (q, k, v))
    emu, emu_lse = sage3.sageattn3_emulated(qp, kp, vp, is_causal=causal, sm_scale=D ** -0.5, return_lse=True)
    cos, l1 = sage3.accuracy(hnd(out).float().cpu(), emu[..., :D].float())
    assert cos >= COS_MIN and l1 <= REL_L1_MAX, (cos, l1)
    assert torch.allclose(lse.cpu(), emu_lse, atol=5e-3, rtol=1e-4)


def test_sdpa_hook_runs_the_fp4_operator_on_the_gpu():
    """hooks.as_sdpa / patched_sdpa: bf16 CUDA tensors without a mask go to the FP4 operator (same bits as a direct
    call), anything else to PyTorch's own function."""
    import torch.nn.functional as F
    from sageattention_b200 import hooks
    q, k, v = U.make_qkv(1, 4, 4, 300, 300, 128, seed=8, device=DEV)
    want = sa.sageattn(q, k, v, is_causal=True)
    with hooks.patched_sdpa():
        got = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        masked = F.scaled_dot_product_attention(q, k, v, attn_mask=torch.ones(300, 300, dtype=torch.bool, device=DEV))
    assert torch.equal(got, want)
    ref = F.scaled_dot_product_attention(q, k, v)
    assert torch.allclose(masked.float(), ref.float(), atol=2e-2)      # went to PyTorch: an all-true mask changes nothing


def test_sm_margin_changes_the_grid_but_not_one_bit_of_the_result():
    """sm_margin leaves SMs to kernels running beside the persistent attention kernel (a collective's): fewer CTAs
    walk the same work list, every item is computed exactly as before."""
    q, k, v = U.make_qkv(1, 6, 2, 3000, 3000, 128, seed=31, k_offset_std=2.0, device="cuda")
    want, want_lse = sa.sageattn3_blackwell(q, k, v, is_causal=True, return_lse=True, check_status=True)
    for margin in (8, 40, 147, 500):
        got, lse = sa.sageattn3_blackwell(q, k, v, is_causal=True, return_lse=True, check_status=True, sm_margin=margin)
        assert torch.equal(got, want) and torch.equal(lse, want_lse), margin
    qz = sa.quantize_qkv(q, k, v)
    assert torch.equal(sa.fp4_attention(qz, is_causal=True, sm_margin=16), sa.fp4_attention(qz, is_causal=True))
    with pytest.raises(RuntimeError):
        sa.fp4_attention(qz, sm_margin=-1)
