"""sage3_k_mean_static: the K channel means for callers that cannot allocate device memory (the
reduction scratch is a fixed array inside the library).  Called through the C ABI and compared with
the K means the allocating entry point (sage3_quant_qkv, caller-provided scratch) produces - same
kernel, same summation order, so the results must be identical.  Two calls in a row on different
problems check that whatever the first call left in the shared array does not leak into the second.
This file sorts last on purpose: a run that stops at the first failure has then already run every
other test."""
import ctypes as C

import pytest
import torch

import sageattention_b200 as sa
from sageattention_b200 import _lib
from tests import _util as U

pytestmark = pytest.mark.gpu


def k_mean_static(k: torch.Tensor) -> torch.Tensor:
    lib = _lib.load()
    B, H, N, D = k.shape
    out = torch.full((B, H, D), float("nan"), dtype=torch.bfloat16, device=k.device)
    shape = _lib.Shape(B, H, H, N, N, D)
    kt = _lib.Tensor(k.data_ptr(), k.stride(0), k.stride(1), k.stride(2))
    stream = torch.cuda.current_stream(k.device).cuda_stream
    _lib.check(lib.sage3_k_mean_static(C.byref(shape), C.byref(kt), out.data_ptr(), stream), "sage3_k_mean_static")
    return out


def test_static_scratch_matches_allocating_entry_point_twice_in_a_row():
    for (B, H, N, D, seed) in [(2, 6, 5000, 128, 1), (1, 3, 777, 64, 2)]:
        q, k, v = U.make_qkv(B, H, H, 128, N, D, seed=seed, k_offset_std=2.0, device="cuda")
        want = sa.quantize_qkv(q, k, v, with_delta_s=False).km
        got = k_mean_static(k)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (B, H, N, D)
        ref = k.float().mean(dim=-2)
        assert (got.float() - ref).abs().max() <= ref.abs().max() * 2.0 ** -7


def test_static_scratch_rejects_oversized_problems():
    lib = _lib.load()
    k = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    kt = _lib.Tensor(k.data_ptr(), k.stride(0), k.stride(1), k.stride(2))
    out = torch.empty(1, 1, 128, dtype=torch.bfloat16, device="cuda")
    big = _lib.Shape(64, 64, 64, 128, 128, 128)          # 4096 heads > 2048 counters; rejected before any launch
    assert lib.sage3_k_mean_static(C.byref(big), C.byref(kt), out.data_ptr(), None) == _lib.ERR_TOO_LARGE
    assert b"fixed scratch" in lib.sage3_status_string(_lib.ERR_TOO_LARGE)
    # the other limit: few enough heads (64 <= 2048) but too many partial rows - 64 heads x 49 chunks of 4096 tokens
    rows = _lib.Shape(1, 64, 64, 128, 200000, 128)
    assert lib.sage3_k_mean_static(C.byref(rows), C.byref(kt), out.data_ptr(), None) == _lib.ERR_TOO_LARGE
    assert lib.sage3_k_mean_static(None, C.byref(kt), out.data_ptr(), None) == _lib.ERR_ARGUMENT
