"""Python operator API of the B200 FP4 attention path.

Mirrors the reference's operator interface:

* ``sageattn(q, k, v, tensor_layout, is_causal, sm_scale, return_lse)`` - signature and semantics
  of ``sageattention/core.py:79-157`` (layouts "HND" ``[B,H,N,D]`` / "NHD" ``[B,N,H,D]``, GQA with
  ``Hq % Hkv == 0``, default scale ``D**-0.5``, optional log-sum-exp output);
* ``sageattn3_blackwell(q, k, v, ...)`` - the FP4 operator of
  ``sageattention3_blackwell/sageattn4/api.py:250-288`` without the fork's K-packing steps;
* ``sageattn4_blackwell(q, k, v, ...)`` - the same operator with the K-packing steps (15 tokens -> group
  mean + 15 residuals, ``api.py:122-177,267-274``);
* ``sageattn_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, ...)`` - ``sageattention/core.py:334-448``.

All tensor work happens in ``libsage3_b200.so`` (hand-written sm_100a CUDA behind a C ABI); this
file only allocates buffers, turns layouts into strides and passes pointers.  There is no
fallback path: without the library, or on a GPU that is not compute capability 10.x, the calls
raise.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib

_LOG2E = 1.4426950408889634


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _as_bhnd_strides(x: torch.Tensor, tensor_layout: str):
    """(B, H, N, D, stride_b, stride_h, stride_n) of a 4-D tensor in either layout."""
    if x.dim() != 4:
        raise ValueError("expected a 4-D tensor")
    if x.stride(-1) != 1:
        raise ValueError("the last dimension must be contiguous")       # core.py:274-277
    if tensor_layout == "HND":
        B, H, N, D = x.shape
        return B, H, N, D, x.stride(0), x.stride(1), x.stride(2)
    if tensor_layout == "NHD":
        B, N, H, D = x.shape
        return B, H, N, D, x.stride(0), x.stride(2), x.stride(1)
    raise ValueError(f"Unknown tensor layout: {tensor_layout}")


def _tensor_arg(x: torch.Tensor, sb, sh, sn) -> _lib.Tensor:
    return _lib.Tensor(x.data_ptr(), sb, sh, sn)


def _check_device(x: torch.Tensor):
    if not x.is_cuda:
        raise ValueError("sageattention_b200 runs on CUDA tensors only (no CPU path)")
    major, _ = torch.cuda.get_device_capability(x.device)
    if major != 10:
        raise ValueError(f"unsupported GPU: compute capability {torch.cuda.get_device_capability(x.device)}; "
                         "this build targets B200 (sm_100a) only")


def buffer_sizes(B: int, Hq: int, Hkv: int, Nq: int, Nk: int, D: int, per_block_mean: int = 1) -> _lib.Sizes:
    lib = _lib.load()
    z = _lib.Sizes()
    shape = _lib.Shape(B, Hq, Hkv, Nq, Nk, D)
    _lib.check(lib.sage3_buffer_sizes(C.byref(shape), per_block_mean, C.byref(z)), "sage3_buffer_sizes")
    return z


@dataclass
class QuantizedQKV:
    """Device buffers produced by :func:`quantize_qkv` (layouts in ``include/sage3_b200.h``)."""
    shape: Tuple[int, int, int, int, int, int]       # B, Hq, Hkv, Nq, Nk, D
    q_codes: torch.Tensor
    q_sf: torch.Tensor
    k_codes: torch.Tensor
    k_sf: torch.Tensor
    vt_codes: torch.Tensor
    vt_sf: torch.Tensor
    qm: Optional[torch.Tensor]
    km: Optional[torch.Tensor]
    delta_s: Optional[torch.Tensor]
    delta_s_rows: int
    k_lambda: Optional[torch.Tensor] = None          # K-packing mode: fp32 [B,Hkv,Tk*128]
    nk_slots: Optional[int] = None                   # K-packing mode: occupied key slots (<= Nk)
    mean_slot_first: bool = False                    # K-packing mode: the mean slot takes the first token's score


def quantize_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                 per_block_mean: Optional[bool] = True, smooth_k: bool = True, with_delta_s: bool = True,
                 km: Optional[torch.Tensor] = None, qm_fp32: Optional[torch.Tensor] = None) -> QuantizedQKV:
    """Smoothing + NVFP4 quantisation of Q, K, V in one fused launch.

    Stands in for ``preprocess_qkv`` + ``scale_and_quant_fp4`` / ``_permute`` / ``_transpose`` of
    ``sageattn4/api.py:112-229``.  ``per_block_mean``: True = per-128-token Q mean, False = whole
    sequence Q mean, None = leave Q as is.  ``with_delta_s=False`` skips delta_s.  ``km`` / ``qm_fp32``
    let a caller supply the means (used by the parity tests to separate rounding of the means from
    the quantiser).
    """
    lib = _lib.load()
    _check_device(q)
    for t in (q, k, v):
        if t.dtype != torch.bfloat16:
            raise AssertionError("TODO: support inputs other than bfloat16")     # api.py:257
    B, Hq, Nq, D, qsb, qsh, qsn = _as_bhnd_strides(q, tensor_layout)
    Bk, Hkv, Nk, Dk, ksb, ksh, ksn = _as_bhnd_strides(k, tensor_layout)
    Bv, Hv, Nv, Dv, vsb, vsh, vsn = _as_bhnd_strides(v, tensor_layout)
    if not (B == Bk == Bv and D == Dk == Dv and Hkv == Hv and Nk == Nv):
        raise ValueError("q, k, v shapes do not match")
    pbm = -1 if per_block_mean is None else int(bool(per_block_mean))
    z = buffer_sizes(B, Hq, Hkv, Nq, Nk, D, pbm)
    dev = q.device
    u8 = dict(dtype=torch.uint8, device=dev)
    Tq, Tk = (Nq + 127) // 128, (Nk + 127) // 128
    out = QuantizedQKV(
        shape=(B, Hq, Hkv, Nq, Nk, D),
        q_codes=torch.empty((B, Hq, Tq, 128, D // 2), **u8), q_sf=torch.empty((B, Hq, Tq, D // 64, 512), **u8),
        k_codes=torch.empty((B, Hkv, Tk, 128, D // 2), **u8), k_sf=torch.empty((B, Hkv, Tk, D // 64, 512), **u8),
        vt_codes=torch.empty((B, Hkv, Tk, D, 64), **u8), vt_sf=torch.empty((B, Hkv, Tk, 2, 512), **u8),
        qm=None, km=None, delta_s=None, delta_s_rows=1)
    ds_rows = Tq if pbm == 1 else 1
    if pbm >= 0:
        out.qm = torch.empty((B, Hq, ds_rows, D), dtype=torch.bfloat16, device=dev)
        if with_delta_s:
            out.delta_s = torch.empty((B, Hq, ds_rows, Tk * 128), dtype=torch.bfloat16, device=dev)
            out.delta_s_rows = ds_rows
    if smooth_k:
        out.km = km.contiguous() if km is not None else torch.empty((B, Hkv, D), dtype=torch.bfloat16, device=dev)
    scratch = torch.empty(max(int(z.scratch), 256), **u8)
    a = _lib.QuantArgs()
    a.shape = _lib.Shape(B, Hq, Hkv, Nq, Nk, D)
    a.q, a.k, a.v = _tensor_arg(q, qsb, qsh, qsn), _tensor_arg(k, ksb, ksh, ksn), _tensor_arg(v, vsb, vsh, vsn)
    a.per_block_mean, a.smooth_k = pbm, int(smooth_k)
    a.km_in = out.km.data_ptr() if (smooth_k and km is not None) else None
    if qm_fp32 is not None:
        qm_fp32 = qm_fp32.to(device=dev, dtype=torch.float32).contiguous()
        a.qm_in = qm_fp32.data_ptr()
    a.q_codes, a.q_sf = out.q_codes.data_ptr(), out.q_sf.data_ptr()
    a.k_codes, a.k_sf = out.k_codes.data_ptr(), out.k_sf.data_ptr()
    a.vt_codes, a.vt_sf = out.vt_codes.data_ptr(), out.vt_sf.data_ptr()
    a.qm = out.qm.data_ptr() if out.qm is not None else None
    a.km = out.km.data_ptr() if out.km is not None else None
    a.delta_s = out.delta_s.data_ptr() if out.delta_s is not None else None
    a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    with torch.cuda.device(dev):
        _lib.check(lib.sage3_quant_qkv(C.byref(a), _stream_ptr(dev)), "sage3_quant_qkv")
    return out


def fp4_attention(qz: QuantizedQKV, sm_scale: Optional[float] = None, is_causal: bool = False,
                  tensor_layout: str = "HND", return_lse: bool = False, check_status: bool = False,
                  sm_margin: int = 0):
    """Attention on quantised operands (``blockscaled_fp4_attn``, ``sageattn4/api.py:231-243`` ->
    ``mha_fwd``, ``blackwell/api.cpp:258``).  ``sm_margin``: SMs to leave to kernels that run at the same time
    (see :func:`sageattn3_blackwell`)."""
    lib = _lib.load()
    B, Hq, Hkv, Nq, Nk, D = qz.shape
    dev = qz.q_codes.device
    if sm_scale is None:
        sm_scale = D ** -0.5
    if tensor_layout == "HND":
        out = torch.empty((B, Hq, Nq, D), dtype=torch.bfloat16, device=dev)
        osb, osh, osn = out.stride(0), out.stride(1), out.stride(2)
    else:
        out = torch.empty((B, Nq, Hq, D), dtype=torch.bfloat16, device=dev)
        osb, osh, osn = out.stride(0), out.stride(2), out.stride(1)
    lse = torch.empty((B, Hq, Nq), dtype=torch.float32, device=dev) if return_lse else None
    status = torch.empty(1, dtype=torch.int32, device=dev)
    a = _lib.AttnArgs()
    a.shape = _lib.Shape(B, Hq, Hkv, Nq, Nk, D)
    a.q_codes, a.q_sf = qz.q_codes.data_ptr(), qz.q_sf.data_ptr()
    a.k_codes, a.k_sf = qz.k_codes.data_ptr(), qz.k_sf.data_ptr()
    a.vt_codes, a.vt_sf = qz.vt_codes.data_ptr(), qz.vt_sf.data_ptr()
    a.delta_s = qz.delta_s.data_ptr() if qz.delta_s is not None else None
    a.delta_s_rows = qz.delta_s_rows
    a.out, a.out_stride_b, a.out_stride_h, a.out_stride_n = out.data_ptr(), osb, osh, osn
    a.lse = lse.data_ptr() if lse is not None else None
    a.sm_scale, a.is_causal = float(sm_scale), int(bool(is_causal))
    a.device_status = status.data_ptr()
    a.sm_margin = int(sm_margin)
    with torch.cuda.device(dev):
        if qz.k_lambda is not None:
            a.shape = _lib.Shape(B, Hq, Hkv, Nq, int(qz.nk_slots), D)
            _lib.check(lib.sage3_attn_fwd_packed(C.byref(a), qz.k_lambda.data_ptr(), int(qz.mean_slot_first),
                                                 _stream_ptr(dev)), "sage3_attn_fwd_packed")
        else:
            _lib.check(lib.sage3_attn_fwd(C.byref(a), _stream_ptr(dev)), "sage3_attn_fwd")
        if check_status:
            _lib.check(lib.sage3_read_device_status(status.data_ptr(), _stream_ptr(dev), None), "attention kernel")
    return (out, lse) if return_lse else out


def pack_kv(k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND", smooth_k: bool = True,
            split_first: bool = False):
    """K-packing preprocessing (``quant_pack_k`` / ``quant_pack_v`` and the K centring of
    ``sageattn4/api.py:122-177,184``): every 15 key tokens become 16 slots (FP4-rounded group mean + 15
    residuals), V gets a zero row per mean slot - or, with ``split_first`` (the reference's ``v_trick``), the
    group's first V row split into its FP4 rounding (slot 1) and the remainder (slot 0).  Returns ``(k_packed, v_packed, k_lambda, km)`` with the
    packed tensors in HND ``[B,Hkv,16*ceil(Nk/15),D]`` and ``k_lambda`` fp32 padded to a multiple of 128."""
    lib = _lib.load()
    _check_device(k)
    B, Hkv, Nk, D, ksb, ksh, ksn = _as_bhnd_strides(k, tensor_layout)
    Bv, Hv, Nv, Dv, vsb, vsh, vsn = _as_bhnd_strides(v, tensor_layout)
    if (B, Hkv, Nk, D) != (Bv, Hv, Nv, Dv):
        raise ValueError("k and v shapes do not match")
    dev = k.device
    rows = lib.sage3_packed_rows(Nk)
    kp = torch.empty((B, Hkv, rows, D), dtype=torch.bfloat16, device=dev)
    vp = torch.empty((B, Hkv, rows, D), dtype=torch.bfloat16, device=dev)
    lam = torch.empty((B, Hkv, (rows + 127) // 128 * 128), dtype=torch.float32, device=dev)
    km = torch.empty((B, Hkv, D), dtype=torch.bfloat16, device=dev) if smooth_k else None
    z = buffer_sizes(B, Hkv, Hkv, Nk, Nk, D, 1)
    scratch = torch.empty(max(int(z.scratch), 256), dtype=torch.uint8, device=dev)
    a = _lib.PackArgs()
    a.shape = _lib.Shape(B, Hkv, Hkv, Nk, Nk, D)
    a.k, a.v = _tensor_arg(k, ksb, ksh, ksn), _tensor_arg(v, vsb, vsh, vsn)
    a.smooth_k = int(smooth_k)
    a.km = km.data_ptr() if km is not None else None
    a.k_packed, a.v_packed, a.k_lambda = kp.data_ptr(), vp.data_ptr(), lam.data_ptr()
    a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    a.split_first = int(bool(split_first))
    with torch.cuda.device(dev):
        _lib.check(lib.sage3_pack_kv(C.byref(a), _stream_ptr(dev)), "sage3_pack_kv")
    return kp, vp, lam, km


def sageattn4_blackwell(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                        is_causal: bool = False, sm_scale: Optional[float] = None, per_block_mean: bool = True,
                        quant_block: int = 16, v_trick: Optional[bool] = None, attn_mask=None,
                        check_status: bool = False, **kwargs):
    """The fork's K-packing operator (``sageattn4_blackwell``, ``sageattn4/api.py:250-288``): K is centred,
    packed 15 -> 16 (group mean + residuals) and the kernel restores every score as
    ``q.residual + lambda * q.mean``.  ``per_block_mean`` selects the kernel variant as in the reference
    (``fwd_mainloop.cu:878-888``): True = per-128-token Q mean, the mean slot is masked out; False =
    whole-sequence Q mean, the mean slot takes the first token's score.  ``v_trick`` (default
    ``not per_block_mean``, ``api.py:180-181``) selects the split-first V layout.  ``quant_block`` must be 16."""
    lib = _lib.load()
    if attn_mask is not None:
        raise NotImplementedError("attn_mask is not supported (the reference ignores it, api.py:250)")
    if quant_block != 16:
        raise AssertionError("quant_block must be 16")                                   # api.py:251
    if q.shape[-1] not in (64, 128):
        raise ValueError(f"Unsupported Headdim {q.shape[-1]}")
    if v_trick is None:
        v_trick = not per_block_mean
    kp, vp, lam, _ = pack_kv(k, v, tensor_layout, smooth_k=True, split_first=bool(v_trick))
    if tensor_layout == "NHD":
        kp, vp = kp.transpose(1, 2), vp.transpose(1, 2)          # views; the quantiser takes strides
    qz = quantize_qkv(q, kp, vp, tensor_layout, per_block_mean=bool(per_block_mean), smooth_k=False)
    qz.k_lambda = lam
    qz.mean_slot_first = not per_block_mean
    Nk = k.shape[2] if tensor_layout == "HND" else k.shape[1]
    qz.nk_slots = lib.sage3_packed_len(Nk)
    return fp4_attention(qz, sm_scale=sm_scale, is_causal=is_causal, tensor_layout=tensor_layout,
                         check_status=check_status)


def sageattn3_blackwell(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                        is_causal: bool = False, sm_scale: Optional[float] = None, per_block_mean: bool = True,
                        return_lse: bool = False, smooth_k: bool = True, attn_mask=None,
                        check_status: bool = False, sm_margin: int = 0, **kwargs):
    """FP4 attention, drop-in for ``sageattn4_blackwell`` (``sageattn4/api.py:250-288``) with the wider
    argument set of ``sageattn`` (``sageattention/core.py:79-88``).

    q ``[B,Hq,Nq,D]`` ("HND") or ``[B,Nq,Hq,D]`` ("NHD"), k/v likewise with ``Hkv`` heads
    (``Hq % Hkv == 0``), bf16, D <= 128 (head dims other than 64 and 128 are zero-padded to the next of the two,
    ``sageattention/core.py:925-937``).  Returns a tensor shaped like q (and the natural-log LSE ``[B,Hq,Nq]`` of
    ``sm_scale * q.k`` when ``return_lse``; ``-inf`` for rows that see no key).  Causal masking is bottom-right
    aligned when Nq != Nk.

    ``sm_margin`` (no counterpart in the reference): the attention kernel is persistent with one CTA per SM and a
    static work list, so a CTA whose SM is held by another kernel - a collective running beside it on another
    stream - starts late and the whole launch ends late.  With ``sm_margin = m`` it launches on ``SMs - m`` SMs
    only; the result is the same bit for bit.
    """
    if attn_mask is not None:
        raise NotImplementedError("attn_mask is not supported (the reference ignores it as well)")
    lib = _lib.load()
    _check_device(q)
    for t in (q, k, v):
        if t.dtype != torch.bfloat16:
            raise AssertionError("TODO: support inputs other than bfloat16")     # api.py:257
    B, Hq, Nq, D, qsb, qsh, qsn = _as_bhnd_strides(q, tensor_layout)
    Bk, Hkv, Nk, Dk, ksb, ksh, ksn = _as_bhnd_strides(k, tensor_layout)
    Bv, Hv, Nv, Dv, vsb, vsh, vsn = _as_bhnd_strides(v, tensor_layout)
    if not (B == Bk == Bv and D == Dk == Dv and Hkv == Hv and Nk == Nv):
        raise ValueError("q, k, v shapes do not match")
    if Hq % Hkv != 0:
        raise ValueError("num_qo_heads must be a multiple of num_kv_heads")
    # head-dim padding of sageattention/core.py:925-937: below 64 -> 64, between 64 and 128 -> 128, zeros in the
    # extra channels, default scale from the original head dim, output cut back (:990).  The kernels read rows of the
    # original width and take the rest as zero, so nothing is copied - if the width is a multiple of 8 (16-byte
    # loads); other widths are padded here first, as the reference does.
    d_og = D
    if D > 128:
        raise ValueError(f"Unsupported head_dim: {D}")                            # core.py:937
    if D not in (64, 128) and D % 8 != 0:
        pad = (64 if D < 64 else 128) - D
        if sm_scale is None:
            sm_scale = D ** -0.5
        q, k, v = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
        res = sageattn3_blackwell(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale,
                                  per_block_mean=per_block_mean, return_lse=return_lse, smooth_k=smooth_k,
                                  check_status=check_status, sm_margin=sm_margin)
        return (res[0][..., :d_og].contiguous(), res[1]) if return_lse else res[..., :d_og].contiguous()
    if D not in (64, 128):
        D = 64 if D < 64 else 128
    dev = q.device
    pbm = int(bool(per_block_mean))
    z = buffer_sizes(B, Hq, Hkv, Nq, Nk, D, pbm)
    out = torch.empty_like(q)
    _, _, _, _, osb, osh, osn = _as_bhnd_strides(out, tensor_layout)
    ws = torch.empty(int(z.workspace), dtype=torch.uint8, device=dev)
    lse = torch.empty((B, Hq, Nq), dtype=torch.float32, device=dev) if return_lse else None
    status = torch.empty(1, dtype=torch.int32, device=dev)
    a = _lib.FwdArgs()
    a.shape = _lib.Shape(B, Hq, Hkv, Nq, Nk, D)
    a.q, a.k, a.v = _tensor_arg(q, qsb, qsh, qsn), _tensor_arg(k, ksb, ksh, ksn), _tensor_arg(v, vsb, vsh, vsn)
    a.out, a.out_stride_b, a.out_stride_h, a.out_stride_n = out.data_ptr(), osb, osh, osn
    a.lse = lse.data_ptr() if lse is not None else None
    a.km_out = None           # the K-mean term of the LSE is put back on the device (q . km in the quantisation kernel)
    a.sm_scale = float(sm_scale) if sm_scale is not None else 0.0
    a.is_causal, a.per_block_mean, a.smooth_k = int(bool(is_causal)), pbm, int(bool(smooth_k))
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.device_status = status.data_ptr()
    a.head_dim = d_og if d_og != D else 0
    a.sm_margin = int(sm_margin)
    with torch.cuda.device(dev):
        _lib.check(lib.sage3_attention(C.byref(a), _stream_ptr(dev)), "sage3_attention")
        if check_status:
            _lib.check(lib.sage3_read_device_status(status.data_ptr(), _stream_ptr(dev), None), "attention kernel")
    return (out, lse) if return_lse else out


def sageattn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND", is_causal: bool = False,
             sm_scale: Optional[float] = None, return_lse: bool = False, **kwargs):
    """Automatic entry point (``sageattention/core.py:79-157``).  The reference picks a kernel family
    by GPU architecture and raises ``ValueError`` for architectures it has no kernel for; this build
    has exactly one family, the FP4 kernels for compute capability 10.x."""
    _check_device(q)
    return sageattn3_blackwell(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal, sm_scale=sm_scale,
                               return_lse=return_lse, **kwargs)


def sageattn_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                    cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, is_causal: bool = False,
                    sm_scale: Optional[float] = None, smooth_k: bool = True, check_status: bool = False,
                    **kwargs) -> torch.Tensor:
    """Variable-length batch (``sageattention/core.py:334-448``): q ``[sum(len_q), Hq, D]``, k/v
    ``[sum(len_k), Hkv, D]``, ``cu_seqlens_*`` the int32 prefix sums (length batch + 1, on the device).
    One pass over the four kernels for the whole batch (``sage3_attention_varlen``); every sequence is
    smoothed, quantised and attended on its own (K means never mix sequences); sequences without keys give
    zeros.  ``max_seqlen_*`` must bound the longest sequence - they size the workspace."""
    lib = _lib.load()
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("varlen tensors must be [tokens, heads, head_dim]")
    _check_device(q)
    for t in (q, k, v):
        if t.dtype != torch.bfloat16:
            raise AssertionError("TODO: support inputs other than bfloat16")
        if t.stride(-1) != 1:
            raise ValueError("the head dimension must be contiguous")
    nseq = cu_seqlens_q.numel() - 1
    if cu_seqlens_k.numel() != nseq + 1 or nseq < 1:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must both have batch + 1 entries")
    if max_seqlen_q <= 0 or max_seqlen_k <= 0:
        raise ValueError("max_seqlen_q and max_seqlen_k must be positive")
    dev = q.device
    cq = cu_seqlens_q.to(device=dev, dtype=torch.int32).contiguous()
    ck = cu_seqlens_k.to(device=dev, dtype=torch.int32).contiguous()
    Hq, D = q.shape[1], q.shape[2]
    Hkv = k.shape[1]
    if Hq % Hkv != 0 or v.shape != k.shape or k.shape[2] != D:
        raise ValueError("q, k, v shapes do not match")
    out = torch.empty_like(q)
    z = buffer_sizes(nseq, Hq, Hkv, int(max_seqlen_q), int(max_seqlen_k), D, 1)
    ws = torch.empty(int(z.workspace), dtype=torch.uint8, device=dev)
    status = torch.empty(1, dtype=torch.int32, device=dev)
    a = _lib.VarlenArgs()
    a.shape = _lib.Shape(nseq, Hq, Hkv, int(max_seqlen_q), int(max_seqlen_k), D)
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.q_stride_n, a.q_stride_h = q.stride(0), q.stride(1)
    a.k_stride_n, a.k_stride_h = k.stride(0), k.stride(1)
    a.v_stride_n, a.v_stride_h = v.stride(0), v.stride(1)
    a.cu_seqlens_q, a.cu_seqlens_k = cq.data_ptr(), ck.data_ptr()
    a.out, a.out_stride_n, a.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    a.sm_scale = float(sm_scale) if sm_scale is not None else 0.0
    a.is_causal, a.smooth_k = int(bool(is_causal)), int(bool(smooth_k))
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.device_status = status.data_ptr()
    with torch.cuda.device(dev):
        _lib.check(lib.sage3_attention_varlen(C.byref(a), _stream_ptr(dev)), "sage3_attention_varlen")
        if check_status:
            _lib.check(lib.sage3_read_device_status(status.data_ptr(), _stream_ptr(dev), None), "attention kernel")
    return out


_host_streams = {}


def sageattn_from_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                       device=None, head_chunks=8, is_causal: bool = False, sm_scale: Optional[float] = None,
                       **kwargs) -> torch.Tensor:
    """Attention on HOST tensors (HND ``[B,H,N,D]`` bf16, ideally pinned): the heads are processed in
    ``head_chunks`` groups of kv heads (a number, or an explicit list of kv heads per group), and the host-to-device copy of group ``i+1`` and the
    device-to-host copy of group ``i-1`` run on their own streams while group ``i`` is computed (groups
    alternate between two compute streams so that their kernels overlap at the seams), so the
    PCIe transfers hide behind the kernels (or the other way round).  Returns the output as a host tensor
    (``out`` if given, else a new pinned tensor).  The work is ordered after the caller's current stream
    and the current stream waits for the last copy, so CUDA events recorded around the call time all of it;
    the host must still synchronise before reading ``out``."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("sageattn_from_host takes host tensors; use sageattn for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, Hq, Nq, D = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv != 0:
        raise ValueError("num_qo_heads must be a multiple of num_kv_heads")
    g = Hq // Hkv
    if out is None:
        out = torch.empty_like(q).pin_memory()
    # group sizes: about Hkv / head_chunks heads, but ramping up from one head at the start and down to one at
    # the end, so that the first kernel starts after a small copy and little is left to copy out after the last.
    # A group should also carry enough bytes (about 96 MB of q, k, v) for its copy to be worth a pipeline stage:
    # every group costs a few host-side calls, which small problems cannot hide.
    if isinstance(head_chunks, (list, tuple)):
        sizes = [int(n) for n in head_chunks]                    # explicit group sizes (kv heads per group)
        if sum(sizes) != Hkv or min(sizes) < 1:
            raise ValueError(f"head_chunks {sizes} must be positive and add up to the {Hkv} kv heads")
    else:
        in_bytes = (q.numel() + k.numel() + v.numel()) * q.element_size()
        head_chunks = max(1, min(head_chunks, int(in_bytes // (96 << 20)) or 1))
        base = max(1, Hkv // max(1, min(head_chunks, Hkv)))
        ramp = [n for n in (1, 2, 4) if n < base] if head_chunks > 1 else []
        sizes = list(ramp)
        left = Hkv - sum(ramp)
        tail = [n for n in reversed(ramp) if n <= left - base]      # keep at least one full group in the middle
        left -= sum(tail)
        while left > 0:
            sizes.append(min(base, left))
            left -= sizes[-1]
        sizes += tail
    bounds = [0]
    for n in sizes:
        bounds.append(bounds[-1] + n)
    assert bounds[-1] == Hkv
    chunks = len(sizes)
    if dev not in _host_streams:
        _host_streams[dev] = tuple(torch.cuda.Stream(dev) for _ in range(4))
    s_in, s_run_a, s_run_b, s_out = _host_streams[dev]
    cur = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(cur)
    for st in (s_in, s_run_a, s_run_b, s_out):
        st.wait_event(start)
    keep = []
    for c in range(chunks):
        h0, h1 = bounds[c], bounds[c + 1]
        if h0 == h1:
            continue
        with torch.cuda.stream(s_in):
            # one copy per batch entry: q[b, h0:h1] is one contiguous block of a [B,H,N,D] tensor, q[:, h0:h1] is not
            # (for B > 1 a strided host-to-device copy falls back to a slow path)
            qd = torch.empty((B, (h1 - h0) * g, Nq, D), dtype=q.dtype, device=dev)
            kd = torch.empty((B, h1 - h0) + tuple(k.shape[2:]), dtype=k.dtype, device=dev)
            vd = torch.empty_like(kd)
            for b in range(B):
                qd[b].copy_(q[b, h0 * g:h1 * g], non_blocking=True)
                kd[b].copy_(k[b, h0:h1], non_blocking=True)
                vd[b].copy_(v[b, h0:h1], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        # groups alternate between two compute streams: the attention kernel is persistent (one CTA per SM), so
        # the kernels of the next group fill the SMs that the last, partly filled round of this group leaves idle
        s_run = s_run_a if c % 2 == 0 else s_run_b
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in)
            od = sageattn3_blackwell(qd, kd, vd, tensor_layout="HND", is_causal=is_causal, sm_scale=sm_scale, **kwargs)
            ev_run = torch.cuda.Event()
            ev_run.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run)
            for b in range(B):
                out[b, h0 * g:h1 * g].copy_(od[b], non_blocking=True)
        keep.append((qd, kd, vd, od))
    done = torch.cuda.Event()
    done.record(s_out)
    cur.wait_event(done)
    for st in (s_run_a, s_run_b):                 # nothing of this call may outlive the caller's next operation
        ev = torch.cuda.Event()
        ev.record(st)
        cur.wait_event(ev)
    # the device buffers were allocated on side streams: tell the allocator the current stream orders their reuse
    for tensors in keep:
        for t in tensors:
            t.record_stream(cur)
    return out
