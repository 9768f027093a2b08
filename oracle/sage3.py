"""CPU restatement (PyTorch, fp32) of the reference's SageAttention3 FP4 attention pipeline.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; never by the product.

Parity status: the quantiser part is pinned (see ``oracle/nvfp4.py``).  The attention part
restates a kernel that exists only for sm_120a/sm_121a (the reference host code refuses other
GPUs, ``blackwell/api.cpp:276-279``) and the reference ships no expected outputs for it, so for
the attention output this oracle is **parity unpinned**: it follows the reference source line
by line but cannot be checked against a run of the reference kernel on this hardware.

Reference paths (inside ``sageattention3_blackwell/``):

* the K-packing steps ``quant_pack_k`` / ``quant_pack_v`` (api.py:122-177, :193-194) of the fork's
  SageAttention4 extension are restated separately (``pack_k``, ``pack_v``, ``sageattn4_emulated``;
  the packing is pinned by golden vectors made with the reference's own ``preprocess_qkv``).
* preprocessing ``sageattn4/api.py:179-205`` without those packing steps: K minus its
  per-channel mean over tokens (:184), Q padded to 128 and minus its per-128-token mean
  (:26-72, :186-191), ``delta_s = qm @ k^T`` in bf16 then widened to fp32 (:201), zero padding
  of K and V to a multiple of 128 (:196-203).
* kernel arithmetic ``sageattn4/blackwell/softmax_fused.h:39-187`` and
  ``sageattn4/blackwell/fwd_mainloop.cu:766-794`` (scores start from delta_s), ``:921-964``
  (masks), ``:967-1014`` (P scale / code conversion), ``:1079-1121`` (K tiles visited from the
  last to the first, fresh PV accumulator per tile, ``O = O * alpha + O_tile``).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import nvfp4

BLOCK = 128
LOG2E = 1.4426950408889634
# softmax_fused.h:32-34
LOG2_INV_2688 = -11.392317422778762   # log2(1 / (448 * 6))
LOG2_INV_6 = -2.584962500721156       # log2(1 / 6)


# ---------------------------------------------------------------------------------------------
# preprocessing
# ---------------------------------------------------------------------------------------------

def pad_tokens(x: torch.Tensor, mult: int = BLOCK) -> torch.Tensor:
    """Zero-pad dim -2 to a multiple of ``mult`` (api.py:116-121)."""
    n = x.shape[-2]
    pad = (-n) % mult
    if pad == 0:
        return x.contiguous()
    return torch.nn.functional.pad(x, (0, 0, 0, pad)).contiguous()


def smooth_k(k: torch.Tensor):
    """api.py:184.  Returns (k - mean, mean) both in k's dtype; mean over the true length."""
    km = k.mean(dim=-2, keepdim=True)
    return k - km, km


def q_block_mean(q_pad: torch.Tensor):
    """api.py:26-72: per 128 tokens, fp32 mean (padding rows included), ``q - mean`` rounded to
    q's dtype, mean rounded to q's dtype."""
    B, H, L, D = q_pad.shape
    g = q_pad.float().reshape(B, H, L // BLOCK, BLOCK, D)
    mean = g.sum(dim=-2) / BLOCK
    q_out = (g - mean.unsqueeze(-2)).to(q_pad.dtype).reshape(B, H, L, D)
    return q_out, mean.to(q_pad.dtype)


def preprocess(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, per_block_mean: bool = True):
    """HND bf16 tensors -> (q_s, k_s, v_pad, delta_s, km) exactly as api.py:179-205 minus packing.
    Also returns the K mean (needed for the LSE correction of sageattention/core.py:993-994)."""
    k_s, km = smooth_k(k)
    q_pad = pad_tokens(q)
    if per_block_mean:
        q_s, qm = q_block_mean(q_pad)
    else:
        qm = q_pad.mean(dim=-2, keepdim=True)
        q_s = q_pad - qm
    k_s = pad_tokens(k_s)
    delta_s = torch.matmul(qm, k_s.transpose(-2, -1)).to(torch.float32).contiguous()
    return q_s, k_s, pad_tokens(v), delta_s, km


# ---------------------------------------------------------------------------------------------
# quantiser wrappers (torch <-> numpy)
# ---------------------------------------------------------------------------------------------

def quant_rows(x: torch.Tensor, mode: str = "exact"):
    """Quantise along the last dim; returns (codes u8 [..., D/2], sf u8 [..., D/16])."""
    codes, sf = nvfp4.quantize_nvfp4(x.float().numpy(), mode)
    return torch.from_numpy(codes), torch.from_numpy(sf)


def quant_v_transposed(v_pad: torch.Tensor, mode: str = "exact"):
    """fp4_quantization_4d.cu:286-412: V [B,H,N,D] -> codes [B,H,D,N/2], sf [B,H,D,N/16],
    scale blocks run over 16 consecutive tokens."""
    return quant_rows(v_pad.transpose(-1, -2).contiguous(), mode)


def dequant(codes: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    return torch.from_numpy(nvfp4.dequantize_nvfp4(codes.numpy(), sf.numpy()))


def _e4m3_round(x: torch.Tensor) -> torch.Tensor:
    return torch.from_numpy(nvfp4.e4m3_decode(nvfp4.e4m3_encode(x.numpy())))


def _e2m1_round(x: torch.Tensor) -> torch.Tensor:
    return torch.from_numpy(nvfp4.e2m1_decode(nvfp4.e2m1_encode(x.numpy())))


# ---------------------------------------------------------------------------------------------
# attention on quantised operands (kernel arithmetic)
# ---------------------------------------------------------------------------------------------

def attention_quantised(qd: torch.Tensor, kd: torch.Tensor, vtd: torch.Tensor, delta_s: torch.Tensor,
                        len_q: int, len_k: int, sm_scale: float, causal: bool = False,
                        return_lse: bool = False, lamb: torch.Tensor | None = None,
                        q_tiles=None, mean_slot: str = "mask"):
    """Flash-style forward on de-quantised operands with the reference's P re-quantisation.

    qd  [B,Hq,Nq_pad,D]  fp32 = dequantised Q codes
    kd  [B,Hk,Nk_pad,D]  fp32 = dequantised K codes
    vtd [B,Hk,D,Nk_pad]  fp32 = dequantised V^T codes
    delta_s [B,Hq,Nq_pad/128,Nk_pad] fp32 (or None)
    lamb [B,Hk,Nk_pad] fp32 (or None): K-packing mode (fwd_mainloop.cu:796-891).  Keys then come in
    groups of 16 = one mean slot + 15 residual tokens, ``len_k`` is the PACKED length, every score
    gets ``lamb * (score of its group's mean slot)`` added before masking, the causal mask works on the
    logical token of each packed key (:273-281, :921-934) and the mean slot itself is masked out
    (:878-881, per-block-mean variant).
    mean_slot (K-packing mode only): "mask" = the per-block-mean kernels, the slot is masked out;
    "first" = the other kernel variant (:882-888): the slot takes the (masked) score of the group's first token
    where ``can_use_mean_slot`` (:855-871) allows, its probability multiplies the slot's V row (the first
    token's FP4 remainder under ``v_trick``) but is left out of the row sum (softmax_fused.h:48-64).
    q_tiles (or None): qd holds only these 128-row query tiles of a longer sequence of ``len_q``
    tokens (tile i of qd is query tile ``q_tiles[i]``; delta_s has the same rows); all rows of the
    given tiles are returned, the caller drops those beyond ``len_q``.  Lets a test check a few query
    tiles of a benchmark-sized problem against all of its keys.
    Returns O [B,Hq,len_q,D] fp32 (callers round to bf16) and optionally the log-sum-exp
    (natural log, of the smoothed scores) [B,Hq,len_q].
    """
    B, Hq, Nq, D = qd.shape
    Hk, Nk = kd.shape[1], kd.shape[2]
    g = Hq // Hk
    if g > 1:
        kd = kd.repeat_interleave(g, dim=1)
        vtd = vtd.repeat_interleave(g, dim=1)
        if lamb is not None:
            lamb = lamb.repeat_interleave(g, dim=1)
    len_k_logical = packed_len_to_logical(len_k) if lamb is not None else len_k
    nqb, nkb = Nq // BLOCK, Nk // BLOCK
    c = sm_scale * LOG2E
    q4 = qd.reshape(B, Hq, nqb, BLOCK, D)
    O = torch.zeros(B, Hq, nqb, BLOCK, D)
    m = torch.full((B, Hq, nqb, BLOCK), -math.inf)
    l = torch.zeros(B, Hq, nqb, BLOCK)
    qpos = torch.arange(Nq).reshape(nqb, BLOCK)
    if q_tiles is not None:
        qpos = torch.as_tensor(list(q_tiles)).reshape(nqb, 1) * BLOCK + torch.arange(BLOCK).reshape(1, BLOCK)
    for j in range(nkb - 1, -1, -1):                       # fwd_mainloop.cu:575,1080 (last tile first)
        ks = kd[:, :, j * BLOCK:(j + 1) * BLOCK]           # [B,H,128,D]
        S = torch.einsum("bhqrd,bhkd->bhqrk", q4, ks)
        if delta_s is not None:
            S = S + delta_s[:, :, :, None, j * BLOCK:(j + 1) * BLOCK]
        kpos = torch.arange(j * BLOCK, (j + 1) * BLOCK)
        ktok = kpos
        if lamb is not None:                               # correct_lamb_k, fwd_mainloop.cu:796-845
            S16 = S.reshape(B, Hq, nqb, BLOCK, BLOCK // 16, 16)
            lam16 = lamb[:, :, j * BLOCK:(j + 1) * BLOCK].reshape(B, Hq, 1, 1, BLOCK // 16, 16)
            S = (S16 + lam16 * S16[..., :1]).reshape(B, Hq, nqb, BLOCK, BLOCK)
            lane = kpos % 16
            ktok = (kpos // 16) * 15 + torch.where(lane == 0, lane, lane - 1)   # :273-281
        mask = (kpos >= len_k)[None, None, :].expand(nqb, BLOCK, BLOCK)
        if causal:                                         # fwd_mainloop.cu:926
            mask = mask | (ktok[None, None, :] >= (qpos[:, :, None] + 1 + len_k_logical - len_q))
        is_slot = (kpos % 16 == 0)
        if lamb is not None and mean_slot == "mask":       # the mean slot carries no token (:878-881)
            mask = mask | is_slot[None, None, :]
        if causal and bool(mask.all()):
            continue                                       # tile never visited (get_n_block_max :305-324)
        S = S.masked_fill(mask, -math.inf)
        if lamb is not None and mean_slot == "first":      # set_mean_slot_to_first_score, :847-891
            first = S.reshape(B, Hq, nqb, BLOCK, BLOCK // 16, 16)[..., 1]
            usable = torch.ones(nqb, BLOCK, BLOCK // 16, dtype=torch.bool)
            if causal:
                qk = qpos + len_k_logical - len_q                              # query_key_pos
                col = kpos[0::16]                                              # the slots' packed positions
                usable = (col[None, None, :] < len_k) & (qk[:, :, None] >= 0) & \
                         ((col[None, None, :] // 16) < (qk[:, :, None].clamp(min=0) // 15))
            slot_val = torch.where(usable[None, None], first, torch.full_like(first, -math.inf))
            S = S.clone().reshape(B, Hq, nqb, BLOCK, BLOCK // 16, 16)
            S[..., 0] = slot_val
            S = S.reshape(B, Hq, nqb, BLOCK, BLOCK)
        bm = S.reshape(B, Hq, nqb, BLOCK, BLOCK // 16, 16).amax(dim=-1)       # softmax_fused.h:113-121
        m_new = torch.maximum(m, bm.amax(dim=-1))
        m_fin = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        alpha = torch.exp2((m - m_fin) * c)                                   # :130 (0 on the first tile)
        max_scaled = m_fin * c + LOG2_INV_2688
        P = torch.exp2(S * c - max_scaled[..., None])                         # :138  in (0, 2688]
        if lamb is not None and mean_slot == "first":                         # the slot is not a token: no row-sum share
            l = l * alpha + P.masked_fill(is_slot[None, None, None, None, :], 0.0).sum(dim=-1)
        else:
            l = l * alpha + P.sum(dim=-1)                                     # :135,139 (unquantised P)
        sb = torch.exp2(bm * c - max_scaled[..., None] + LOG2_INV_6)          # :142-144
        P6 = P.reshape(B, Hq, nqb, BLOCK, BLOCK // 16, 16)
        Pn = torch.where(sb[..., None] > 0, P6 / sb[..., None], torch.zeros_like(P6))  # :148-153
        Pq = _e2m1_round(Pn) * _e4m3_round(sb)[..., None]                     # fwd_mainloop.cu:967-1002
        Pq = Pq.reshape(B, Hq, nqb, BLOCK, BLOCK)
        vt = vtd[:, :, :, j * BLOCK:(j + 1) * BLOCK]                           # [B,H,D,128]
        O = O * alpha[..., None] + torch.einsum("bhqrk,bhdk->bhqrd", Pq, vt)  # softmax_fused.h:183
        m = m_new
    inv = torch.where((l == 0) | torch.isnan(l), torch.zeros_like(l), 1.0 / l)  # :167
    keep = Nq if q_tiles is not None else len_q
    out = (O * inv[..., None]).reshape(B, Hq, Nq, D)[:, :, :keep]
    if not return_lse:
        return out
    lse = (m * sm_scale + torch.log(l / 2688.0)).reshape(B, Hq, Nq)[:, :, :keep]
    return out, lse


def sageattn3_emulated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
                       sm_scale: float | None = None, per_block_mean: bool = True,
                       mode: str = "exact", return_lse: bool = False, smooth: bool = True):
    """Whole pipeline on HND bf16 CPU tensors (GQA allowed: Hq multiple of Hk)."""
    D = q.shape[-1]
    Lq, Lk = q.shape[-2], k.shape[-2]
    if sm_scale is None:
        sm_scale = D ** -0.5
    g = q.shape[1] // k.shape[1]
    k_s, km = smooth_k(k) if smooth else (k, torch.zeros_like(k[..., :1, :]))
    q_pad = pad_tokens(q)
    if per_block_mean:
        q_s, qm = q_block_mean(q_pad)
    else:
        qm = q_pad.mean(dim=-2, keepdim=True)
        q_s = q_pad - qm
    k_s = pad_tokens(k_s)
    k_rep = k_s.repeat_interleave(g, dim=1) if g > 1 else k_s
    delta_s = torch.matmul(qm, k_rep.transpose(-2, -1)).to(torch.float32)
    if not per_block_mean:
        delta_s = delta_s.expand(-1, -1, q_pad.shape[-2] // BLOCK, -1)
    qd = dequant(*quant_rows(q_s, mode))
    kd = dequant(*quant_rows(k_s, mode))
    vtd = dequant(*quant_v_transposed(pad_tokens(v), mode))
    res = attention_quantised(qd, kd, vtd, delta_s, Lq, Lk, sm_scale, is_causal, return_lse)
    if return_lse:
        out, lse = res
        # K smoothing shifts every score of a row by -sm_scale * q.km (core.py:993-994 pattern)
        km_rep = km.repeat_interleave(g, dim=1) if g > 1 else km
        lse = lse + sm_scale * torch.matmul(q.float(), km_rep.float().transpose(-2, -1)).squeeze(-1)
        return out.to(q.dtype), lse
    return res.to(q.dtype)


# ---------------------------------------------------------------------------------------------
# K-packing mode of the fork (SageAttention4): api.py:122-177, 193-203, 267-274
# ---------------------------------------------------------------------------------------------

def logical_to_packed_len(n: int) -> int:
    """api.py:270-274 / fwd_mainloop.cu:294-303: 15 tokens take 16 slots, a partial group one more."""
    return (n // 15) * 16 + (0 if n % 15 == 0 else 1 + n % 15)


def packed_len_to_logical(n: int) -> int:
    """fwd_mainloop.cu:283-292."""
    return (n // 16) * 15 + (0 if n % 16 == 0 else n % 16 - 1)


def pack_k(k_s: torch.Tensor):
    """api.py:122-149 (quant_block_size 16).  k_s: smoothed K [B,H,N,D] bf16.  Per group of 15 tokens
    (the last one zero-padded): slot 0 = the FP4-rounded group mean, slots 1..15 = k - lambda * mean
    with lambda = <k, mean> / |mean|^2.  Returns (packed [B,H,16*G,D] in k's dtype, lambda fp32
    [B,H,16*G], 0 in the mean slots)."""
    B, H, _, D = k_s.shape
    x = pad_tokens(k_s, 15)
    G = x.shape[-2] // 15
    xb = x.reshape(B, H, G, 15, D)
    mean = xb.mean(dim=-2)                                                    # bf16 result, fp32 accumulate
    mean = torch.from_numpy(nvfp4.fake_quant(mean.float().numpy())).to(k_s.dtype)   # round_to_blockscaled_fp4
    mf = mean.float()
    nsq = (mf * mf).sum(dim=-1, keepdim=True)
    direction = torch.where(nsq > 0, mf / nsq, torch.zeros_like(mf))
    lamb = torch.einsum("bhnmd,bhnd->bhnm", xb.float(), direction)
    res = (xb.float() - lamb.unsqueeze(-1) * mf.unsqueeze(-2)).to(k_s.dtype)
    lamb = torch.cat([torch.zeros(B, H, G, 1), lamb.float()], dim=-1)
    packed = torch.cat([mean.unsqueeze(-2), res], dim=-2)
    return packed.reshape(B, H, G * 16, D), lamb.reshape(B, H, G * 16)


def pack_v(v: torch.Tensor, split_first: bool = False):
    """api.py:150-177.  ``split_first=False``: a zero row in every mean slot.  ``split_first=True`` (the
    ``v_trick``): the group's first token is stored twice over - slot 1 holds its value as the V^T quantiser will
    round it (FP4 along tokens, with the slot still zero), slot 0 the remainder - so that a kernel which gives slot 0
    the first token's probability recovers that token's V to two FP4 terms."""
    B, H, _, D = v.shape
    x = pad_tokens(v, 15)
    G = x.shape[-2] // 15
    xb = x.reshape(B, H, G, 15, D)
    zero = torch.zeros(B, H, G, 1, D, dtype=v.dtype)
    if not split_first:
        return torch.cat([zero, xb], dim=-2).reshape(B, H, G * 16, D)
    base = pad_tokens(torch.cat([zero, xb], dim=-2).reshape(B, H, G * 16, D))
    rounded = torch.from_numpy(nvfp4.fake_quant(base.float().transpose(-1, -2).contiguous().numpy()))
    rounded = rounded.transpose(-1, -2)[:, :, :G * 16].to(v.dtype).reshape(B, H, G, 16, D)
    hi = rounded[:, :, :, 1]
    slot = (xb[:, :, :, 0].float() - hi.float()).to(v.dtype)
    split = xb.clone()
    split[:, :, :, 0] = hi
    return torch.cat([slot.unsqueeze(-2), split], dim=-2).reshape(B, H, G * 16, D)


def sageattn4_emulated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
                       sm_scale: float | None = None, mode: str = "exact", per_block_mean: bool = True,
                       v_trick: bool | None = None):
    """The fork's K-packing pipeline (api.py:179-205, 250-288) on HND bf16 CPU tensors.  ``per_block_mean`` selects
    the kernel variant (per-128-token Q mean and a masked mean slot, or whole-sequence Q mean and a mean slot that
    takes the first token's score); ``v_trick`` (default ``not per_block_mean``, api.py:180-181) the V layout."""
    D = q.shape[-1]
    Lq, Lk = q.shape[-2], k.shape[-2]
    if sm_scale is None:
        sm_scale = D ** -0.5
    if v_trick is None:
        v_trick = not per_block_mean
    g = q.shape[1] // k.shape[1]
    k_s, _ = smooth_k(k)
    q_pad = pad_tokens(q)
    if per_block_mean:
        q_s, qm = q_block_mean(q_pad)
    else:
        qm = q_pad.mean(dim=-2, keepdim=True)
        q_s = q_pad - qm
    k_p, lamb = pack_k(k_s)
    v_p = pack_v(v, split_first=v_trick)
    k_p = pad_tokens(k_p)
    lamb = pad_tokens(lamb.unsqueeze(-1)).squeeze(-1)
    k_rep = k_p.repeat_interleave(g, dim=1) if g > 1 else k_p
    delta_s = torch.matmul(qm, k_rep.transpose(-2, -1)).to(torch.float32)     # from the unrounded packed K
    if not per_block_mean:
        delta_s = delta_s.expand(-1, -1, q_pad.shape[-2] // BLOCK, -1)
    qd = dequant(*quant_rows(q_s, mode))
    kd = dequant(*quant_rows(k_p, mode))
    vtd = dequant(*quant_v_transposed(pad_tokens(v_p), mode))
    out = attention_quantised(qd, kd, vtd, delta_s, Lq, logical_to_packed_len(Lk), sm_scale, is_causal, lamb=lamb,
                              mean_slot="mask" if per_block_mean else "first")
    return out.to(q.dtype)


def sdpa_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
              sm_scale: float | None = None) -> torch.Tensor:
    """Plain fp32 attention with the reference's bottom-right causal alignment
    (scripts/compare_k_smoothing_cosim.py:250-263)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    g = qf.shape[1] // kf.shape[1]
    if g > 1:
        kf = kf.repeat_interleave(g, dim=1)
        vf = vf.repeat_interleave(g, dim=1)
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    s = torch.matmul(qf, kf.transpose(-2, -1)) * sm_scale
    if is_causal:
        Lq, Lk = q.shape[-2], k.shape[-2]
        keep = torch.ones(Lq, Lk, dtype=torch.bool).tril(diagonal=Lk - Lq)
        s = s.masked_fill(~keep, -math.inf)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf)


def accuracy(out: torch.Tensor, ref: torch.Tensor):
    """(cosine similarity over all elements, relative L1) - the two numbers the parity bar uses."""
    a, b = out.double().flatten(), ref.double().flatten()
    cos = float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))
    rel_l1 = float((a - b).abs().sum() / (b.abs().sum() + 1e-30))
    return cos, rel_l1
