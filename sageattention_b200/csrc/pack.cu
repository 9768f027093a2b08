// K / V packing of the K-packing mode ("SageAttention4" of the fork): every 15 tokens become 16 key slots.
//
// Replaces the eager PyTorch preprocessing of sageattn4/api.py:122-177 (quant_pack_k, quant_pack_v with either
// value of split_first) and the K centring of :184.  Per (batch, kv head) and group g of 15 tokens (the last
// group zero-padded), with x_j = bf16(k_j - k_mean):
//   slot 0      m    = FP4-rounded group mean   (bf16(sum_j x_j / 15), then the block-scaled FP4 round trip
//                                                of api.py:77-106 along the head dimension)
//   slots 1..15 r_j  = bf16(x_j - lambda_j * m), lambda_j = <x_j, m> / |m|^2          (fp32)
//   lambda      [0, lambda_1 .. lambda_15]       fp32, one value per slot
//   V           a zero row in slot 0, the 15 value rows behind it; or ("split first", the reference's v_trick): slot 1
//               holds the first token's row as the V^T quantiser will round it (block-scaled FP4 over the 16 slots
//               of the group, per channel), slot 0 the remainder v_1 - round(v_1), so that a kernel which gives slot 0
//               the first token's probability sees that token's V to two FP4 terms
// The attention kernel later restores q.k_j as q.r_j + lambda_j * (q.m) (fwd_mainloop.cu:796-845).
//
// HBM-bound: one warp per group, rows read once with 8-byte loads (a warp reads one 256-byte row per
// instruction), the 15 rows of the group live in registers between the two passes (mean, residual).
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

namespace sage3 {

namespace {

constexpr int kPackThreads = 256;
constexpr int kGroup = 15;

// magnitude of an E2M1 code: 0, 0.5, 1, 1.5, 2, 3, 4, 6 (sign in bit 3)
__device__ __forceinline__ float e2m1_value(const uint32_t code) {
  const uint32_t mag = code & 7u;
  const float lvl = mag < 2 ? 0.5f * mag : (mag < 4 ? 1.0f + 0.5f * (mag - 2) : (mag < 6 ? 2.0f + (mag - 4) : (mag == 6 ? 4.0f : 6.0f)));
  return (code & 8u) ? -lvl : lvl;
}

template <int D>
__global__ void __launch_bounds__(kPackThreads) pack_kv_kernel(
    const __nv_bfloat16* __restrict__ k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
    const __nv_bfloat16* __restrict__ v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
    const __nv_bfloat16* __restrict__ km, __nv_bfloat16* __restrict__ kp, __nv_bfloat16* __restrict__ vp,
    float* __restrict__ lam, int H, int N, int G, int lam_len, int split_first) {
  constexpr int C = D / 32;                         // channels per lane (4 or 2)
  constexpr int kLanesPerBlock = 16 / C;            // lanes that share one 16-channel scale block
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int Np = G * 16;
  const __nv_bfloat16* kbase = k + b * k_sb + h * k_sh + lane * C;
  const __nv_bfloat16* vbase = v ? v + b * v_sb + h * v_sh + lane * C : nullptr;
  __nv_bfloat16* kpb = kp + (int64_t)bh * Np * D + lane * C;
  __nv_bfloat16* vpb = vp ? vp + (int64_t)bh * Np * D + lane * C : nullptr;
  float* lamb = lam + (int64_t)bh * lam_len;

  float kmf[C];
#pragma unroll
  for (int c = 0; c < C; ++c) kmf[c] = km ? __bfloat162float(km[(int64_t)bh * D + lane * C + c]) : 0.f;

  for (int g = blockIdx.x * (kPackThreads / 32) + warp; g < G; g += gridDim.x * (kPackThreads / 32)) {
    const int t0 = g * kGroup;
    // ---- load the 15 rows, centre them (bf16 arithmetic of `k - k.mean()`: fp32 subtract, round to bf16)
    float x[kGroup][C];
    float sum[C];
#pragma unroll
    for (int c = 0; c < C; ++c) sum[c] = 0.f;
#pragma unroll
    for (int j = 0; j < kGroup; ++j) {
      const int t = t0 + j;
      if (t < N) {
        if constexpr (C == 4) {
          const uint2 raw = *reinterpret_cast<const uint2*>(kbase + (int64_t)t * k_sn);
          x[j][0] = bf16_lo(raw.x); x[j][1] = bf16_hi(raw.x); x[j][2] = bf16_lo(raw.y); x[j][3] = bf16_hi(raw.y);
        } else {
          const uint32_t raw = *reinterpret_cast<const uint32_t*>(kbase + (int64_t)t * k_sn);
          x[j][0] = bf16_lo(raw); x[j][1] = bf16_hi(raw);
        }
#pragma unroll
        for (int c = 0; c < C; ++c) x[j][c] = __bfloat162float(__float2bfloat16(x[j][c] - kmf[c]));
      } else {
#pragma unroll
        for (int c = 0; c < C; ++c) x[j][c] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < C; ++c) sum[c] += x[j][c];
    }
    // ---- group mean -> bf16 -> block-scaled FP4 round trip along the head dimension (16-channel blocks)
    float m[C];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
      m[c] = __bfloat162float(__float2bfloat16(__fdiv_rn(sum[c], (float)kGroup)));
      amax = fmaxf(amax, fabsf(m[c]));
    }
#pragma unroll
    for (int o = 1; o < kLanesPerBlock; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = e4m3_to_f32(f32_to_e4m3(__fdiv_rn(amax, 6.0f)));
    const float inv = scale == 0.f ? 0.f : __frcp_rn(scale);
    {
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < C; ++c) sc[c] = __fmul_rn(m[c], inv);
      // E2M1 round-to-nearest-even with saturation, then back to fp32 through the 8 magnitudes
      uint32_t codes = f32x8_to_e2m1x8(sc[0], sc[1], sc[2], sc[3], 0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < C; ++c) {
        m[c] = __bfloat162float(__float2bfloat16(__fmul_rn(e2m1_value((codes >> (4 * c)) & 0xFu), scale)));
      }
    }
    // ---- direction = m / |m|^2
    float nsq = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) nsq = fmaf(m[c], m[c], nsq);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nsq += __shfl_xor_sync(0xffffffffu, nsq, o);
    float dir[C];
#pragma unroll
    for (int c = 0; c < C; ++c) dir[c] = nsq > 0.f ? __fdiv_rn(m[c], nsq) : 0.f;

    // ---- slot 0: the rounded mean
    const int64_t row0 = (int64_t)g * 16;
    if constexpr (C == 4) {
      *reinterpret_cast<uint2*>(kpb + row0 * D) = make_uint2(pack_bf16(m[0], m[1]), pack_bf16(m[2], m[3]));
    } else {
      *reinterpret_cast<uint32_t*>(kpb + row0 * D) = pack_bf16(m[0], m[1]);
    }
    // ---- slots 1..15: lambda and residual
    float my_lam = 0.f;                               // lane s keeps lambda of slot s
#pragma unroll
    for (int j = 0; j < kGroup; ++j) {
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < C; ++c) dot = fmaf(x[j][c], dir[c], dot);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == j + 1) my_lam = dot;
      float r[C];
#pragma unroll
      for (int c = 0; c < C; ++c) r[c] = __fsub_rn(x[j][c], __fmul_rn(dot, m[c]));
      const int64_t row = row0 + 1 + j;
      if constexpr (C == 4) {
        *reinterpret_cast<uint2*>(kpb + row * D) = make_uint2(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]));
      } else {
        *reinterpret_cast<uint32_t*>(kpb + row * D) = pack_bf16(r[0], r[1]);
      }
    }
    // ---- V: the 15 rows behind their slots; slot 0 zero, or (split first) the first row in two FP4 terms
    if (vpb) {
      float vf[kGroup][C];
#pragma unroll
      for (int j = 0; j < kGroup; ++j) {
        const int t = t0 + j;
        if constexpr (C == 4) {
          uint2 raw = make_uint2(0u, 0u);
          if (t < N) raw = *reinterpret_cast<const uint2*>(vbase + (int64_t)t * v_sn);
          vf[j][0] = bf16_lo(raw.x); vf[j][1] = bf16_hi(raw.x); vf[j][2] = bf16_lo(raw.y); vf[j][3] = bf16_hi(raw.y);
        } else {
          uint32_t raw = 0u;
          if (t < N) raw = *reinterpret_cast<const uint32_t*>(vbase + (int64_t)t * v_sn);
          vf[j][0] = bf16_lo(raw); vf[j][1] = bf16_hi(raw);
        }
      }
      float slot[C];
#pragma unroll
      for (int c = 0; c < C; ++c) slot[c] = 0.f;
      if (split_first) {
        // what scaled_fp4_quant_trans will make of the first row: one scale per channel over the group's 16 slots
        // (slot 0 still zero), emulation arithmetic of api.py:77-110 (true division, round to nearest even)
#pragma unroll
        for (int c = 0; c < C; ++c) {
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < kGroup; ++j) amax = fmaxf(amax, fabsf(vf[j][c]));
          const float scale = e4m3_to_f32(f32_to_e4m3(__fdiv_rn(amax, 6.0f)));
          const float inv = scale == 0.f ? 0.f : __frcp_rn(scale);
          const uint32_t code = f32x8_to_e2m1x8(__fmul_rn(vf[0][c], inv), 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f) & 0xFu;
          const float hi = __bfloat162float(__float2bfloat16(__fmul_rn(e2m1_value(code), scale)));
          slot[c] = __fsub_rn(vf[0][c], hi);
          vf[0][c] = hi;
        }
      }
      if constexpr (C == 4) {
        *reinterpret_cast<uint2*>(vpb + row0 * D) = make_uint2(pack_bf16(slot[0], slot[1]), pack_bf16(slot[2], slot[3]));
#pragma unroll
        for (int j = 0; j < kGroup; ++j)
          *reinterpret_cast<uint2*>(vpb + (row0 + 1 + j) * D) = make_uint2(pack_bf16(vf[j][0], vf[j][1]), pack_bf16(vf[j][2], vf[j][3]));
      } else {
        *reinterpret_cast<uint32_t*>(vpb + row0 * D) = pack_bf16(slot[0], slot[1]);
#pragma unroll
        for (int j = 0; j < kGroup; ++j) *reinterpret_cast<uint32_t*>(vpb + (row0 + 1 + j) * D) = pack_bf16(vf[j][0], vf[j][1]);
      }
    }
    if (lane < 16) lamb[row0 + lane] = my_lam;
    // the slots behind the last group, up to the padded length, carry lambda = 0
    if (g == G - 1)
      for (int i = Np + lane; i < lam_len; i += 32) lamb[i] = 0.f;
  }
}

}  // namespace

cudaError_t launch_pack_kv(const PackArgs& a, cudaStream_t stream) {
  const int G = (a.Nk + kGroup - 1) / kGroup;
  if (G == 0) return cudaSuccess;
  const int lam_len = ((G * 16 + 127) / 128) * 128;
  const int per_block = kPackThreads / 32;
  int gx = (G + per_block - 1) / per_block;
  // enough blocks to fill the GPU a few times over; warps loop over the remaining groups
  const int cap = max(1, (148 * 16) / max(1, a.B * a.Hkv));
  if (gx > cap) gx = cap;
  dim3 grid(gx, a.B * a.Hkv);
  auto K = (const __nv_bfloat16*)a.k;
  auto V = (const __nv_bfloat16*)a.v;
  if (a.D == 128)
    pack_kv_kernel<128><<<grid, kPackThreads, 0, stream>>>(K, a.k_sb, a.k_sh, a.k_sn, V, a.v_sb, a.v_sh, a.v_sn,
                                                           (const __nv_bfloat16*)a.km, (__nv_bfloat16*)a.kp,
                                                           (__nv_bfloat16*)a.vp, a.lam, a.Hkv, a.Nk, G, lam_len, a.split_first);
  else
    pack_kv_kernel<64><<<grid, kPackThreads, 0, stream>>>(K, a.k_sb, a.k_sh, a.k_sn, V, a.v_sb, a.v_sh, a.v_sn,
                                                          (const __nv_bfloat16*)a.km, (__nv_bfloat16*)a.kp,
                                                          (__nv_bfloat16*)a.vp, a.lam, a.Hkv, a.Nk, G, lam_len, a.split_first);
  return cudaGetLastError();
}

}  // namespace sage3
