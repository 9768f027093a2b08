// Row-wise NVFP4 quantisation of one 128-token tile held in registers, shared by the fused quantisation kernel
// (quant.cu, Q and K roles) and the K quantisation + delta_s kernel (delta_s.cu).
#pragma once

#include "common.cuh"

namespace sage3 {

constexpr int kTile = 128;
constexpr int kThreads = 256;

// Row-wise quantisation of one 128-token tile held in registers (Q and K roles).
// Thread t owns 8 consecutive channels (chunk c) of rows rl, rl+RPP, ... ; w[p] = 4 packed bf16x2.
// ------------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void quant_rows_store(const uint4 (&w)[kTile / (kThreads / (D / 8))],
                                                 uint8_t* __restrict__ codes_tile, uint8_t* __restrict__ sf_tile,
                                                 uint8_t* sf_smem) {
  constexpr int CH = D / 8, RPP = kThreads / CH, NP = kTile / RPP;
  const int t = threadIdx.x, c = t % CH, rl = t / CH;
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int row = p * RPP + rl;
    uint32_t m2 = habsmax2(habsmax2(w[p].x, w[p].y), habsmax2(w[p].z, w[p].w));
    float amax = fmaxf(bf16_lo(m2), bf16_hi(m2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));       // 16-element block = 2 threads
    uint32_t sfb; float inv;
    block_scale(amax, sfb, inv);
    uint32_t code = f32x8_to_e2m1x8(
        mul_ftz(bf16_lo(w[p].x), inv), mul_ftz(bf16_hi(w[p].x), inv), mul_ftz(bf16_lo(w[p].y), inv),
        mul_ftz(bf16_hi(w[p].y), inv), mul_ftz(bf16_lo(w[p].z), inv), mul_ftz(bf16_hi(w[p].z), inv),
        mul_ftz(bf16_lo(w[p].w), inv), mul_ftz(bf16_hi(w[p].w), inv));
    *reinterpret_cast<uint32_t*>(codes_tile + row * (D / 2) + c * 4) = code;
    if ((c & 1) == 0) {
      const int blk = c >> 1;                                        // 16-channel block index
      sf_smem[(blk >> 2) * 512 + sf_atom_offset(row, blk & 3)] = (uint8_t)sfb;
    }
  }
  __syncthreads();
  constexpr int SFV = (D / 64) * 512 / 16;                           // 16-byte vectors of scales
  if (t < SFV) reinterpret_cast<uint4*>(sf_tile)[t] = reinterpret_cast<const uint4*>(sf_smem)[t];
}


}  // namespace sage3
