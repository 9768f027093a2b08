// delta_s[b, hq, qb, n] = bf16( sum_d qm[b, hq, qb, d] * ks[b, hkv, n, d] ),  ks = bf16(k - km)
//
// Replaces `delta_s = torch.matmul(qm, k.transpose(-2, -1)).to(torch.float32)` of
// sageattn4/api.py:201: a bf16 GEMM (fp32 accumulation, bf16 result) that the reference then
// widens to fp32.  It stays bf16 here - the same values in half the bytes - because the
// attention kernel feeds each row to the tensor core as a bf16 operand (rank-1 update of the
// score accumulator), which restores the Q block mean that was removed before quantisation.
//
// One CTA per (128-key tile, kv head): the smoothed K tile is rebuilt in shared memory once and
// multiplied against the block means of every query head of the GQA group.  The output
// ([Tq x 128] bf16 per CTA and head) dominates the traffic, so the small contraction runs on
// mma.sync m16n8k16 with fragments read straight from shared memory, and results are staged per
// warp so that they leave as whole 256-byte rows.
#include "common.cuh"
#include "kernels.h"

namespace sage3 {

template <int D>
__global__ void __launch_bounds__(256, 3) delta_s_kernel(
    const __nv_bfloat16* __restrict__ qm, const __nv_bfloat16* __restrict__ k, int64_t k_sb, int64_t k_sh,
    int64_t k_sn, const __nv_bfloat16* __restrict__ km, __nv_bfloat16* __restrict__ ds, int Hq, int Hkv, int Tq,
    int Nk, int Nk_pad, const int* __restrict__ cu_k) {
  constexpr int PITCH = D + 8;                         // bf16 elements; 4-bank skew per row
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(dyn_smem);              // [128][PITCH]
  __nv_bfloat16* cs = ks + 128 * PITCH;                                        // [8 warps][16][136]
  const int tile = blockIdx.x, bh = blockIdx.y, b = bh / Hkv, hkv = bh % Hkv, G = Hq / Hkv;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tg = lane & 3;

  // A fragments (rows m0+g and m0+g+8 of the stacked block means of this GQA group) come from global memory /
  // L2; the first set is requested before the K tile is built and the next one while the current one is
  // multiplied, so their latency is not on the critical path
  const int M = G * Tq;
  auto load_a = [&](uint32_t (&a)[D / 16][4], const int m0) {
    const int r0 = m0 + g, r1 = m0 + g + 8;
    const uint32_t* p0 = nullptr; const uint32_t* p1 = nullptr;
    if (r0 < M) p0 = reinterpret_cast<const uint32_t*>(qm + (((int64_t)b * Hq + hkv * G + r0 / Tq) * Tq + r0 % Tq) * D);
    if (r1 < M) p1 = reinterpret_cast<const uint32_t*>(qm + (((int64_t)b * Hq + hkv * G + r1 / Tq) * Tq + r1 % Tq) * D);
#pragma unroll
    for (int s = 0; s < D / 16; ++s) {
      a[s][0] = p0 ? __ldg(p0 + s * 8 + tg) : 0u;
      a[s][1] = p1 ? __ldg(p1 + s * 8 + tg) : 0u;
      a[s][2] = p0 ? __ldg(p0 + s * 8 + 4 + tg) : 0u;
      a[s][3] = p1 ? __ldg(p1 + s * 8 + 4 + tg) : 0u;
    }
  };
  uint32_t a_next[D / 16][4];
  load_a(a_next, warp * 16);

  {  // smoothed K tile -> shared
    constexpr int CH = D / 8, RPP = 256 / CH;
    const int c = t % CH, rl = t / CH;
    float mean[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (km != nullptr) {
      uint4 m = *reinterpret_cast<const uint4*>(km + (int64_t)bh * D + c * 8);
      mean[0] = bf16_lo(m.x); mean[1] = bf16_hi(m.x); mean[2] = bf16_lo(m.y); mean[3] = bf16_hi(m.y);
      mean[4] = bf16_lo(m.z); mean[5] = bf16_hi(m.z); mean[6] = bf16_lo(m.w); mean[7] = bf16_hi(m.w);
    }
    // variable-length batch: sequence b starts at token cu_k[b] of the packed tensor and has its own length
    if (cu_k != nullptr) Nk = min(cu_k[b + 1] - cu_k[b], Nk);   // cut at max_seqlen like every other kernel
    const __nv_bfloat16* src = k + (cu_k ? (int64_t)cu_k[b] * k_sn : b * k_sb) + hkv * k_sh + c * 8;
    uint4 w[128 / RPP];
#pragma unroll
    for (int p = 0; p < 128 / RPP; ++p) {                  // all loads in flight before the first use
      const int n = tile * 128 + p * RPP + rl;
      w[p] = make_uint4(0, 0, 0, 0);
      if (n < Nk) w[p] = *reinterpret_cast<const uint4*>(src + (int64_t)n * k_sn);
    }
#pragma unroll
    for (int p = 0; p < 128 / RPP; ++p) {
      const int r = p * RPP + rl, n = tile * 128 + r;
      uint4 x = w[p];
      if (n < Nk) {
        x.x = pack_bf16(bf16_lo(x.x) - mean[0], bf16_hi(x.x) - mean[1]);
        x.y = pack_bf16(bf16_lo(x.y) - mean[2], bf16_hi(x.y) - mean[3]);
        x.z = pack_bf16(bf16_lo(x.z) - mean[4], bf16_hi(x.z) - mean[5]);
        x.w = pack_bf16(bf16_lo(x.w) - mean[6], bf16_hi(x.w) - mean[7]);
      }
      *reinterpret_cast<uint4*>(&ks[r * PITCH + c * 8]) = x;
    }
  }
  __syncthreads();

  const uint32_t* ks32 = reinterpret_cast<const uint32_t*>(ks);
  for (int m0 = warp * 16; m0 < M; m0 += 8 * 16) {
    uint32_t a[D / 16][4];
#pragma unroll
    for (int s = 0; s < D / 16; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i) a[s][i] = a_next[s][i];
    if (m0 + 8 * 16 < M) load_a(a_next, m0 + 8 * 16);
    __nv_bfloat16* cw = cs + warp * (16 * 136);
#pragma unroll 4
    for (int nt = 0; nt < 16; ++nt) {
      float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
      const uint32_t* brow = ks32 + (nt * 8 + g) * (PITCH / 2) + tg;
#pragma unroll
      for (int s = 0; s < D / 16; ++s) {
        uint32_t b0 = brow[s * 8], b1 = brow[s * 8 + 4];
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
            : "r"(a[s][0]), "r"(a[s][1]), "r"(a[s][2]), "r"(a[s][3]), "r"(b0), "r"(b1));
      }
      *reinterpret_cast<uint32_t*>(&cw[g * 136 + nt * 8 + tg * 2]) = pack_bf16(c0, c1);
      *reinterpret_cast<uint32_t*>(&cw[(g + 8) * 136 + nt * 8 + tg * 2]) = pack_bf16(c2, c3);
    }
    __syncwarp();
    // 16 rows x 256 bytes leave as whole rows: two rows per warp store instruction
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i * 2 + (lane >> 4), m = m0 + r;
      if (m < M) {
        uint4 v = *reinterpret_cast<const uint4*>(&cw[r * 136 + (lane & 15) * 8]);
        __nv_bfloat16* dst = ds + ((((int64_t)b * Hq + hkv * G + m / Tq) * Tq + m % Tq) * Nk_pad + tile * 128);
        reinterpret_cast<uint4*>(dst)[lane & 15] = v;
      }
    }
    __syncwarp();
  }
}

cudaError_t launch_delta_s(const DeltaSArgs& a, cudaStream_t stream) {
  const int Tk = (a.Nk + 127) / 128;
  dim3 grid(Tk, a.B * a.Hkv);
  const int smem = (128 * (a.D + 8) + 8 * 16 * 136) * 2;
  // per device and cheap, so set on every call rather than cached per process
  cudaError_t e = a.D == 128
      ? cudaFuncSetAttribute(delta_s_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
      : cudaFuncSetAttribute(delta_s_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  if (a.D == 128)
    delta_s_kernel<128><<<grid, 256, smem, stream>>>((const __nv_bfloat16*)a.qm, (const __nv_bfloat16*)a.k, a.k_sb, a.k_sh,
                                                  a.k_sn, (const __nv_bfloat16*)a.km, (__nv_bfloat16*)a.ds, a.Hq, a.Hkv,
                                                  a.Tq, a.Nk, Tk * 128, a.cu_k);
  else
    delta_s_kernel<64><<<grid, 256, smem, stream>>>((const __nv_bfloat16*)a.qm, (const __nv_bfloat16*)a.k, a.k_sb, a.k_sh,
                                                 a.k_sn, (const __nv_bfloat16*)a.km, (__nv_bfloat16*)a.ds, a.Hq, a.Hkv,
                                                 a.Tq, a.Nk, Tk * 128, a.cu_k);
  return cudaGetLastError();
}

}  // namespace sage3
