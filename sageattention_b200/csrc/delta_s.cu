// K quantisation + delta_s in one pass over K:
//   ks            = bf16(k - km)                                       sageattn4/api.py:184
//   K codes / SF  = NVFP4(ks), 128-token tiles                         quantization/fp4_quantization_4d.cu:492-569
//   delta_s[b, hq, qb, n] = bf16( sum_d qm[b, hq, qb, d] * ks[b, hkv, n, d] )   api.py:201
//
// The reference computes delta_s with a bf16 GEMM (fp32 accumulation, bf16 result) that it then widens to fp32.
// It stays bf16 here - the same values in half the bytes - because the attention kernel feeds each row to the
// tensor core as a bf16 operand (rank-1 update of the score accumulator), which restores the Q block mean that
// was removed before quantisation.
//
// One CTA per (128-key tile, kv head): the K tile is read from HBM ONCE, smoothed in registers, quantised (the
// same device function as the fused quantisation kernel, so codes and scales are bit-identical) and laid out
// in shared memory as the B operand of tcgen05.mma kind::f16; the Q block means of every query head of the GQA
// group (rows of A, 128 query blocks at a time) are multiplied against it with the accumulator in tensor
// memory; the [128 query blocks x 128 keys] result goes as bf16 through a swizzled staging tile in shared memory
// and leaves with two TMA stores (whole 128-byte lines; rows beyond the last query block are clipped by the
// tensor map).  HBM-bound: the output ([Tq x 128] bf16 per CTA and query head) dominates the traffic.
//
// Operand layout in shared memory (K-major, no swizzle): 8-row x 16-byte core matrices; the 16 row groups of one
// 8-channel chunk are contiguous (128 B apart), chunks are kChunk bytes apart - 16 bytes more than their size so
// that the 16 lanes which write one row's chunks hit different banks.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "quant_rows.cuh"
#include "tensor_map.h"

namespace sage3 {

namespace {

constexpr uint32_t kChunk = 128 * 16 + 16;            // one 8-channel chunk of 128 rows (+ bank skew)

struct KDsParams {
  const __nv_bfloat16 *qm, *k, *km;
  int64_t k_sb, k_sh, k_sn;
  uint8_t *k_codes, *k_sf;                             // null: K is quantised elsewhere
  __nv_bfloat16* ds;
  int* status;                                         // optional device status word
  int Hq, Hkv, Tq, Tk, Nk;
  const int* cu_k;
  int d_in;                                            // channels the K rows really have; the rest are zero
};

constexpr int kDsStageBytes = 2 * 128 * 128;          // output staging: [2 key halves][128 rows x 128 bytes], 128-byte swizzle

template <int D>
__global__ void __launch_bounds__(kThreads, 2) k_quant_delta_s_kernel(const __grid_constant__ CUtensorMap tm_ds,
                                                                      const KDsParams P) {
  constexpr int CH = D / 8, RPP = kThreads / CH, NP = kTile / RPP;
  constexpr uint32_t kTileBytes = CH * kChunk;
  extern __shared__ uint8_t dyn_raw[];
  uint8_t* dyn_smem = dyn_raw + ((1024u - (smem_u32(dyn_raw) & 1023u)) & 1023u);   // the swizzled staging tile needs it
  uint8_t* stage = dyn_smem;                           // output staging (first: 1024-byte aligned)
  uint8_t* sB = dyn_smem + kDsStageBytes;              // smoothed K tile  [CH][kChunk]
  uint8_t* sA = sB + kTileBytes;                       // 128 Q block means [CH][kChunk]
  uint8_t* sf_smem = sA + kTileBytes;                  // 2048 B
  uint8_t* misc = sf_smem + 2048;                      // mbarrier (8 B), tensor-memory slot (4 B), abort flag (4 B)
  const uint32_t bar = smem_u32(misc), slot = smem_u32(misc + 8);
  int* abort_s = reinterpret_cast<int*>(misc + 12);
  const int tile = blockIdx.x, bh = blockIdx.y, b = bh / P.Hkv, hkv = bh % P.Hkv, G = P.Hq / P.Hkv;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, c = t % CH, rl = t / CH;

  if (t == 0) {
    mbar_init(bar, 1);
    *abort_s = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(slot, 128);
    tmem_relinquish();
  }

  // ---- the K tile: load, smooth, quantise, lay out as the B operand
  int Nk = P.Nk;
  if (P.cu_k != nullptr) Nk = min(P.cu_k[b + 1] - P.cu_k[b], Nk);   // a packed batch: this sequence, cut at max_seqlen
  const __nv_bfloat16* src = P.k + (P.cu_k ? (int64_t)P.cu_k[b] * P.k_sn : b * P.k_sb) + hkv * P.k_sh + c * 8;
  uint4 w[NP];
#pragma unroll
  for (int p = 0; p < NP; ++p) {                       // all loads in flight before the first use
    const int n = tile * kTile + p * RPP + rl;
    w[p] = (n < Nk && c * 8 < P.d_in) ? *reinterpret_cast<const uint4*>(src + (int64_t)n * P.k_sn) : make_uint4(0, 0, 0, 0);
  }
  if (P.km != nullptr) {
    const uint4 m = *reinterpret_cast<const uint4*>(P.km + (int64_t)bh * D + c * 8);
    const float mean[8] = {bf16_lo(m.x), bf16_hi(m.x), bf16_lo(m.y), bf16_hi(m.y),
                           bf16_lo(m.z), bf16_hi(m.z), bf16_lo(m.w), bf16_hi(m.w)};
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      if (tile * kTile + p * RPP + rl < Nk) {          // padding rows stay zero (the reference subtracts before padding)
        w[p].x = pack_bf16(bf16_lo(w[p].x) - mean[0], bf16_hi(w[p].x) - mean[1]);
        w[p].y = pack_bf16(bf16_lo(w[p].y) - mean[2], bf16_hi(w[p].y) - mean[3]);
        w[p].z = pack_bf16(bf16_lo(w[p].z) - mean[4], bf16_hi(w[p].z) - mean[5]);
        w[p].w = pack_bf16(bf16_lo(w[p].w) - mean[6], bf16_hi(w[p].w) - mean[7]);
      }
    }
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int row = p * RPP + rl;
    *reinterpret_cast<uint4*>(sB + c * kChunk + (row >> 3) * 128 + (row & 7) * 16) = w[p];
  }
  if (P.k_codes != nullptr) {
    const int64_t kt = (int64_t)bh * P.Tk + tile;
    quant_rows_store<D>(w, P.k_codes + kt * (kTile * D / 2), P.k_sf + kt * ((D / 64) * 512), sf_smem);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(misc + 8);

  // ---- delta_s: for every query head of the group, 128 query blocks at a time
  constexpr uint32_t idesc = make_idesc_bf16(128, 128);
  constexpr uint32_t HI = (128u >> 4) | (1u << 14);                     // 8-row groups 128 B apart, no swizzle
  const uint32_t a_lo = (smem_u32(sA) >> 4) | ((kChunk >> 4) << 16);    // leading (K) offset = one chunk
  const uint32_t b_lo = (smem_u32(sB) >> 4) | ((kChunk >> 4) << 16);
  const int n_mb = (P.Tq + 127) / 128;
  uint32_t iter = 0;
  bool ok = true;
  // rounds = (query head of the group, block of 128 query blocks); the A tile of the next round is fetched into
  // registers while the current round's MMA runs and its result is written out
  const int rounds = G * n_mb;
  auto load_a = [&](uint4 (&a)[NP], const int round) {
    const int hq = hkv * G + round / n_mb, mb = round % n_mb;
    const __nv_bfloat16* qm_h = P.qm + ((int64_t)b * P.Hq + hq) * P.Tq * D;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int m = mb * 128 + p * RPP + rl;
      a[p] = m < P.Tq ? __ldg(reinterpret_cast<const uint4*>(qm_h + (int64_t)m * D + c * 8)) : make_uint4(0, 0, 0, 0);
    }
  };
  uint4 a_next[NP];
  load_a(a_next, 0);
  for (int round = 0; round < rounds && ok; ++round, ++iter) {
    const int hq = hkv * G + round / n_mb, mb = round % n_mb;
    // A: block means of query blocks mb*128 ... +127 (zeros beyond the last one)
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int row = p * RPP + rl;
      *reinterpret_cast<uint4*>(sA + c * kChunk + (row >> 3) * 128 + (row & 7) * 16) = a_next[p];
    }
    if (t == 0) bulk_wait_read0();                     // the previous round's stores have left the staging tile
    fence_proxy_async_smem();
    __syncthreads();
    if (t == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)              // K = 16 per instruction = two chunks
        tc_mma_bf16(tmem, a_lo + kk * (2 * kChunk >> 4), HI, b_lo + kk * (2 * kChunk >> 4), HI, idesc, kk > 0 ? 1u : 0u);
      tc_commit(bar);
    }
    if (round + 1 < rounds) load_a(a_next, round + 1);
    // bounded: a few microseconds normally; gives up after about a second
    if (P.status != nullptr) {
      ok = wait_bar_warp<false, (1u << 19)>(bar, iter & 1, abort_s, P.status, 50);
    } else {
      ok = __all_sync(0xffffffffu, mbar_wait(bar, iter & 1, 1u << 19));
    }
    tc_fence_after();
    if (ok) {
      // lane = query block (row of the staging tile), 64 keys per thread: warps 0-3 the tile's keys 0-63, warps 4-7
      // keys 64-127 (= the two 128-byte-wide store boxes)
      const int row = (warp & 3) * 32 + lane, half = warp >> 2;
      const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)half * 64;
      uint8_t* srow = stage + half * (128 * 128) + row * 128;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t r[32];
        tmem_ld32(taddr + 32 * part, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(srow + (((4 * part + i) ^ (row & 7)) << 4)) =
              make_uint4(pack_bf16(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                         pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                         pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                         pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])));
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();                                   // the staging tile is complete (and the accumulator read)
    if (ok && t == 0) {
      const int z = b * P.Hq + hq;
      tma_store_3d(&tm_ds, smem_u32(stage), tile * kTile, mb * 128, z);
      tma_store_3d(&tm_ds, smem_u32(stage) + 128 * 128, tile * kTile + 64, mb * 128, z);
      bulk_commit_group();
    }
    // the accumulator and the A tile are rewritten by the next round; every thread leaves the loop together
    tc_fence_before();
    ok = __syncthreads_and(ok);
  }
  if (t == 0) bulk_wait_read0();                       // the last stores have read the staging tile before the CTA ends
  if (!ok && t == 0) {
    // the MMAs issued last may still be running: give them time to drain before tensor memory is freed
    mbar_wait(bar, iter & 1, 1u << 16);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace

cudaError_t launch_delta_s(const DeltaSArgs& a, cudaStream_t stream) {
  KDsParams P;
  P.qm = (const __nv_bfloat16*)a.qm; P.k = (const __nv_bfloat16*)a.k; P.km = (const __nv_bfloat16*)a.km;
  P.k_sb = a.k_sb; P.k_sh = a.k_sh; P.k_sn = a.k_sn;
  P.k_codes = (uint8_t*)a.k_codes; P.k_sf = (uint8_t*)a.k_sf;
  P.ds = (__nv_bfloat16*)a.ds; P.status = a.status;
  P.Hq = a.Hq; P.Hkv = a.Hkv; P.Tq = a.Tq; P.Nk = a.Nk; P.Tk = (a.Nk + 127) / 128;
  P.cu_k = a.cu_k;
  P.d_in = (a.d_in > 0 && a.d_in <= a.D) ? a.d_in : a.D;
  dim3 grid(P.Tk, a.B * a.Hkv);
  // delta_s as a 3-D bf16 tensor (key, query block, batch x query head); store boxes of 64 keys x 128 query blocks
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return cudaErrorInvalidValue;
  CUtensorMap tm;
  {
    const cuuint64_t nk_pad = (cuuint64_t)P.Tk * kTile;
    cuuint64_t dims[3] = {nk_pad, (cuuint64_t)a.Tq, (cuuint64_t)a.B * a.Hq};
    cuuint64_t strides[2] = {nk_pad * 2, nk_pad * 2 * (cuuint64_t)a.Tq};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.ds, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  const int smem = kDsStageBytes + 2 * (a.D / 8) * (int)kChunk + 2048 + 16 + 1024;
  // per device and cheap, so set on every call rather than cached per process
  cudaError_t e = a.D == 128
      ? cudaFuncSetAttribute(k_quant_delta_s_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
      : cudaFuncSetAttribute(k_quant_delta_s_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  if (a.D == 128) k_quant_delta_s_kernel<128><<<grid, kThreads, smem, stream>>>(tm, P);
  else            k_quant_delta_s_kernel<64><<<grid, kThreads, smem, stream>>>(tm, P);
  return cudaGetLastError();
}

}  // namespace sage3
