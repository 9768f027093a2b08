// Fused smoothing + NVFP4 quantisation of Q, K and V for the FP4 attention kernel (sm_100a).
//
// Replaces, in one launch (plus one small reduction launch for the K channel means):
//   * K minus its per-channel mean over tokens        sageattn4/api.py:184
//   * Q zero-padded to 128 rows, minus per-128-row mean sageattn4/api.py:26-72,186-191
//   * NVFP4 quantisation of Q                          quantization/fp4_quantization_4d.cu:164-284,414-490
//   * NVFP4 quantisation of K (the reference permutes rows for its mma.sync fragment layout,
//     :146-162; tensor memory accumulators make that unnecessary, rows stay in token order)
//   * transpose + NVFP4 quantisation of V along tokens :286-412,571-648
//
// The arithmetic per 16-element block is the reference's, instruction for instruction
// (common.cuh: block_scale, f32x8_to_e2m1x8), so codes and scale bytes are bit-identical.
//
// Memory plan (HBM-bound): every thread issues all of its 128-bit loads for a 128-token tile
// before the first use (a whole 32 KB tile in flight per CTA), pairs of threads combine their
// 8-element absmax with one warp shuffle, codes leave as full 32-byte sectors and the scale
// bytes are staged in shared memory so that they leave as 16-byte vectors in the exact order
// the attention kernel's tcgen05.cp expects.
//
// Output layouts (per batch b, head h; Np = tokens padded to a multiple of 128, T = Np/128):
//   codes  Q,K : [T][128 rows][D/2] bytes            (row-major, element 2i in the low nibble)
//   scales Q,K : [T][D/64][512] bytes                (SF atom, sf_atom_offset())
//   codes  V^T : [T][D rows][64] bytes               (row d holds the tile's 128 tokens)
//   scales V^T : [T][2][512] bytes                   (atom rows = d, columns = 16-token blocks)
//   qm         : [T][D] bf16 block means of Q;  km : [D] bf16 channel means of K
#include "common.cuh"
#include "kernels.h"
#include "quant_rows.cuh"

namespace sage3 {

// ------------------------------------------------------------------------------------------------
// Channel sums over tokens (K channel mean; also the whole-sequence Q mean when per_block_mean=0).
// grid = (chunks, B*H).  Each CTA writes one fp32 partial row; the last CTA of a (b,h) to finish
// adds the partial rows in chunk order (deterministic) and writes mean = sum / divisor as bf16.
// scratch: partial[B*H][chunks][D] fp32 followed by counters[B*H] u32 (zeroed by the host).
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads) channel_mean_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sh, int64_t sn, int H, int N,
    int chunk_tokens, float divisor, float* __restrict__ partial, unsigned int* __restrict__ counters,
    __nv_bfloat16* __restrict__ mean_out, const int* __restrict__ cu, int d_in) {
  constexpr int CH = D / 8;              // 16-byte chunks per row
  constexpr int RPP = kThreads / CH;     // rows per pass
  __shared__ float red[RPP][D];
  __shared__ bool is_last;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int chunk = blockIdx.x, nchunks = gridDim.x;
  const int t = threadIdx.x, c = t % CH, rl = t / CH;
  // variable-length batch: sequence b starts at token cu[b] of the packed tensor and has its own length
  if (cu != nullptr) {
    N = min(cu[b + 1] - cu[b], N);         // never beyond the caller's max_seqlen (the grid covers no more)
    divisor = (float)max(N, 1);
  }
  const __nv_bfloat16* base = x + (cu ? (int64_t)cu[b] * sn : b * sb) + h * sh + c * 8;
  const int n0 = chunk * chunk_tokens;
  const int n1 = min(N, n0 + chunk_tokens);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int n = n0 + rl; n < n1; n += RPP * 4) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int nn = n + u * RPP;
      v[u] = (nn < n1 && c * 8 < d_in) ? *reinterpret_cast<const uint4*>(base + (int64_t)nn * sn) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      acc[0] += bf16_lo(v[u].x); acc[1] += bf16_hi(v[u].x);
      acc[2] += bf16_lo(v[u].y); acc[3] += bf16_hi(v[u].y);
      acc[4] += bf16_lo(v[u].z); acc[5] += bf16_hi(v[u].z);
      acc[6] += bf16_lo(v[u].w); acc[7] += bf16_hi(v[u].w);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rl][c * 8 + i] = acc[i];
  __syncthreads();
  float* prow = partial + ((int64_t)bh * nchunks + chunk) * D;
  if (t < D) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < RPP; ++r) s += red[r][t];
    prow[t] = s;
  }
  __threadfence();
  __syncthreads();
  if (t == 0) is_last = (atomicAdd(&counters[bh], 1u) == (unsigned)(nchunks - 1));
  __syncthreads();
  if (is_last) {
    __threadfence();
    if (t < D) {
      const float* p = partial + (int64_t)bh * nchunks * D + t;
      float s = 0.f;
      for (int i = 0; i < nchunks; ++i) s += __ldcg(p + (int64_t)i * D);
      mean_out[(int64_t)bh * D + t] = __float2bfloat16_rn(s / divisor);
    }
    if (t == 0) counters[bh] = 0;        // leave the scratch clean for the next call
  }
}

struct QuantLaunch {
  const __nv_bfloat16 *q, *k, *v;
  int64_t q_sb, q_sh, q_sn, k_sb, k_sh, k_sn, v_sb, v_sh, v_sn;
  int B, Hq, Hkv, Nq, Nk, Tq, Tk;        // T* = number of 128-token tiles
  int q_mean_mode;                       // 0 none, 1 per 128-token block, 2 whole sequence (mean given)
  const __nv_bfloat16* km;               // [B,Hkv,D] K channel means
  const __nv_bfloat16* q_mean_seq;       // [B,Hq,D] (mode 2)
  const float* qm_override;              // optional fp32 block means [B,Hq,Tq,D] (mode 1)
  uint8_t *q_codes, *q_sf, *k_codes, *k_sf, *vt_codes, *vt_sf;
  __nv_bfloat16* qm;                     // [B,Hq,Tq,D] (mode 1)
  int q_blocks, k_blocks, v_blocks;      // CTAs per role
  const int *cu_q, *cu_k;                // variable-length batches (else null)
  int d_in;                              // channels the input rows really have (<= D, multiple of 8); the rest are zero
  float* q_dot_km;                       // optional fp32 [B,Hq,Nq]: raw q . K channel mean of the row's kv head
  const __nv_bfloat16* km_for_q;         //   (the term K smoothing removes from every score of the row)
};

template <int D>
__global__ void __launch_bounds__(kThreads) quant_qkv_kernel(const QuantLaunch P) {
  constexpr int CH = D / 8, RPP = kThreads / CH, NP = kTile / RPP;
  __shared__ __align__(16) uint8_t sf_smem[2048];
  __shared__ float red[kThreads / 32][D];
  __shared__ float mean_s[D];
  const int t = threadIdx.x, c = t % CH, rl = t / CH;
  int bid = blockIdx.x;

  if (bid < P.q_blocks + P.k_blocks) {
    // ----------------------------------------------------------------------------- Q / K roles
    const bool is_q = bid < P.q_blocks;
    if (!is_q) bid -= P.q_blocks;
    const int T = is_q ? P.Tq : P.Tk, H = is_q ? P.Hq : P.Hkv;
    int N = is_q ? P.Nq : P.Nk;
    const int tile = bid % T, bh = bid / T, b = bh / H, h = bh % H;
    const int64_t sn = is_q ? P.q_sn : P.k_sn;
    const int* cu = is_q ? P.cu_q : P.cu_k;
    const __nv_bfloat16* src = is_q ? P.q + b * P.q_sb + h * P.q_sh : P.k + b * P.k_sb + h * P.k_sh;
    if (cu != nullptr) {                   // sequence b of a packed [tokens, H, D] tensor
      N = min(cu[b + 1] - cu[b], N);       // cut at max_seqlen, which sizes the output layouts
      src = (is_q ? P.q + h * P.q_sh : P.k + h * P.k_sh) + (int64_t)cu[b] * sn;
    }
    uint4 w[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int n = tile * kTile + p * RPP + rl;
      w[p] = (n < N && c * 8 < P.d_in) ? *reinterpret_cast<const uint4*>(src + (int64_t)n * sn + c * 8) : make_uint4(0, 0, 0, 0);
    }
    if (is_q && P.q_dot_km != nullptr) {
      // q . km in fp32 from the raw rows: what K smoothing took out of every score of the row; the attention
      // kernel adds sm_scale times it to the log-sum-exp (the pattern of sageattention/core.py:993-994)
      const int hkv = h / (P.Hq / P.Hkv);
      const uint4 m = *reinterpret_cast<const uint4*>(P.km_for_q + ((int64_t)b * P.Hkv + hkv) * D + c * 8);
      const float kmv[8] = {bf16_lo(m.x), bf16_hi(m.x), bf16_lo(m.y), bf16_hi(m.y),
                            bf16_lo(m.z), bf16_hi(m.z), bf16_lo(m.w), bf16_hi(m.w)};
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        float d = bf16_lo(w[p].x) * kmv[0];
        d = fmaf(bf16_hi(w[p].x), kmv[1], d); d = fmaf(bf16_lo(w[p].y), kmv[2], d); d = fmaf(bf16_hi(w[p].y), kmv[3], d);
        d = fmaf(bf16_lo(w[p].z), kmv[4], d); d = fmaf(bf16_hi(w[p].z), kmv[5], d); d = fmaf(bf16_lo(w[p].w), kmv[6], d);
        d = fmaf(bf16_hi(w[p].w), kmv[7], d);
#pragma unroll
        for (int o = 1; o < CH; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const int n = tile * kTile + p * RPP + rl;
        if (c == 0 && n < N) P.q_dot_km[(int64_t)bh * P.Nq + n] = d;
      }
    }
    float mean[8];
    bool subtract = true;
    if (is_q && P.q_mean_mode == 1) {
      if (P.qm_override != nullptr) {
        const float* mp = P.qm_override + ((int64_t)bh * T + tile) * D + c * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) mean[i] = mp[i];
      } else {
        // fp32 column sums over the tile's 128 rows (zero rows of the padding included), / 128
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          acc[0] += bf16_lo(w[p].x); acc[1] += bf16_hi(w[p].x);
          acc[2] += bf16_lo(w[p].y); acc[3] += bf16_hi(w[p].y);
          acc[4] += bf16_lo(w[p].z); acc[5] += bf16_hi(w[p].z);
          acc[6] += bf16_lo(w[p].w); acc[7] += bf16_hi(w[p].w);
        }
        if (CH == 16) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
          }
        }
        if ((t & 31) < CH) {
#pragma unroll
          for (int i = 0; i < 8; ++i) red[t >> 5][c * 8 + i] = acc[i];
        }
        __syncthreads();
        if (t < D) {
          float s = 0.f;
#pragma unroll
          for (int r = 0; r < kThreads / 32; ++r) s += red[r][t];
          mean_s[t] = s * (1.0f / kTile);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) mean[i] = mean_s[c * 8 + i];
      }
      if (rl == 0) {   // bf16 block mean, consumed by the delta_s kernel
        uint4 o;
        o.x = pack_bf16(mean[0], mean[1]); o.y = pack_bf16(mean[2], mean[3]);
        o.z = pack_bf16(mean[4], mean[5]); o.w = pack_bf16(mean[6], mean[7]);
        *reinterpret_cast<uint4*>(P.qm + ((int64_t)bh * T + tile) * D + c * 8) = o;
      }
    } else if (is_q && P.q_mean_mode == 2) {
      uint4 m = *reinterpret_cast<const uint4*>(P.q_mean_seq + (int64_t)bh * D + c * 8);
      mean[0] = bf16_lo(m.x); mean[1] = bf16_hi(m.x); mean[2] = bf16_lo(m.y); mean[3] = bf16_hi(m.y);
      mean[4] = bf16_lo(m.z); mean[5] = bf16_hi(m.z); mean[6] = bf16_lo(m.w); mean[7] = bf16_hi(m.w);
    } else if (!is_q && P.km != nullptr) {
      uint4 m = *reinterpret_cast<const uint4*>(P.km + (int64_t)bh * D + c * 8);
      mean[0] = bf16_lo(m.x); mean[1] = bf16_hi(m.x); mean[2] = bf16_lo(m.y); mean[3] = bf16_hi(m.y);
      mean[4] = bf16_lo(m.z); mean[5] = bf16_hi(m.z); mean[6] = bf16_lo(m.w); mean[7] = bf16_hi(m.w);
    } else {
      subtract = false;
    }
    if (subtract) {
      // x - mean in fp32, rounded to bf16 (what a bf16 tensor subtraction does).  Q: padding rows
      // become -mean like the reference (it pads before subtracting); K: padding rows stay zero
      // (the reference subtracts before padding).
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        const int n = tile * kTile + p * RPP + rl;
        if (is_q || n < N) {
          w[p].x = pack_bf16(bf16_lo(w[p].x) - mean[0], bf16_hi(w[p].x) - mean[1]);
          w[p].y = pack_bf16(bf16_lo(w[p].y) - mean[2], bf16_hi(w[p].y) - mean[3]);
          w[p].z = pack_bf16(bf16_lo(w[p].z) - mean[4], bf16_hi(w[p].z) - mean[5]);
          w[p].w = pack_bf16(bf16_lo(w[p].w) - mean[6], bf16_hi(w[p].w) - mean[7]);
        }
      }
    }
    uint8_t* codes = (is_q ? P.q_codes : P.k_codes) + ((int64_t)bh * T + tile) * (kTile * D / 2);
    uint8_t* sf = (is_q ? P.q_sf : P.k_sf) + ((int64_t)bh * T + tile) * ((D / 64) * 512);
    quant_rows_store<D>(w, codes, sf, sf_smem);
    return;
  }

  // ------------------------------------------------------------------------------------- V role
  // One warp = 4 groups of 4 channels x the 8 token blocks of a tile; a thread loads 16 tokens x
  // 4 channels (8-byte loads; a warp load touches 8 rows x one full 32-byte sector) and emits,
  // per channel, 8 bytes of codes + 1 scale.  Eight lanes with the same channel write one
  // contiguous 64-byte row of the V^T tile.
  bid -= P.q_blocks + P.k_blocks;
  constexpr int WPT = D / 16;                    // warps per tile
  constexpr int TPB = (kThreads / 32) / WPT;     // tiles per CTA (1 for D=128, 2 for D=64)
  const int warp = t >> 5, lane = t & 31;
  const int tl = warp / WPT;                     // tile slot inside this CTA
  const int64_t gt = (int64_t)bid * TPB + tl;    // global tile index over (b, h, tile)
  const int64_t total = (int64_t)P.B * P.Hkv * P.Tk;
  for (int i = t; i < 2048 / 16; i += kThreads) reinterpret_cast<uint4*>(sf_smem)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (gt < total) {
    const int tile = (int)(gt % P.Tk), bh = (int)(gt / P.Tk), b = bh / P.Hkv, h = bh % P.Hkv;
    const int c4 = (warp % WPT) * 4 + (lane >> 3);        // group of 4 channels
    const int blk = lane & 7;                              // 16-token block
    const __nv_bfloat16* src = P.v + (P.cu_k ? (int64_t)P.cu_k[b] * P.v_sn : b * P.v_sb) + h * P.v_sh + c4 * 4;
    const int Nv = P.cu_k ? min(P.cu_k[b + 1] - P.cu_k[b], P.Nk) : P.Nk;
    uint2 x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int n = tile * kTile + blk * 16 + i;
      x[i] = (n < Nv && c4 * 4 < P.d_in) ? *reinterpret_cast<const uint2*>(src + (int64_t)n * P.v_sn) : make_uint2(0, 0);
    }
    uint8_t* codes = P.vt_codes + gt * (D * 64);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        uint32_t wv = (j < 2) ? x[i].x : x[i].y;
        f[i] = (j & 1) ? bf16_hi(wv) : bf16_lo(wv);
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
      uint32_t sfb; float inv;
      block_scale(amax, sfb, inv);
      uint2 o;
      o.x = f32x8_to_e2m1x8(mul_ftz(f[0], inv), mul_ftz(f[1], inv), mul_ftz(f[2], inv), mul_ftz(f[3], inv),
                            mul_ftz(f[4], inv), mul_ftz(f[5], inv), mul_ftz(f[6], inv), mul_ftz(f[7], inv));
      o.y = f32x8_to_e2m1x8(mul_ftz(f[8], inv), mul_ftz(f[9], inv), mul_ftz(f[10], inv), mul_ftz(f[11], inv),
                            mul_ftz(f[12], inv), mul_ftz(f[13], inv), mul_ftz(f[14], inv), mul_ftz(f[15], inv));
      const int d = c4 * 4 + j;
      *reinterpret_cast<uint2*>(codes + d * 64 + blk * 8) = o;
      sf_smem[tl * 1024 + (blk >> 2) * 512 + sf_atom_offset(d, blk & 3)] = (uint8_t)sfb;
    }
  }
  __syncthreads();
  // each tile's 1 KB of scales leaves as 64 x 16 bytes
  {
    const int slot = t / 64, vec = t % 64;
    const int64_t g2 = (int64_t)bid * TPB + slot;
    if (slot < TPB && g2 < total)
      reinterpret_cast<uint4*>(P.vt_sf + g2 * 1024)[vec] = reinterpret_cast<const uint4*>(sf_smem + slot * 1024)[vec];
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static int pick_chunk_tokens(int N, int BH) {
  // enough CTAs (8 per SM on 148 SMs) to keep the memory system full, but at most 64 partial rows per (b,h)
  int chunk = 4096;
  while (chunk > 256 && (int64_t)BH * ((N + chunk - 1) / chunk) < 1184) chunk >>= 1;
  while ((N + chunk - 1) / chunk > 64) chunk <<= 1;
  return chunk;
}

size_t quant_scratch_bytes(int B, int H, int N, int D) {
  int chunk = pick_chunk_tokens(N, B * H);
  int nchunks = (N + chunk - 1) / chunk;
  size_t part = (size_t)B * H * nchunks * D * sizeof(float);
  part = (part + 255) & ~(size_t)255;
  return part + (size_t)B * H * sizeof(unsigned int);
}

cudaError_t launch_channel_mean(const void* x, int64_t sb, int64_t sh, int64_t sn, int B, int H, int N, int D,
                                float divisor, void* scratch, void* mean_out, cudaStream_t stream, const int* cu,
                                int d_in) {
  if (d_in <= 0 || d_in > D) d_in = D;
  int chunk = pick_chunk_tokens(N, B * H);
  int nchunks = (N + chunk - 1) / chunk;
  size_t part = (size_t)B * H * nchunks * D * sizeof(float);
  part = (part + 255) & ~(size_t)255;
  float* partial = reinterpret_cast<float*>(scratch);
  unsigned int* counters = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(scratch) + part);
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)B * H * sizeof(unsigned int), stream);
  if (e != cudaSuccess) return e;
  dim3 grid(nchunks, B * H);
  if (D == 128)
    channel_mean_kernel<128><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, sb, sh, sn, H, N, chunk, divisor,
                                                            partial, counters, (__nv_bfloat16*)mean_out, cu, d_in);
  else
    channel_mean_kernel<64><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, sb, sh, sn, H, N, chunk, divisor,
                                                           partial, counters, (__nv_bfloat16*)mean_out, cu, d_in);
  return cudaGetLastError();
}

cudaError_t launch_quant_qkv(const QuantArgs& a, cudaStream_t stream) {
  QuantLaunch P;
  P.q = (const __nv_bfloat16*)a.q; P.k = (const __nv_bfloat16*)a.k; P.v = (const __nv_bfloat16*)a.v;
  P.q_sb = a.q_sb; P.q_sh = a.q_sh; P.q_sn = a.q_sn;
  P.k_sb = a.k_sb; P.k_sh = a.k_sh; P.k_sn = a.k_sn;
  P.v_sb = a.v_sb; P.v_sh = a.v_sh; P.v_sn = a.v_sn;
  P.B = a.B; P.Hq = a.Hq; P.Hkv = a.Hkv; P.Nq = a.Nq; P.Nk = a.Nk;
  P.Tq = (a.Nq + kTile - 1) / kTile; P.Tk = (a.Nk + kTile - 1) / kTile;
  P.q_mean_mode = a.q_mean_mode;
  P.km = (const __nv_bfloat16*)a.km; P.q_mean_seq = (const __nv_bfloat16*)a.q_mean_seq;
  P.qm_override = (const float*)a.qm_override;
  P.q_codes = (uint8_t*)a.q_codes; P.q_sf = (uint8_t*)a.q_sf;
  P.k_codes = (uint8_t*)a.k_codes; P.k_sf = (uint8_t*)a.k_sf;
  P.vt_codes = (uint8_t*)a.vt_codes; P.vt_sf = (uint8_t*)a.vt_sf;
  P.qm = (__nv_bfloat16*)a.qm;
  P.cu_q = a.cu_q; P.cu_k = a.cu_k;
  P.d_in = (a.d_in > 0 && a.d_in <= a.D) ? a.d_in : a.D;
  P.q_dot_km = (a.q_dot_km != nullptr && a.km != nullptr && a.cu_q == nullptr) ? (float*)a.q_dot_km : nullptr;
  P.km_for_q = (const __nv_bfloat16*)a.km;
  P.q_blocks = a.q ? a.B * a.Hq * P.Tq : 0;
  P.k_blocks = a.k ? a.B * a.Hkv * P.Tk : 0;
  const int tpb = a.D == 128 ? 1 : 2;
  P.v_blocks = a.v ? (int)(((int64_t)a.B * a.Hkv * P.Tk + tpb - 1) / tpb) : 0;
  const int grid = P.q_blocks + P.k_blocks + P.v_blocks;
  if (grid == 0) return cudaSuccess;
  if (a.D == 128) quant_qkv_kernel<128><<<grid, kThreads, 0, stream>>>(P);
  else            quant_qkv_kernel<64><<<grid, kThreads, 0, stream>>>(P);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Channel means with the reduction scratch inside the library.
//
// Some hosts of this library may not call cudaMalloc at the point where they need the K means: an
// inference server that handed all device memory to its own pool at start-up, or a plug-in hook that
// runs where an allocation (which synchronises the device and can fail under memory pressure) is not
// acceptable.  For them the partial sums and arrival counters of channel_mean_kernel live in the
// fixed array below instead of a caller buffer.  Every GPU that loads the library holds the array
// (1 MiB + 8 KiB) until the process exits.
//
// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the address
// on the current device comes from cudaGetSymbolAddress, once per device, on the first call made
// with that device current.
// ------------------------------------------------------------------------------------------------
constexpr int kStaticMaxRows = 2048;                                   // partial rows: B * H * chunks
constexpr int kStaticMaxHeads = 2048;                                  // arrival counters: B * H
constexpr size_t kStaticPartialBytes = (size_t)kStaticMaxRows * 128 * sizeof(float);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialBytes + kStaticMaxHeads * sizeof(unsigned int)];

cudaError_t launch_channel_mean_static(const void* x, int64_t sb, int64_t sh, int64_t sn, int B, int H, int N, int D,
                                       float divisor, void* mean_out, cudaStream_t stream, bool* too_large) {
  *too_large = false;
  const int chunk = pick_chunk_tokens(N, B * H);
  const int nchunks = (N + chunk - 1) / chunk;
  if ((int64_t)B * H * nchunks > kStaticMaxRows || (int64_t)B * H > kStaticMaxHeads) {
    *too_large = true;
    return cudaSuccess;
  }
  static void* base_of_device[64] = {};                                // device ordinal -> address of the array there
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  void* base = __atomic_load_n(&base_of_device[dev], __ATOMIC_ACQUIRE);
  if (base == nullptr) {
    e = cudaGetSymbolAddress(&base, g_static_scratch);
    if (e != cudaSuccess) return e;
    __atomic_store_n(&base_of_device[dev], base, __ATOMIC_RELEASE);    // same value whoever stores first
  }
  float* partial = reinterpret_cast<float*>(base);
  unsigned int* counters = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(base) + kStaticPartialBytes);
  // The array keeps whatever the previous call left.  Partial rows are fully overwritten before they
  // are read; only the arrival counters must start at zero.
  e = cudaMemsetAsync(counters, 0, (size_t)B * H * sizeof(unsigned int), stream);
  if (e != cudaSuccess) return e;
  dim3 grid(nchunks, B * H);
  if (D == 128)
    channel_mean_kernel<128><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, sb, sh, sn, H, N, chunk, divisor,
                                                            partial, counters, (__nv_bfloat16*)mean_out, nullptr, D);
  else
    channel_mean_kernel<64><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, sb, sh, sn, H, N, chunk, divisor,
                                                           partial, counters, (__nv_bfloat16*)mean_out, nullptr, D);
  return cudaGetLastError();
}

}  // namespace sage3
