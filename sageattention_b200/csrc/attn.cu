// FP4 (NVFP4 block-scaled) flash-attention forward for B200 (sm_100a): TMA -> shared memory ->
// tcgen05.mma kind::mxf4nvf4 with accumulators in tensor memory -> online softmax in registers
// with two-level FP4 re-quantisation of P -> second block-scaled MMA for P.V.
//
// Replaces the reference's sm_120-only mma.sync kernel (sageattn4/blackwell/fwd_kernel.cu:45-200,
// fwd_mainloop.cu:639-1125, softmax_fused.h:39-187, fwd_epilogue.cu:30-183) and its host launcher
// (fwd_kernel.cu:202-293).  Arithmetic follows the reference step by step:
//   S = delta_s + Q^ K^T                              fwd_mainloop.cu:766-794, 908-919
//   masks (key padding, bottom-right causal)          fwd_mainloop.cu:921-964
//   online softmax with P in (0, 448*6], per-16-key scale = blockmax/6 stored as E4M3, P/scale
//   stored as E2M1                                    softmax_fused.h:107-153, fwd_mainloop.cu:967-1002
//   O = O * alpha + P^ V^ with a fresh accumulator per key tile     softmax_fused.h:175-187
//   O /= l, bf16                                      softmax_fused.h:156-173, fwd_epilogue.cu:103-147
// Key tiles are visited from the last to the first as the reference does (fwd_mainloop.cu:575).
//
// CTA = one 128-row query tile of one head.  8 warps:
//   warps 0-3  softmax: thread r owns score row r (tensor-memory lane r) and the O row in registers
//   warp  4    TMA producer (Q once, then a ring of K / V stages; scale factors and the delta_s
//              row by plain bulk copies)
//   warp  5    MMA issuer (one elected lane): tcgen05.cp of scale factors, 2x QK MMA, 2x PV MMA
//   warps 6-7  idle (they keep the softmax warps a whole warpgroup for setmaxnreg)
// Two CTAs are resident per SM: while one waits for its MMAs the other runs softmax.
//
// Tensor memory (256 columns per CTA): [0,128) scores S, [128,128+D) the per-tile P.V product.
// The scale factors of the QK MMA live in the first 16 columns of the P.V region and those of the
// PV MMA in the first 16 columns of the S region; the issue order makes that safe (QK of tile j+1
// is issued only after the softmax warps have drained the P.V product of tile j, and PV of tile j
// only after they have consumed S of tile j).
//
// Every wait on an mbarrier is bounded; if one gives up the CTA records a code in *status and
// runs to its end without further waiting, so a mistake cannot hang the GPU.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace sage3 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kStages = 3;
constexpr int kAttnThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLog2Inv2688 = -11.392317422778762f;   // log2(1 / (448 * 6))  softmax_fused.h:33
constexpr float kLog2Inv6 = -2.584962500721156f;       // log2(1 / 6)          softmax_fused.h:34

template <int D>
struct Smem {
  static constexpr int kQBytes = kBlockM * D / 2;
  static constexpr int kKBytes = kBlockN * D / 2;
  static constexpr int kVBytes = D * kBlockN / 2;
  static constexpr int kSfRow = (D / 64) * 512;         // Q / K scales per tile
  static constexpr int kSfV = 1024;                      // V^T scales per tile
  // offsets (all 1024-byte aligned tiles first)
  static constexpr int q = 0;
  static constexpr int k = q + kQBytes;
  static constexpr int v = k + kStages * kKBytes;
  static constexpr int p = v + kStages * kVBytes;        // P^ codes, 128 rows x 64 bytes
  static constexpr int sfq = p + kBlockM * kBlockN / 2;
  static constexpr int sfk = sfq + 1024;
  static constexpr int sfv = sfk + kStages * 1024;
  static constexpr int sfp = sfv + kStages * 1024;
  static constexpr int ds = sfp + 1024;                  // delta_s rows, 128 fp32 per stage
  static constexpr int bars = ds + kStages * 512;
  static constexpr int total = bars + 256;
};

struct Bars {            // byte offsets inside the barrier block
  static constexpr int q_full = 0;
  static constexpr int k_full = 8;                       // [kStages]
  static constexpr int k_empty = k_full + 8 * kStages;
  static constexpr int v_full = k_empty + 8 * kStages;
  static constexpr int v_empty = v_full + 8 * kStages;
  static constexpr int s_full = v_empty + 8 * kStages;
  static constexpr int p_full = s_full + 8;
  static constexpr int o_full = p_full + 8;
  static constexpr int o_free = o_full + 8;
  static constexpr int drain = o_free + 8;               // MMA warp's last commit when giving up
  static constexpr int tmem_slot = drain + 8;            // u32 written by tcgen05.alloc
  static constexpr int abort_flag = tmem_slot + 8;
  static constexpr int run_flag = abort_flag + 4;
};

struct KParams {
  const uint8_t *q_sf, *k_sf, *vt_sf;
  const float* ds;
  __nv_bfloat16* out;
  float* lse;
  int* status;
  int64_t o_sb, o_sh, o_sn;
  int B, Hq, Hkv, Nq, Nk, Tq, Tk, ds_rows;
  float scale_log2;      // sm_scale * log2(e)
};

// wait with a poll limit; also gives up as soon as any CTA has reported a failure
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_s, int* status, int code) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && (*abort_s != 0 || *reinterpret_cast<volatile int*>(status) != 0)) break;
  }
  *abort_s = 1;
  atomicCAS(status, 0, code);
  return false;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

template <int D, bool kCausal>
__global__ void __launch_bounds__(kAttnThreads, 2) attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                   const __grid_constant__ CUtensorMap tm_k,
                                                                   const __grid_constant__ CUtensorMap tm_v,
                                                                   const KParams P) {
  using L = Smem<D>;
  constexpr int kKB = D / 64;                              // K=64 blocks of the QK contraction
  constexpr uint32_t kSwzQK = (D == 128) ? 4u : 6u;        // 64-byte / 32-byte swizzle
  constexpr uint32_t kSboQK = (D == 128) ? 512u : 256u;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles need 1024-byte alignment
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + L::bars;
  volatile int* abort_s = reinterpret_cast<volatile int*>(smem + L::bars + Bars::abort_flag);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // tile coordinates: query tiles of one head are adjacent in the grid (they share K/V in L2);
  // the longest causal tiles start first
  const int bid = blockIdx.x;
  const int qt = P.Tq - 1 - (bid % P.Tq);
  const int bh = bid / P.Tq, b = bh / P.Hq, hq = bh % P.Hq;
  const int hkv = hq / (P.Hq / P.Hkv);
  const int q0 = qt * kBlockM;

  int n_tiles = P.Tk;
  if (kCausal) {
    const int q_end = min(q0 + kBlockM, P.Nq);
    const int lim = q_end + P.Nk - P.Nq;                   // keys [0, lim) can be visible
    n_tiles = lim <= 0 ? 0 : min(P.Tk, (lim + kBlockN - 1) / kBlockN);
  }

  if (threadIdx.x == 0) {
    mbar_init(bars + Bars::q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bars + Bars::k_full + 8 * s, 1);
      mbar_init(bars + Bars::k_empty + 8 * s, 4);          // one lane of each softmax warp
      mbar_init(bars + Bars::v_full + 8 * s, 1);
      mbar_init(bars + Bars::v_empty + 8 * s, 1);          // tcgen05.commit
    }
    mbar_init(bars + Bars::s_full, 1);
    mbar_init(bars + Bars::p_full, 128);
    mbar_init(bars + Bars::o_full, 1);
    mbar_init(bars + Bars::o_free, 128);
    mbar_init(bars + Bars::drain, 1);
    // a failure reported by an earlier CTA (or an earlier launch that shares *status) stops new work
    const int bad = *reinterpret_cast<volatile int*>(P.status) != 0;
    *abort_s = bad;
    *reinterpret_cast<volatile int*>(smem + L::bars + Bars::run_flag) = !bad;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(bars + Bars::tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + L::bars + Bars::tmem_slot);
  const uint32_t tm_S = tmem, tm_O = tmem + 128;
  const uint32_t tm_sfq = tm_O, tm_sfk = tm_O + 8;        // QK scales: inside the P.V region
  const uint32_t tm_sfp = tm_S, tm_sfv = tm_S + 8;        // PV scales: inside the S region

  // read once after the barrier: every warp takes the same branch, so the register hand-over
  // below (setmaxnreg) is always executed by whole warpgroups
  const bool run = *reinterpret_cast<volatile int*>(smem + L::bars + Bars::run_flag) != 0;
  if (n_tiles > 0 && run) {
    if (warp == 4) {
      // ------------------------------------------------------------------ TMA producer
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
      if (lane == 0) {
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
        const int64_t qtile = ((int64_t)b * P.Hq + hq) * P.Tq + qt;
        mbar_arrive_expect_tx(bars + Bars::q_full, L::kQBytes + L::kSfRow);
        tma_load_2d(sbase + L::q, &tm_q, 0, (int)(qtile * kBlockM), bars + Bars::q_full);
        bulk_load(sbase + L::sfq, P.q_sf + qtile * L::kSfRow, L::kSfRow, bars + Bars::q_full);
        const int64_t kvhead = ((int64_t)b * P.Hkv + hkv) * P.Tk;
        const int64_t ds_row = ((int64_t)b * P.Hq + hq) * P.ds_rows + (P.ds_rows == 1 ? 0 : qt);
        int issued = 0;
        for (int it = 0; it < n_tiles; ++it) {
          const int j = n_tiles - 1 - it, s = it % kStages;
          const uint32_t ph = ((it / kStages) & 1) ^ 1;
          if (!wait_bar(bars + Bars::k_empty + 8 * s, ph, abort_s, P.status, 10)) break;
          const uint32_t kb = bars + Bars::k_full + 8 * s;
          mbar_arrive_expect_tx(kb, L::kKBytes + L::kSfRow + (P.ds ? 512 : 0));
          tma_load_2d(sbase + L::k + s * L::kKBytes, &tm_k, 0, (int)((kvhead + j) * kBlockN), kb);
          bulk_load(sbase + L::sfk + s * 1024, P.k_sf + (kvhead + j) * L::kSfRow, L::kSfRow, kb);
          if (P.ds) bulk_load(sbase + L::ds + s * 512, P.ds + (ds_row * P.Tk + j) * kBlockN, 512, kb);
          if (!wait_bar(bars + Bars::v_empty + 8 * s, ph, abort_s, P.status, 11)) break;
          const uint32_t vb = bars + Bars::v_full + 8 * s;
          mbar_arrive_expect_tx(vb, L::kVBytes + L::kSfV);
          tma_load_2d(sbase + L::v + s * L::kVBytes, &tm_v, 0, (int)((kvhead + j) * D), vb);
          bulk_load(sbase + L::sfv + s * 1024, P.vt_sf + (kvhead + j) * L::kSfV, L::kSfV, vb);
          ++issued;
        }
        if (*abort_s) {
          // giving up: the copies this thread started must land before the CTA may exit
          mbar_wait(bars + Bars::q_full, 0, 1u << 20);
          for (int it = max(0, issued - kStages); it < issued; ++it) {
            mbar_wait(bars + Bars::k_full + 8 * (it % kStages), (it / kStages) & 1, 1u << 20);
            mbar_wait(bars + Bars::v_full + 8 * (it % kStages), (it / kStages) & 1, 1u << 20);
          }
        }
      }
    } else if (warp == 5) {
      // ------------------------------------------------------------------ MMA issuer
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
      if (lane == 0) {
        constexpr uint32_t idesc_qk = make_idesc_nvf4(kBlockM, kBlockN);
        constexpr uint32_t idesc_pv = make_idesc_nvf4(kBlockM, D);
        bool ok = wait_bar(bars + Bars::q_full, 0, abort_s, P.status, 20);
        for (int it = 0; ok && it < n_tiles; ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          // S = Q K^T
          if (!(ok = wait_bar(bars + Bars::k_full + 8 * s, ph, abort_s, P.status, 21))) break;
          if (it > 0 && !(ok = wait_bar(bars + Bars::o_free, (it - 1) & 1, abort_s, P.status, 22))) break;
          tc_fence_after();
#pragma unroll
          for (int kb = 0; kb < kKB; ++kb) {
            tc_cp_sf(tm_sfq + 4 * kb, make_smem_desc(sbase + L::sfq + kb * 512, 128, 0, 0));
            tc_cp_sf(tm_sfk + 4 * kb, make_smem_desc(sbase + L::sfk + s * 1024 + kb * 512, 128, 0, 0));
          }
#pragma unroll
          for (int kb = 0; kb < kKB; ++kb) {
            const uint64_t da = make_smem_desc(sbase + L::q + kb * 32, kSboQK, 16, kSwzQK);
            const uint64_t db = make_smem_desc(sbase + L::k + s * L::kKBytes + kb * 32, kSboQK, 16, kSwzQK);
            tc_mma_nvf4(tm_S, da, db, idesc_qk, tm_sfq + 4 * kb, tm_sfk + 4 * kb, kb > 0);
          }
          tc_commit(bars + Bars::s_full);
          // O_tile = P V
          if (!(ok = wait_bar(bars + Bars::p_full, it & 1, abort_s, P.status, 23))) break;
          if (!(ok = wait_bar(bars + Bars::v_full + 8 * s, ph, abort_s, P.status, 24))) break;
          tc_fence_after();
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            tc_cp_sf(tm_sfp + 4 * kb, make_smem_desc(sbase + L::sfp + kb * 512, 128, 0, 0));
            tc_cp_sf(tm_sfv + 4 * kb, make_smem_desc(sbase + L::sfv + s * 1024 + kb * 512, 128, 0, 0));
          }
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            const uint64_t da = make_smem_desc(sbase + L::p + kb * 32, 512, 16, 4);
            const uint64_t db = make_smem_desc(sbase + L::v + s * L::kVBytes + kb * 32, 512, 16, 4);
            tc_mma_nvf4(tm_O, da, db, idesc_pv, tm_sfp + 4 * kb, tm_sfv + 4 * kb, kb > 0);
          }
          tc_commit(bars + Bars::v_empty + 8 * s);
          tc_commit(bars + Bars::o_full);
        }
        if (!ok) {
          // giving up: let every MMA / scale copy already issued finish before tensor memory is freed
          tc_commit(bars + Bars::drain);
          mbar_wait(bars + Bars::drain, 0, 1u << 20);
        }
      }
    } else if (warp < 4) {
      // ------------------------------------------------------------------ softmax + O accumulation
      asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
      const int row = threadIdx.x;                               // 0..127 = tensor-memory lane
      const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
      const int qpos = q0 + row;
      const int causal_lim = kCausal ? qpos + P.Nk - P.Nq : 0x7fffffff;   // last visible key
      const int key_lim = min(P.Nk - 1, causal_lim);
      const float c = P.scale_log2;
      float O[D];
#pragma unroll
      for (int i = 0; i < D; ++i) O[i] = 0.f;
      float m = -INFINITY, l = 0.f;
      uint8_t* p_row = smem + L::p + row * 64;
      const int swz = (row >> 1) & 3;
      uint32_t* sfp_row = reinterpret_cast<uint32_t*>(smem + L::sfp + sf_atom_offset(row, 0));
      bool ok = true;

      for (int it = 0; it < n_tiles; ++it) {
        const int j = n_tiles - 1 - it, s = it % kStages;
        const int n0 = j * kBlockN;
        const bool need_mask = (n0 + kBlockN - 1 >= P.Nk) || (kCausal && n0 + kBlockN - 1 > q0 + P.Nk - P.Nq);
        if (!(ok = wait_bar(bars + Bars::s_full, it & 1, abort_s, P.status, 30))) break;
        tc_fence_after();
        const float4* dsv = reinterpret_cast<const float4*>(smem + L::ds + s * 512);
        const bool has_ds = P.ds != nullptr;

        // ---- pass 1: per-16-key block maxima of t = S*c + ds
        float bm[8];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          tmem_ld32(tm_S + lane_addr + ch * 32, r);
          tmem_wait_ld();
          float t[32];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 d4 = has_ds ? dsv[ch * 8 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
            t[4 * i + 0] = fmaf(__uint_as_float(r[4 * i + 0]), c, d4.x);
            t[4 * i + 1] = fmaf(__uint_as_float(r[4 * i + 1]), c, d4.y);
            t[4 * i + 2] = fmaf(__uint_as_float(r[4 * i + 2]), c, d4.z);
            t[4 * i + 3] = fmaf(__uint_as_float(r[4 * i + 3]), c, d4.w);
          }
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + ch * 32 + i > key_lim) t[i] = -INFINITY;
          }
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            float a = fmax3(t[hb * 16 + 0], t[hb * 16 + 1], t[hb * 16 + 2]);
            float b2 = fmax3(t[hb * 16 + 3], t[hb * 16 + 4], t[hb * 16 + 5]);
            float c2 = fmax3(t[hb * 16 + 6], t[hb * 16 + 7], t[hb * 16 + 8]);
            float d2 = fmax3(t[hb * 16 + 9], t[hb * 16 + 10], t[hb * 16 + 11]);
            float e2 = fmax3(t[hb * 16 + 12], t[hb * 16 + 13], t[hb * 16 + 14]);
            bm[ch * 2 + hb] = fmaxf(fmax3(a, b2, c2), fmax3(d2, e2, t[hb * 16 + 15]));
          }
        }
        const float m_new = fmaxf(fmaxf(fmax3(bm[0], bm[1], bm[2]), fmax3(bm[3], bm[4], bm[5])), fmax3(bm[6], bm[7], m));
        const float m_fin = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = ex2_approx(m - m_fin);                 // 0 on the first tile
        const float off = m_fin + kLog2Inv2688;                    // P = 2^(t - off) in (0, 2688]
        m = m_new;
        // per-block scale (P blockmax / 6) and the exponent offset that yields P / scale directly
        float sb[8], boff[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          sb[i] = ex2_approx(bm[i] - off + kLog2Inv6);
          boff[i] = (bm[i] == -INFINITY) ? 0.f : bm[i] + kLog2Inv6;
        }
        sfp_row[0] = f32x2_to_e4m3x2(sb[0], sb[1]) | (f32x2_to_e4m3x2(sb[2], sb[3]) << 16);
        sfp_row[128] = f32x2_to_e4m3x2(sb[4], sb[5]) | (f32x2_to_e4m3x2(sb[6], sb[7]) << 16);

        // ---- pass 2: P / scale = 2^(t - boff) in [0, 6] -> E2M1; row sum from the unrounded values
        float lsum = 0.f;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          tmem_ld32(tm_S + lane_addr + ch * 32, r);
          tmem_wait_ld();
          uint32_t code[4];
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            float pn[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float4 d4 = has_ds ? dsv[ch * 8 + hb * 4 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
              pn[4 * i + 0] = fmaf(__uint_as_float(r[hb * 16 + 4 * i + 0]), c, d4.x);
              pn[4 * i + 1] = fmaf(__uint_as_float(r[hb * 16 + 4 * i + 1]), c, d4.y);
              pn[4 * i + 2] = fmaf(__uint_as_float(r[hb * 16 + 4 * i + 2]), c, d4.z);
              pn[4 * i + 3] = fmaf(__uint_as_float(r[hb * 16 + 4 * i + 3]), c, d4.w);
            }
            if (need_mask) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n0 + ch * 32 + hb * 16 + i > key_lim) pn[i] = -INFINITY;
            }
            const float bo = boff[ch * 2 + hb];
            float bs = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              pn[i] = ex2_approx(pn[i] - bo);
              bs += pn[i];
            }
            lsum = fmaf(bs, sb[ch * 2 + hb], lsum);
            code[hb * 2 + 0] = f32x8_to_e2m1x8(pn[0], pn[1], pn[2], pn[3], pn[4], pn[5], pn[6], pn[7]);
            code[hb * 2 + 1] = f32x8_to_e2m1x8(pn[8], pn[9], pn[10], pn[11], pn[12], pn[13], pn[14], pn[15]);
          }
          *reinterpret_cast<uint4*>(p_row + ((ch ^ swz) << 4)) = make_uint4(code[0], code[1], code[2], code[3]);
        }
        l = fmaf(l, alpha, lsum);
        // S consumed and P^ written: hand both to the MMA warp, release the K stage (delta_s row)
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bars + Bars::p_full);
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + Bars::k_empty + 8 * s);

        // ---- O = O * alpha + P^ V^
        if (!(ok = wait_bar(bars + Bars::o_full, it & 1, abort_s, P.status, 31))) break;
        tc_fence_after();
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t r[32];
          tmem_ld32(tm_O + lane_addr + ch * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) O[ch * 32 + i] = fmaf(O[ch * 32 + i], alpha, __uint_as_float(r[i]));
        }
        tc_fence_before();
        mbar_arrive(bars + Bars::o_free);
      }

      // ---- epilogue: O / l -> bf16 -> global (row-contiguous 16-byte stores)
      if (ok && qpos < P.Nq) {
        const float inv = (l == 0.f || l != l) ? 0.f : 1.0f / l;
        __nv_bfloat16* orow = P.out + b * P.o_sb + hq * P.o_sh + (int64_t)qpos * P.o_sn;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          uint4 o;
          o.x = pack_bf16(O[8 * i + 0] * inv, O[8 * i + 1] * inv);
          o.y = pack_bf16(O[8 * i + 2] * inv, O[8 * i + 3] * inv);
          o.z = pack_bf16(O[8 * i + 4] * inv, O[8 * i + 5] * inv);
          o.w = pack_bf16(O[8 * i + 6] * inv, O[8 * i + 7] * inv);
          reinterpret_cast<uint4*>(orow)[i] = o;
        }
        if (P.lse) {
          // natural-log sum of exp(sm_scale * s) over the row (l carries the factor 2688)
          P.lse[((int64_t)b * P.Hq + hq) * P.Nq + qpos] =
              (l == 0.f) ? -INFINITY : (m + log2f(l) + kLog2Inv2688) * (1.0f / kLog2e);
        }
      }
    } else {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    }
  } else if (n_tiles == 0 && warp < 4) {
    // causal tile that sees no key at all: zeros, like the reference's store_zero (fwd_epilogue.cu:150-183)
    const int qpos = q0 + (int)threadIdx.x;
    if (qpos < P.Nq) {
      __nv_bfloat16* orow = P.out + b * P.o_sb + hq * P.o_sh + (int64_t)qpos * P.o_sn;
      for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0, 0, 0, 0);
      if (P.lse) P.lse[((int64_t)b * P.Hq + hq) * P.Nq + qpos] = INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------------------
// host: tensor maps + launch
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D byte tensor [rows][row_bytes], box = [box_rows][row_bytes]
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint32_t row_bytes, uint32_t box_rows,
              CUtensorMapSwizzle swz) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {row_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool kCausal>
cudaError_t launch(const AttnArgs& a, cudaStream_t stream) {
  using L = Smem<D>;
  const int Tq = (a.Nq + 127) / 128, Tk = (a.Nk + 127) / 128;
  CUtensorMap tq, tk, tv;
  const CUtensorMapSwizzle swz = D == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  if (!make_map(&tq, a.q_codes, (uint64_t)a.B * a.Hq * Tq * 128, D / 2, 128, swz)) return cudaErrorInvalidValue;
  if (!make_map(&tk, a.k_codes, (uint64_t)a.B * a.Hkv * Tk * 128, D / 2, 128, swz)) return cudaErrorInvalidValue;
  if (!make_map(&tv, a.vt_codes, (uint64_t)a.B * a.Hkv * Tk * D, 64, D, CU_TENSOR_MAP_SWIZZLE_64B))
    return cudaErrorInvalidValue;
  KParams P;
  P.q_sf = (const uint8_t*)a.q_sf; P.k_sf = (const uint8_t*)a.k_sf; P.vt_sf = (const uint8_t*)a.vt_sf;
  P.ds = (const float*)a.ds; P.out = (__nv_bfloat16*)a.out; P.lse = a.lse; P.status = a.status;
  P.o_sb = a.o_sb; P.o_sh = a.o_sh; P.o_sn = a.o_sn;
  P.B = a.B; P.Hq = a.Hq; P.Hkv = a.Hkv; P.Nq = a.Nq; P.Nk = a.Nk; P.Tq = Tq; P.Tk = Tk; P.ds_rows = a.ds_rows;
  P.scale_log2 = a.sm_scale * kLog2e;
  auto kern = attn_fwd_kernel<D, kCausal>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total + 1024);
  if (e != cudaSuccess) return e;
  const int64_t grid = (int64_t)a.B * a.Hq * Tq;
  kern<<<(unsigned)grid, kAttnThreads, L::total + 1024, stream>>>(tq, tk, tv, P);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.D == 128) return a.causal ? launch<128, true>(a, stream) : launch<128, false>(a, stream);
  if (a.D == 64) return a.causal ? launch<64, true>(a, stream) : launch<64, false>(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace sage3
