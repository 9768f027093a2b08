// FP4 (NVFP4 block-scaled) flash-attention forward for B200 (sm_100a): TMA -> shared memory ->
// tcgen05.mma kind::mxf4nvf4 with accumulators in tensor memory -> online softmax in registers
// with two-level FP4 re-quantisation of P -> second block-scaled MMA for P.V, accumulated in tensor memory.
//
// Replaces the reference's sm_120-only mma.sync kernel (sageattn4/blackwell/fwd_kernel.cu:45-200,
// fwd_mainloop.cu:639-1125, softmax_fused.h:39-187, fwd_epilogue.cu:30-183) and its host launcher
// (fwd_kernel.cu:202-293).  Arithmetic follows the reference step by step:
//   S = delta_s + Q^ K^T                              fwd_mainloop.cu:766-794, 908-919
//   masks (key padding, bottom-right causal)          fwd_mainloop.cu:921-964
//   online softmax, per-16-key scale = blockmax/6 stored as E4M3, P/scale stored as E2M1
//                                                     softmax_fused.h:107-153, fwd_mainloop.cu:967-1002
//   O = sum over key tiles of P^ V^, rescaled when the row maximum moves     softmax_fused.h:175-187
//   O /= l, bf16                                      softmax_fused.h:156-173, fwd_epilogue.cu:103-147
// Key tiles are visited from the last to the first as the reference does (fwd_mainloop.cu:575).
//
// O lives in tensor memory and the P.V MMAs accumulate into it (the reference keeps O in registers and adds a
// fresh product per key tile); like the reference it is multiplied by 2^((m_old - m_new) c) whenever a row's
// maximum has moved - here in place in tensor memory, and only by the warps in which some row's maximum did move,
// which after the first few key tiles of a long row is rare.  P, its block scales and the row sum are the
// reference's value for value (kLazyLog2 = 0).  A build with kLazyLog2 > 0 rescales only after the maximum has
// grown by more than 2^kLazyLog2 and normalises P to 2688 / 2^kLazyLog2 instead; the E4M3 rounding of the block
// scales then falls differently than in the reference (same size of error, different realisation), which
// measured 2.7-3.1 % relative L1 against the restatement of the reference - outside the 2 % parity bar - for a
// gain of a few percent, so it is not the default.
//
// One persistent CTA per SM walks a static list of work items (round r: item r*grid + i, odd rounds in
// reverse CTA order; causal items sorted by falling cost over all heads);
// an item is TWO adjacent 128-row query tiles of one head, which share every K / V tile.  All
// barrier phases keep counting across items, so the loads and the first Q.K^T of the next item are
// under way while the last softmax and the output store of the current one finish.  12 warps:
//   warps 0-3   softmax warpgroup of query tile 0: thread r owns score row r (tensor-memory lane r).  Per key
//               tile it copies its 128 scores from tensor memory into registers and releases the score buffer at
//               once (the Q.K^T of the other query tile is issued into it while this tile is worked on), then:
//               16-key block maxima, block scales, exponentials, E2M1 codes of P^ into tensor memory (the P.V MMA
//               takes its A operand from there; only the block scales go through shared memory).  It never
//               waits for the P.V product: the MMA accumulates into the tile's O in tensor memory.  At the end of
//               an item O / l goes out as bf16 (D=128: through a swizzled staging tile and TMA stores).
//   warps 4-7   the same for query tile 1; the two warpgroups settle half a period apart
//   warp  8     TMA producer (Q tiles per item, then a ring of K and V stages; scale factors and the
//               delta_s rows by plain bulk copies)
//   warp  9     QK issuer (one lane): scale-factor copies, rank-1 delta_s MMA and Q.K^T MMAs, both tiles in turn
//               into the ONE score buffer
//   warp 10     turns each delta_s row (128 bf16) into the B operand of a rank-1 bf16 MMA
//               (ones x delta_s) that initialises the score accumulator, so the softmax warps never
//               touch delta_s
//   warp 11     PV issuer (one lane): scale-factor copies and P.V MMAs, O_t += P^_t V^
//
// Tensor memory (512 columns): O0 [0,D) O1 [D,2D) S [2D,2D+128), 48 columns of scale factors, P^0 and P^1 (16
// columns each: 128 FP4 codes per row).
//
// Every wait on an mbarrier is bounded; if one gives up the CTA records a code in *status, waits
// (bounded) for its own copies and MMAs in flight, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

// This file is compiled twice: as it is for dense batches, and once more through attn_varlen.cu with
// SAGE3_VARLEN_BUILD = 1 for variable-length batches (per-sequence offsets and lengths from cu_seqlens).  The
// dense build sees exactly the code it had before the second one existed: the kernel is paced by its softmax
// warps and even dead extra code moved their register allocation and timing by a few percent.
#ifndef SAGE3_VARLEN_BUILD
#define SAGE3_VARLEN_BUILD 0
#endif
// lengths of the sequence a work item `wk` belongs to, inside the softmax warps
#if SAGE3_VARLEN_BUILD
#define SEQ_NQ wk.Nq
#define SEQ_NK wk.Nk
#define SEQ_NK_LOG wk.Nk
#define SEQ_TILE_EXISTS (q0 < wk.Nq)
#else
#define SEQ_NQ P.Nq
#define SEQ_NK P.Nk
#define SEQ_NK_LOG P.Nk_log
#define SEQ_TILE_EXISTS (qt < P.Tq)
#endif

namespace sage3 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
#ifndef SAGE3_STAGES
#define SAGE3_STAGES 3
#endif
constexpr int kStages = SAGE3_STAGES;                   // K / V ring depth
constexpr int kAttnThreads = 384;
// Register hand-over (setmaxnreg) moves registers inside the pool the CTA was LAUNCHED with; a request beyond
// it would block forever, so the split is checked here.  kLaunchRegs is what the compiler allocates under
// __launch_bounds__(384, 1).
constexpr int kLaunchRegs = 168;
#ifndef SAGE3_REGS_SOFTMAX
#define SAGE3_REGS_SOFTMAX 224
#define SAGE3_REGS_ROLE 56
#endif
template <int D> struct RegSplit { static constexpr int softmax = SAGE3_REGS_SOFTMAX, role = SAGE3_REGS_ROLE; };
static_assert(256 * RegSplit<128>::softmax + 128 * RegSplit<128>::role <= kAttnThreads * kLaunchRegs,
              "setmaxnreg split exceeds the CTA's register pool");
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLog2Inv2688 = -11.392317422778762f;   // log2(1 / (448 * 6))  softmax_fused.h:33
constexpr float kLog2Inv6 = -2.584962500721156f;       // log2(1 / 6)          softmax_fused.h:34
// O in tensor memory is rescaled when a row maximum has grown by more than this (log2 units of P) since the row's
// reference maximum was set; P is normalised to 2688 / 2^kLazyLog2 at the reference maximum so that it cannot
// exceed 2688 (block scale 448, the E4M3 maximum) before that happens.  0 = the reference's arithmetic.
#ifndef SAGE3_LAZY_LOG2
#define SAGE3_LAZY_LOG2 0
#endif
constexpr float kLazyLog2 = (float)SAGE3_LAZY_LOG2;
constexpr float kLog2InvTop = kLog2Inv2688 + kLazyLog2;

template <int D>
struct Smem {
  static constexpr int kQBytes = kBlockM * D / 2;
  static constexpr int kKBytes = kBlockN * D / 2;
  static constexpr int kVBytes = D * kBlockN / 2;
  static constexpr int kSfRow = (D / 64) * 512;          // Q / K scales per tile
  static constexpr int kSfV = 1024;                       // V^T scales per tile
  static constexpr int q = 0;                             // [2]
  static constexpr int k = q + 2 * kQBytes;               // [kStages]
  static constexpr int v = k + kStages * kKBytes;         // [kStages]
  static constexpr int sfq = v + kStages * kVBytes;       // [2][1024]
  static constexpr int sfk = sfq + 2 * 1024;              // [kStages][1024]
  static constexpr int sfv = sfk + kStages * 1024;        // [kStages][1024]
  static constexpr int sfp = sfv + kStages * 1024;        // [2][1024]
  static constexpr int a1 = sfp + 2 * 1024;               // rank-1 A operand: column 0 = 1.0 (bf16)
  static constexpr int b1 = a1 + 2048;                    // [kStages][2][2048] rank-1 B operands
  static constexpr int zero = b1 + kStages * 2 * 2048;    // second K chunk of every rank-1 operand; it must lie
                                                          // ABOVE them: the descriptor offset to it is unsigned
  static constexpr int dsraw = zero + 2048;               // [kStages][2][256] delta_s rows as loaded
  static constexpr int lam = dsraw + kStages * 2 * 256;   // [2 * kStages][128] f32: lambda of the key slots (K-packing
                                                          // mode), arrives with the K stage; twice as many slots as
                                                          // stages because the softmax reads it after the stage is freed
  static constexpr int bars = lam + 2 * kStages * 512;
  // output staging for the TMA store: [2 tiles][D/64 column halves][128 rows x 128 bytes], 128-byte swizzle
  static constexpr int kOStage = 128 * 128;
  static constexpr int ostage = (bars + 512 + 1023) / 1024 * 1024;
  static constexpr int total = ostage + ((!SAGE3_VARLEN_BUILD && D == 128) ? 2 * (D / 64) * kOStage : 0);
};

struct Bars {            // byte offsets inside the barrier block
  static constexpr int q_full = 0;                        // [2]
  static constexpr int q_empty = 16;                      // [2]
  static constexpr int k_full = 32;                       // [kStages]
  static constexpr int k_empty = k_full + 8 * kStages;
  static constexpr int v_full = k_empty + 8 * kStages;
  static constexpr int v_empty = v_full + 8 * kStages;
  static constexpr int ds_ready = v_empty + 8 * kStages;
  static constexpr int s_full = ds_ready + 8 * kStages;   // [2] Q.K^T of tile t is in the score buffer
  static constexpr int s_free = s_full + 16;              // the score buffer has been copied into registers
  static constexpr int p_full = s_free + 8;               // [2] P^ and its scales written (O rescaled if it had to be)
  static constexpr int pv_done = p_full + 16;             // [2] P.V MMAs of tile t complete: P^ may be rewritten, O_t is current
  static constexpr int o_free = pv_done + 16;             // [2] the epilogue has read O_t out of tensor memory
  static constexpr int drain = o_free + 16;               // [2] the issuers' last commit when giving up
  static constexpr int epi = drain + 16;                  // [2] rendezvous of a softmax warpgroup around its output staging
  static constexpr int tmem_slot = epi + 16;              // u32 written by tcgen05.alloc
  static constexpr int abort_flag = tmem_slot + 8;
  static constexpr int run_flag = abort_flag + 4;
};

struct KParams {
  const uint8_t *q_sf, *k_sf, *vt_sf;
  const __nv_bfloat16* ds;
  __nv_bfloat16* out;
  float* lse;
  const float* lse_add;  // optional [B,Hq,Nq]: sm_scale * lse_add is added to the LSE (K-mean term removed by smoothing)
  int* status;
  int64_t o_sb, o_sh, o_sn;
  int B, Hq, Hkv, Nq, Nk, Tq, Tk, ds_rows;
  float scale_log2;      // sm_scale * log2(e)
  const float* lam;      // K-packing mode: lambda per key slot, fp32 [B,Hkv,Tk*128]; Nk is the packed length
  int Nk_log;            // number of key tokens (= Nk unless packed)
  int d_out;             // columns the output rows really have (<= D, multiple of 8)
  bool slot_first;       // K-packing mode: the mean slot takes the first token's score instead of being masked
  bool o_token_first;    // output tensor map: coordinates (d, token, head, batch) or (d, head, token, batch)
#if SAGE3_VARLEN_BUILD
  const int *cu_q, *cu_k; // token offsets of the sequences (device int32 [B+1]); Nq, Nk, Tq, Tk then describe the
                          // LONGEST sequence, i.e. the rectangular operand layouts
#endif
};

// ---- packed fp32x2 arithmetic (one issue slot for two elements) and 3-input max
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)), "l"(reinterpret_cast<uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float max16(const uint32_t* r) {
  const float a = fmax3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
  const float b = fmax3(__uint_as_float(r[3]), __uint_as_float(r[4]), __uint_as_float(r[5]));
  const float c = fmax3(__uint_as_float(r[6]), __uint_as_float(r[7]), __uint_as_float(r[8]));
  const float d = fmax3(__uint_as_float(r[9]), __uint_as_float(r[10]), __uint_as_float(r[11]));
  const float e = fmax3(__uint_as_float(r[12]), __uint_as_float(r[13]), __uint_as_float(r[14]));
  return fmaxf(fmax3(a, b, c), fmax3(d, e, __uint_as_float(r[15])));
}

// The softmax of one key tile works on one score row (128 values) held in the registers of one thread; every
// loop below is fully unrolled so that the row never leaves the register file.

// K-packing mode (fwd_mainloop.cu:796-845, 878-881): a block of 16 keys is one group - slot 0 holds the
// score of the group mean, which every other score of the group gets added lambda times; the slot itself
// carries no token and is masked out.
__device__ __forceinline__ void apply_lambda(uint32_t* r, const float* lam16) {
  const float s0 = __uint_as_float(r[0]);
  const float2 s02 = make_float2(s0, s0);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 l4 = reinterpret_cast<const float4*>(lam16)[i];
    const float2 a = ffma2(make_float2(l4.x, l4.y), s02, make_float2(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1])));
    const float2 b = ffma2(make_float2(l4.z, l4.w), s02, make_float2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
    r[4 * i] = __float_as_uint(a.x); r[4 * i + 1] = __float_as_uint(a.y);
    r[4 * i + 2] = __float_as_uint(b.x); r[4 * i + 3] = __float_as_uint(b.y);
  }
  r[0] = 0xff800000u;
}

// 128 score columns of this thread's tensor-memory lane -> registers
__device__ __forceinline__ void load_scores(const uint32_t tm_S, uint32_t (&s)[128]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) tmem_ld32(tm_S + 32 * q, *reinterpret_cast<uint32_t (*)[32]>(&s[32 * q]));
  tmem_wait_ld();
}

// P / blockscale = 2^(s*c - (bm*c + log2(1/6))) in [0, 6] -> E2M1 codes into this row's 16 tensor-memory columns of
// P^ (8 codes per column, in key order - the A operand of the P.V MMA is read from there); returns the row sum of the unquantised P = sum over blocks of (sum of P/blockscale) * blockscale
// (softmax_fused.h:135-153).  neg_e[b] = -(bm_b*c + log2(1/6)), sb[b] = the block's unrounded scale.
// K-packing mode with slot_first: the first column of every block is the group's mean slot carrying a copy of the
// first token's score; its P^ goes to the MMA like any other, but it is no token and stays out of the row sum
// (softmax_fused.h:48-64).
template <bool kPacked>
__device__ __forceinline__ float exp_quantise_store(const uint32_t (&s)[128], const float c, const float (&neg_e)[8],
                                                    const float (&sb)[8], const uint32_t tm_P,
                                                    const bool slot_first) {
  const float2 c2 = make_float2(c, c);
  float lsum = 0.f;
  uint32_t code[4];
#pragma unroll
  for (int blk = 0; blk < 8; ++blk) {
    const float2 nb2 = make_float2(neg_e[blk], neg_e[blk]);
    float2 e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      e[i] = ffma2(make_float2(__uint_as_float(s[16 * blk + 2 * i]), __uint_as_float(s[16 * blk + 2 * i + 1])), c2, nb2);
      e[i].x = ex2_approx(e[i].x);
      e[i].y = ex2_approx(e[i].y);
    }
    const float2 s4 = fadd2(fadd2(fadd2(e[0], e[1]), fadd2(e[2], e[3])), fadd2(fadd2(e[4], e[5]), fadd2(e[6], e[7])));
    float bsum = s4.x + s4.y;
    if (kPacked && slot_first) bsum -= e[0].x;
    lsum = fmaf(bsum, sb[blk], lsum);
    code[(blk & 1) * 2 + 0] = f32x8_to_e2m1x8(e[0].x, e[0].y, e[1].x, e[1].y, e[2].x, e[2].y, e[3].x, e[3].y);
    code[(blk & 1) * 2 + 1] = f32x8_to_e2m1x8(e[4].x, e[4].y, e[5].x, e[5].y, e[6].x, e[6].y, e[7].x, e[7].y);
    if (blk & 1) tmem_st4(tm_P + 4 * (blk >> 1), code[0], code[1], code[2], code[3]);     // 32 keys = 4 columns
  }
  return lsum;
}

// K-packing mode: 15 tokens occupy 16 key slots (fwd_mainloop.cu:273-303).  Last slot that token `tok` or an
// earlier one occupies / number of slots the first `len` tokens occupy.
__device__ __forceinline__ int packed_slot_of_token(const int tok) { return (tok / 15) * 16 + tok % 15 + 1; }
__device__ __forceinline__ int packed_len_of(const int len) {
  return len <= 0 ? 0 : (len / 15) * 16 + (len % 15 == 0 ? 0 : len % 15 + 1);
}

// One unit of work of a CTA: two adjacent query tiles of one head.
struct Work {
  int b, hq, hkv, pair;
#if SAGE3_VARLEN_BUILD
  int Nq, Nk;            // lengths of this item's sequence
  int q_base;            // first token of the sequence in the packed output
#endif
  int n_t[2];            // key tiles each query tile visits (0: none / tile does not exist)
  int n_max;
};

// Static schedule: in round r CTA i takes item r*G + i, odd rounds in reverse CTA order, so a CTA that got
// the heaviest item of one round gets the lightest of the next.  Returns -1 when the CTA is done.
__device__ __forceinline__ int work_at(const int r, const int total) {
  const int G = (int)gridDim.x, i = (int)blockIdx.x;
  const int w = r * G + ((r & 1) ? G - 1 - i : i);
  return w < total ? w : -1;
}

template <bool kCausal, bool kPacked>
__device__ __forceinline__ Work get_work(const KParams& P, const int w) {
  Work k;
  const int n_pairs = (P.Tq + 1) >> 1;
  int bh;
  if (kCausal) {
    // item cost grows with the pair index: heaviest pairs of all heads first, so that the rounds of
    // the static schedule hand out work of falling, nearly equal cost
    const int n_bh = P.B * P.Hq;
    k.pair = n_pairs - 1 - w / n_bh;
    bh = w % n_bh;
  } else {
    // equal cost: keep the pairs of one head adjacent in time (they share K/V in L2)
    k.pair = n_pairs - 1 - (w % n_pairs);
    bh = w / n_pairs;
  }
  k.b = bh / P.Hq;
  k.hq = bh % P.Hq;
  k.hkv = k.hq / (P.Hq / P.Hkv);
#if SAGE3_VARLEN_BUILD
  k.q_base = P.cu_q[k.b];
  // a sequence longer than the caller's max_seqlen is cut there: the operand layouts (and the workspace) are
  // sized by max_seqlen, so tile indices beyond it must never be formed
  k.Nq = min(P.cu_q[k.b + 1] - k.q_base, P.Nq);
  k.Nk = min(P.cu_k[k.b + 1] - P.cu_k[k.b], P.Nk);
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt = 2 * k.pair + t;
    int n = 0;
    if (qt * kBlockM < k.Nq) {
      const int Tk = (k.Nk + kBlockN - 1) / kBlockN;
      n = Tk;
      if (kCausal) {
        const int q_end = min((qt + 1) * kBlockM, k.Nq);
        const int lim = q_end + k.Nk - k.Nq;               // key tokens [0, lim) can be visible
        n = lim <= 0 ? 0 : min(Tk, (lim + kBlockN - 1) / kBlockN);
      }
    }
    k.n_t[t] = n;
  }
#else
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt = 2 * k.pair + t;
    int n = 0;
    if (qt < P.Tq) {
      n = P.Tk;
      if (kCausal) {
        const int q_end = min((qt + 1) * kBlockM, P.Nq);
        int lim = q_end + P.Nk_log - P.Nq;                 // key tokens [0, lim) can be visible
        if (kPacked) lim = packed_len_of(lim);             // ... which occupy this many key slots
        n = lim <= 0 ? 0 : min(P.Tk, (lim + kBlockN - 1) / kBlockN);
      }
    }
    k.n_t[t] = n;
  }
#endif
  k.n_max = max(k.n_t[0], k.n_t[1]);
  return k;
}

template <int D, bool kCausal, bool kPacked>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                   const __grid_constant__ CUtensorMap tm_k,
                                                                   const __grid_constant__ CUtensorMap tm_v,
                                                                   const __grid_constant__ CUtensorMap tm_o,
                                                                   const KParams P) {
  using L = Smem<D>;
  constexpr int kKB = D / 64;                              // K=64 blocks of the QK contraction
  constexpr uint32_t kSwzQK = (D == 128) ? 4u : 6u;        // 64-byte / 32-byte swizzle
  constexpr uint32_t kSboQK = (D == 128) ? 512u : 256u;
  constexpr bool kTmaStore = !SAGE3_VARLEN_BUILD && D == 128;   // see the epilogue
  // How the two MMA issuer threads wait (measured, same box): the longer park of a hinted try_wait costs them a
  // little reaction time per key tile but leaves the sub-partition's issue slots to the softmax warp that shares it:
  // +9 % on rows of 256 key tiles, -2 to -4 % on rows of 8 to 64 (and D=64 gains at every length).
  const bool issuer_hint = (D == 64) || P.Tk >= 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles need 1024-byte alignment
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + L::bars;
  volatile int* abort_s = reinterpret_cast<volatile int*>(smem + L::bars + Bars::abort_flag);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool has_ds = P.ds != nullptr;
  const int total_work = P.B * P.Hq * ((P.Tq + 1) >> 1);

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(bars + Bars::q_full + 8 * t, 1);
      mbar_init(bars + Bars::q_empty + 8 * t, 1);          // tcgen05.commit after the last QK that reads the tile
      mbar_init(bars + Bars::s_full + 8 * t, 1);           // tcgen05.commit
      mbar_init(bars + Bars::p_full + 8 * t, 128);
      mbar_init(bars + Bars::pv_done + 8 * t, 1);          // tcgen05.commit
      mbar_init(bars + Bars::o_free + 8 * t, 128);
      mbar_init(bars + Bars::epi + 8 * t, 128);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bars + Bars::k_full + 8 * s, 1);
      mbar_init(bars + Bars::k_empty + 8 * s, 1);          // tcgen05.commit
      mbar_init(bars + Bars::v_full + 8 * s, 1);
      mbar_init(bars + Bars::v_empty + 8 * s, 1);          // tcgen05.commit
      mbar_init(bars + Bars::ds_ready + 8 * s, 1);
    }
    mbar_init(bars + Bars::s_free, 128);
    mbar_init(bars + Bars::drain, 1);
    mbar_init(bars + Bars::drain + 8, 1);
    // a failure reported by an earlier CTA (or an earlier launch that shares *status) stops new work
    const int bad = *reinterpret_cast<volatile int*>(P.status) != 0;
    *abort_s = bad;
    *reinterpret_cast<volatile int*>(smem + L::bars + Bars::run_flag) = !bad;
    fence_mbar_init();
  }
  // rank-1 operands: zero everything, then column 0 of A1 = 1.0
  for (int i = threadIdx.x; i < (L::dsraw - L::a1) / 16; i += kAttnThreads)
    reinterpret_cast<uint4*>(smem + L::a1)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 9) {
    tmem_alloc(bars + Bars::tmem_slot, 512);
    tmem_relinquish();
  }
  __syncthreads();
  if (threadIdx.x < 128)
    *reinterpret_cast<__nv_bfloat16*>(smem + L::a1 + (threadIdx.x >> 3) * 128 + (threadIdx.x & 7) * 16) =
        __float2bfloat16(1.0f);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + L::bars + Bars::tmem_slot);
  // columns: O0 [0, D)  O1 [D, 2D)  S [2D, 2D + 128)  scale factors behind
  const uint32_t tm_Sbuf = tmem + 2 * D;
  const uint32_t tm_sfq = tm_Sbuf + 128, tm_sfk = tm_sfq + 16, tm_sfp = tm_sfk + 8, tm_sfv = tm_sfp + 16;
  const uint32_t tm_P = tm_sfv + 8;                       // [2] P^ codes: the A operand of the P.V MMAs, 16 columns each

  // read once after the barrier: every warp takes the same branch, so the register hand-over
  // below (setmaxnreg) is always executed by whole warpgroups
  const bool run = *reinterpret_cast<volatile int*>(smem + L::bars + Bars::run_flag) != 0;
  // The CTA is persistent: every role walks the same static list of work items (blockIdx.x, +gridDim.x, ...)
  // and all barrier phases simply keep counting across items, so the loads, MMAs and softmax of the
  // next item start while the tail of the current one is still being finished.
  if (run) {
    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(RegSplit<D>::role));
      if (warp == 8 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_o);
        uint32_t g = 0;                       // K/V stages completely issued so far
        uint32_t gk = 0;                      // K stages issued so far (g or g + 1)
        uint32_t qn[2] = {0, 0};              // Q tiles loaded so far per slot
        bool ok = true;
        for (int r = 0, w; ok && (w = work_at(r, total_work)) >= 0; ++r) {
          const Work wk = get_work<kCausal, kPacked>(P, w);
          int64_t ds_row[2];
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int qt = 2 * wk.pair + t;
            ds_row[t] = ((int64_t)wk.b * P.Hq + wk.hq) * P.ds_rows + (P.ds_rows == 1 ? 0 : qt);
            if (ok && wk.n_t[t] > 0) {
              // the slot's previous Q tile must have been read by its last QK MMA
              if (qn[t] > 0 && !(ok = wait_bar<false>(bars + Bars::q_empty + 8 * t, (qn[t] - 1) & 1, abort_s, P.status, 12))) break;
              const int64_t qtile = ((int64_t)wk.b * P.Hq + wk.hq) * P.Tq + qt;
              const uint32_t qb = bars + Bars::q_full + 8 * t;
              mbar_arrive_expect_tx(qb, L::kQBytes + L::kSfRow);
              tma_load_2d(sbase + L::q + t * L::kQBytes, &tm_q, 0, (int)(qtile * kBlockM), qb);
              bulk_load(sbase + L::sfq + t * 1024, P.q_sf + qtile * L::kSfRow, L::kSfRow, qb);
              ++qn[t];
            }
          }
          const int64_t kvhead = ((int64_t)wk.b * P.Hkv + wk.hkv) * P.Tk;
          for (int it = 0; ok && it < wk.n_max; ++it, ++g) {
            const int j = wk.n_max - 1 - it, s = g % kStages;
            const uint32_t ph = ((g / kStages) & 1) ^ 1;
            if (!(ok = wait_bar<false>(bars + Bars::k_empty + 8 * s, ph, abort_s, P.status, 10))) break;
            const uint32_t kb = bars + Bars::k_full + 8 * s;
            const int nds = has_ds ? (int)(j < wk.n_t[0]) + (int)(j < wk.n_t[1]) : 0;
            mbar_arrive_expect_tx(kb, L::kKBytes + L::kSfRow + 256 * nds + (kPacked ? 512 : 0));
            if (kPacked) bulk_load(sbase + L::lam + (g % (2 * kStages)) * 512, P.lam + (kvhead + j) * kBlockN, 512, kb);
            tma_load_2d(sbase + L::k + s * L::kKBytes, &tm_k, 0, (int)((kvhead + j) * kBlockN), kb);
            bulk_load(sbase + L::sfk + s * 1024, P.k_sf + (kvhead + j) * L::kSfRow, L::kSfRow, kb);
            if (has_ds) {
#pragma unroll
              for (int t = 0; t < 2; ++t)
                if (j < wk.n_t[t])
                  bulk_load(sbase + L::dsraw + (s * 2 + t) * 256, P.ds + (ds_row[t] * P.Tk + j) * kBlockN, 256, kb);
            }
            ++gk;
            if (!(ok = wait_bar<false>(bars + Bars::v_empty + 8 * s, ph, abort_s, P.status, 11))) break;
            const uint32_t vb = bars + Bars::v_full + 8 * s;
            mbar_arrive_expect_tx(vb, L::kVBytes + L::kSfV);
            tma_load_2d(sbase + L::v + s * L::kVBytes, &tm_v, 0, (int)((kvhead + j) * D), vb);
            bulk_load(sbase + L::sfv + s * 1024, P.vt_sf + (kvhead + j) * L::kSfV, L::kSfV, vb);
          }
        }
        if (*abort_s) {
          // giving up: the copies this thread started must land before the CTA may exit
          for (int t = 0; t < 2; ++t)
            if (qn[t] > 0) mbar_wait(bars + Bars::q_full + 8 * t, (qn[t] - 1) & 1, 1u << 16);
          for (uint32_t i = (gk > (uint32_t)kStages ? gk - kStages : 0); i < gk; ++i)
            mbar_wait(bars + Bars::k_full + 8 * (i % kStages), (i / kStages) & 1, 1u << 16);
          for (uint32_t i = (g > (uint32_t)kStages ? g - kStages : 0); i < g; ++i)
            mbar_wait(bars + Bars::v_full + 8 * (i % kStages), (i / kStages) & 1, 1u << 16);
        }
      } else if (warp == 10 && has_ds) {
        // ---------------------------------------------------------------- delta_s -> rank-1 B operand
        // B1 is a K-major [128 keys x 16] bf16 operand in 8x16-byte core matrices: key n's first
        // element sits at (n/8)*128 + (n%8)*16; everything else stays zero.
        uint32_t g = 0;
        bool ok = true;
        for (int r = 0, w; ok && (w = work_at(r, total_work)) >= 0; ++r) {
          const Work wk = get_work<kCausal, kPacked>(P, w);
          for (int it = 0; ok && it < wk.n_max; ++it, ++g) {
            const int j = wk.n_max - 1 - it, s = g % kStages;
            if (!(ok = wait_bar<false>(bars + Bars::k_full + 8 * s, (g / kStages) & 1, abort_s, P.status, 40))) break;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (j < wk.n_t[t]) {
                const uint16_t* raw = reinterpret_cast<const uint16_t*>(smem + L::dsraw + (s * 2 + t) * 256);
                uint8_t* dst = smem + L::b1 + (s * 2 + t) * 2048 + (lane >> 3) * 128 + (lane & 7) * 16;   // keys lane + 32 i
#pragma unroll
                for (int i = 0; i < 4; ++i) *reinterpret_cast<uint16_t*>(dst + i * 512) = raw[lane + 32 * i];
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + Bars::ds_ready + 8 * s);
          }
        }
      } else if (warp == 9 && lane == 0) {
        // ---------------------------------------------------------------- QK issuer
        // This one thread paces the CTA, so its instruction stream is kept minimal: every shared-memory
        // descriptor is a constant high word (stride / swizzle / version bits) plus a low word
        // (address >> 4, leading-offset field) that only needs an integer add per use.
        constexpr uint32_t idesc_qk = make_idesc_nvf4(kBlockM, kBlockN);
        constexpr uint32_t idesc_r1 = make_idesc_bf16(kBlockM, kBlockN);
        constexpr uint32_t HI_QK = (kSboQK >> 4) | (1u << 14) | (kSwzQK << 29);
        constexpr uint32_t HI_SF = (128u >> 4) | (1u << 14);          // 8x16-byte core matrices, no swizzle
        constexpr uint32_t LBO1 = 1u << 16;                            // leading offset field of swizzled operands
        const uint32_t q_lo = ((sbase + L::q) >> 4) | LBO1, k_lo = ((sbase + L::k) >> 4) | LBO1;
        const uint32_t sfq_lo = (sbase + L::sfq) >> 4, sfk_lo = (sbase + L::sfk) >> 4;
        const uint32_t a1_lo = ((sbase + L::a1) >> 4) | (((uint32_t)(L::zero - L::a1) >> 4) << 16);
        const uint32_t b1_lo = ((sbase + L::b1) >> 4) | (((uint32_t)(L::zero - L::b1) >> 4) << 16);
        bool ok = true;
        uint32_t g = 0;                       // K stages consumed so far
        uint32_t nqk = 0;                     // QK groups issued so far (= uses of the score buffer)
        uint32_t qn[2] = {0, 0};              // Q tiles taken so far per slot
        for (int r = 0, w; ok && (w = work_at(r, total_work)) >= 0; ++r) {
          const Work wk = get_work<kCausal, kPacked>(P, w);
          for (int it = 0; ok && it < wk.n_max; ++it, ++g) {
            const int j = wk.n_max - 1 - it, s = g % kStages;
            const uint32_t ph = (g / kStages) & 1;
            if (!(ok = wait_bar_dyn(bars + Bars::k_full + 8 * s, ph, issuer_hint, abort_s, P.status, 21))) break;
            if (has_ds && !(ok = wait_bar_dyn(bars + Bars::ds_ready + 8 * s, ph, issuer_hint, abort_s, P.status, 25))) break;
            bool first = true;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (!ok || j >= wk.n_t[t]) continue;
              // the one score buffer must be free: the softmax warpgroup that got the previous Q.K^T (the other
              // query tile, or this one in the previous key tile) has copied it into registers
              if (nqk > 0 && !(ok = wait_bar_dyn(bars + Bars::s_free, (nqk - 1) & 1, issuer_hint, abort_s, P.status, 23))) break;
              if (it == wk.n_max - wk.n_t[t]) {                    // first key tile of this query tile
                if (!(ok = wait_bar_dyn(bars + Bars::q_full + 8 * t, qn[t] & 1, issuer_hint, abort_s, P.status, 20))) break;
                ++qn[t];
                tc_fence_after();
#pragma unroll
                for (int kb = 0; kb < kKB; ++kb) tc_cp_sf(tm_sfq + 8 * t + 4 * kb, sfq_lo + t * 64 + kb * 32, HI_SF);
              }
              tc_fence_after();
              if (first) {
                first = false;
#pragma unroll
                for (int kb = 0; kb < kKB; ++kb) tc_cp_sf(tm_sfk + 4 * kb, sfk_lo + s * 64 + kb * 32, HI_SF);
              }
              if (has_ds) {
                // buffer i sits i*2048 bytes higher, so its distance to the shared zero chunk is i*2048 smaller
                const uint32_t i = (uint32_t)(s * 2 + t);
                tc_mma_bf16(tm_Sbuf, a1_lo, HI_SF, b1_lo + i * 128u - ((i * 128u) << 16), HI_SF, idesc_r1, 0);
              }
#pragma unroll
              for (int kb = 0; kb < kKB; ++kb)
                tc_mma_nvf4(tm_Sbuf, q_lo + t * (L::kQBytes >> 4) + kb * 2, HI_QK, k_lo + s * (L::kKBytes >> 4) + kb * 2, HI_QK,
                            idesc_qk, tm_sfq + 8 * t + 4 * kb, tm_sfk + 4 * kb, (has_ds || kb > 0) ? 1u : 0u);
              tc_commit(bars + Bars::s_full + 8 * t);
              ++nqk;
              if (it == wk.n_max - 1) tc_commit(bars + Bars::q_empty + 8 * t);   // last read of this Q tile
            }
            if (ok) tc_commit(bars + Bars::k_empty + 8 * s);
          }
        }
        if (!ok) {
          // giving up: let every MMA / scale copy already issued finish before tensor memory is freed
          tc_commit(bars + Bars::drain);
          mbar_wait(bars + Bars::drain, 0, 1u << 16);
        }
      } else if (warp == 11 && lane == 0) {
        // ---------------------------------------------------------------- PV issuer
        // O_t += P^_t V^ for both tiles, from its own thread so that waiting for P^ never delays the next QK.
        // The first key tile of a work item overwrites O_t (no accumulate) - once the epilogue of the previous item
        // in that slot has read it out.
        constexpr uint32_t idesc_pv = make_idesc_nvf4(kBlockM, D);
        constexpr uint32_t HI_PV = (512u >> 4) | (1u << 14) | (4u << 29);
        constexpr uint32_t HI_SF = (128u >> 4) | (1u << 14);
        constexpr uint32_t LBO1 = 1u << 16;
        const uint32_t v_lo = ((sbase + L::v) >> 4) | LBO1;
        const uint32_t sfv_lo = (sbase + L::sfv) >> 4, sfp_lo = (sbase + L::sfp) >> 4;
        bool ok = true;
        uint32_t g = 0, pv_cnt[2] = {0, 0}, n_epi[2] = {0, 0};
        for (int r = 0, w; ok && (w = work_at(r, total_work)) >= 0; ++r) {
          const Work wk = get_work<kCausal, kPacked>(P, w);
          for (int it = 0; ok && it < wk.n_max; ++it, ++g) {
            const int j = wk.n_max - 1 - it, s = g % kStages;
            const bool act1 = j < wk.n_t[1];
            // the V stage and its scale factors do not depend on the softmax: fetch them before waiting for P
            if (!(ok = wait_bar_dyn(bars + Bars::v_full + 8 * s, (g / kStages) & 1, issuer_hint, abort_s, P.status, 24))) break;
            tc_fence_after();
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) tc_cp_sf(tm_sfv + 4 * kb, sfv_lo + s * 64 + kb * 32, HI_SF);
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const bool act = t == 0 ? (j < wk.n_t[0]) : act1;
              if (!(ok && act)) continue;
              const bool first_tile = it == wk.n_max - wk.n_t[t];
              if (!(ok = wait_bar_dyn(bars + Bars::p_full + 8 * t, pv_cnt[t] & 1, issuer_hint, abort_s, P.status, 26))) break;
              if (first_tile) {
                if (n_epi[t] > 0 && !(ok = wait_bar_dyn(bars + Bars::o_free + 8 * t, (n_epi[t] - 1) & 1, issuer_hint, abort_s, P.status, 22))) break;
                ++n_epi[t];
              }
              tc_fence_after();
#pragma unroll
              for (int kb = 0; kb < 2; ++kb) tc_cp_sf(tm_sfp + 8 * t + 4 * kb, sfp_lo + t * 64 + kb * 32, HI_SF);
#pragma unroll
              for (int kb = 0; kb < 2; ++kb)
                tc_mma_nvf4_ta(tmem + t * D, tm_P + 16 * t + 8 * kb, v_lo + s * (L::kVBytes >> 4) + kb * 2, HI_PV,
                               idesc_pv, tm_sfp + 8 * t + 4 * kb, tm_sfv + 4 * kb, (first_tile && kb == 0) ? 0u : 1u);
              tc_commit(bars + Bars::pv_done + 8 * t);
              ++pv_cnt[t];
              if (t == 1 || !act1) tc_commit(bars + Bars::v_empty + 8 * s);   // last PV of this stage
            }
          }
        }
        if (!ok) {
          tc_commit(bars + Bars::drain + 8);
          mbar_wait(bars + Bars::drain + 8, 0, 1u << 16);
        }
      }
    } else {
      // ------------------------------------------------------------------ softmax
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(RegSplit<D>::softmax));
      const int t = warp >> 2;                                   // query tile slot of this warpgroup
      const int row = threadIdx.x & 127;                         // tensor-memory lane
      const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
      const uint32_t tm_S = tm_Sbuf + lane_addr;
      const uint32_t tm_O = tmem + t * D + lane_addr;
      const float c = P.scale_log2;
      const uint32_t tm_Prow = tm_P + 16 * t + lane_addr;        // this row of P^: 16 columns of 8 codes
      uint32_t* sfp_row = reinterpret_cast<uint32_t*>(smem + L::sfp + t * 1024 + sf_atom_offset(row, 0));
      const uint32_t bar_s = bars + Bars::s_full + 8 * t, bar_p = bars + Bars::p_full + 8 * t;
      const uint32_t bar_pv = bars + Bars::pv_done + 8 * t;
      uint32_t sc = 0;                                           // key tiles processed so far by this warpgroup
      uint32_t ne = 0;                                           // epilogue rendezvous so far
      uint32_t g0 = 0;                                           // K/V stages the CTA used before this work item
      bool ok = true;
      for (int r = 0, w; ok && (w = work_at(r, total_work)) >= 0; ++r) {
        const Work wk = get_work<kCausal, kPacked>(P, w);
        const int n_mine = wk.n_t[t];
        const uint32_t g_first = g0 + (uint32_t)(wk.n_max - n_mine);   // stage counter of this tile's first key tile
        g0 += (uint32_t)wk.n_max;
        const int qt = 2 * wk.pair + t;
        const int q0 = qt * kBlockM, qpos = q0 + row;
#if SAGE3_VARLEN_BUILD
        __nv_bfloat16* orow = P.out + wk.hq * P.o_sh + (int64_t)(wk.q_base + qpos) * P.o_sn;   // packed output
#else
        __nv_bfloat16* orow = P.out + wk.b * P.o_sb + wk.hq * P.o_sh + (int64_t)qpos * P.o_sn;
#endif
        if (n_mine == 0) {
          // query tile that sees no key at all (causal, more queries than keys): zeros, like the
          // reference's store_zero (fwd_epilogue.cu:150-183); nothing if the tile does not exist
          if (SEQ_TILE_EXISTS && qpos < SEQ_NQ) {
            for (int i = 0; i < P.d_out / 8; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0, 0, 0, 0);
            if (P.lse) P.lse[((int64_t)wk.b * P.Hq + wk.hq) * P.Nq + qpos] = -INFINITY;
          }
          continue;
        }
        // last visible key (slot): key padding, and the bottom-right aligned causal diagonal - in K-packing mode
        // the slots of the tokens up to the diagonal one
        auto causal_limit = [&](const int qp) {
          const int tok = qp + SEQ_NK_LOG - SEQ_NQ;              // last visible key token
          if (!kPacked) return tok;
          return tok < 0 ? -1 : packed_slot_of_token(tok);
        };
        const int key_lim = min(SEQ_NK - 1, kCausal ? causal_limit(qpos) : 0x7fffffff);
        const int first_row_lim = kCausal ? causal_limit(q0) : 0x7fffffff;
        float m_ref = -INFINITY, l = 0.f;                        // reference maximum (raw score units), row sum

        for (int it = 0; it < n_mine; ++it, ++sc) {
          const int j = n_mine - 1 - it;
          const int n0 = j * kBlockN;
          const bool need_mask = (n0 + kBlockN - 1 >= SEQ_NK) || (kCausal && n0 + kBlockN - 1 > first_row_lim);
          if (!(ok = wait_bar<false>(bar_s, sc & 1, abort_s, P.status, 30))) break;
          tc_fence_after();
          uint32_t s[128];
          float bm[8];
          load_scores(tm_S, s);
          // the scores are in registers: the Q.K^T of the other query tile may overwrite the buffer
          tc_fence_before();
          mbar_arrive(bars + Bars::s_free);
          if (kPacked) {
            // lambda of this key tile arrived with its K stage, i.e. before the Q.K^T MMA whose completion was
            // awaited above.  Its slot is rewritten 2*kStages key tiles later, which the producer can only do
            // after the Q.K^T of tile g+kStages is complete - issued after both warpgroups finished tile g.
            const uint32_t g = g_first + (uint32_t)it;
            const float* lam_s = reinterpret_cast<const float*>(smem + L::lam) + (g % (2 * kStages)) * 128;
#pragma unroll
            for (int blk = 0; blk < 8; ++blk) apply_lambda(&s[16 * blk], lam_s + 16 * blk);
          }
          if (need_mask) {
            const int lim = key_lim - n0;                        // columns beyond it are masked
#pragma unroll
            for (int i = 0; i < 128; ++i) s[i] = (i > lim) ? 0xff800000u : s[i];
          }
          if (kPacked && P.slot_first) {
            // the other K-packing variant (fwd_mainloop.cu:847-891): the mean slot carries the (masked) score of the
            // group's first token - its V row holds that token's FP4 remainder - except, under the causal mask, in
            // the group of the diagonal token and beyond
            const int qk = qpos + SEQ_NK_LOG - SEQ_NQ;           // the diagonal key token of this row
            const int last_group = kCausal ? (qk < 0 ? -1 : qk / 15 - 1) : 0x7ffffff;   // last group whose slot may be used
#pragma unroll
            for (int blk = 0; blk < 8; ++blk) {
              const int col = n0 + 16 * blk;
              const bool usable = !kCausal || (col < SEQ_NK && (col >> 4) <= last_group);
              s[16 * blk] = usable ? s[16 * blk + 1] : 0xff800000u;
            }
          }
#pragma unroll
          for (int blk = 0; blk < 8; ++blk)
            bm[blk] = max16(&s[16 * blk]);
          const float m_loc = fmax3(fmax3(bm[0], bm[1], bm[2]), fmax3(bm[3], bm[4], bm[5]), fmaxf(bm[6], bm[7]));
          // O_t *= alpha for the rows whose reference maximum moves, in place in tensor memory - but only after this
          // tile's exponentials (below): by then the P.V of the previous key tile, which must land first, has long
          // finished, so nothing waits for it.  Warps in which no row's maximum moved skip the pass.
          float alpha = 1.0f;
          bool rescale = false;
          if (it == 0) {
            m_ref = m_loc;                                       // O_t is overwritten by this tile's P.V
          } else {
            // (-inf) - (-inf) = NaN compares false: a row that has seen no key yet and sees none now stays put
            const bool grow = (m_loc - m_ref) * c > kLazyLog2;
            rescale = __any_sync(0xffffffffu, grow);
            if (grow) {
              alpha = ex2_approx((m_ref - m_loc) * c);
              m_ref = m_loc;
              l *= alpha;
            }
          }
          const float m_fin = (m_ref == -INFINITY) ? 0.f : m_ref;
          const float off = fmaf(m_fin, c, kLog2InvTop);          // P = 2^(s*c - off) in (0, 2688]
          float neg_e[8], sb[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float e = fmaf(bm[i], c, kLog2Inv6);
            sb[i] = ex2_approx(e - off);
            neg_e[i] = (bm[i] == -INFINITY) ? 0.f : -e;
          }
          // P^ and its scales of the previous key tile must have been consumed by its P.V MMAs
          if (sc > 0 && !(ok = wait_bar<false>(bar_pv, (sc - 1) & 1, abort_s, P.status, 31))) break;
          sfp_row[0] = f32x2_to_e4m3x2(sb[0], sb[1]) | (f32x2_to_e4m3x2(sb[2], sb[3]) << 16);     // keys 0-63 of the tile
          sfp_row[128] = f32x2_to_e4m3x2(sb[4], sb[5]) | (f32x2_to_e4m3x2(sb[6], sb[7]) << 16);   // keys 64-127
          l += exp_quantise_store<kPacked>(s, c, neg_e, sb, tm_Prow, P.slot_first);
          if (rescale) {
            if (!(ok = wait_bar<false>(bar_pv, (sc - 1) & 1, abort_s, P.status, 32))) break;
            tc_fence_after();
            const float2 al2 = make_float2(alpha, alpha);
            // the whole O row at once (the score registers are free by now): all loads in flight together, one
            // wait, then scale and store - a chunk-by-chunk round trip would expose the tensor-memory latency 8 times
            uint32_t o[D];
#pragma unroll
            for (int ch = 0; ch < D / 32; ++ch) tmem_ld32(tm_O + 32 * ch, *reinterpret_cast<uint32_t (*)[32]>(&o[32 * ch]));
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < D / 2; ++i) {
              const float2 x = ffma2(make_float2(__uint_as_float(o[2 * i]), __uint_as_float(o[2 * i + 1])), al2,
                                     make_float2(0.f, 0.f));
              o[2 * i] = __float_as_uint(x.x); o[2 * i + 1] = __float_as_uint(x.y);
            }
#pragma unroll
            for (int ch = 0; ch < D / 16; ++ch) tmem_st16(tm_O + 16 * ch, *reinterpret_cast<const uint32_t (*)[16]>(&o[16 * ch]));
            tmem_wait_st();
          }
          // P^ written (and O_t rescaled if it had to be): hand the tile to the PV issuer.  The codes went to tensor
          // memory (tcgen05.st), their block scales to shared memory for the issuer's tcgen05.cp.
          tmem_wait_st();
          tc_fence_before();
          fence_proxy_async_smem();
          mbar_arrive(bar_p);
        }

        // ---- epilogue: O / l -> bf16 -> global.  D=128, dense batches: through a swizzled staging tile in shared
        // memory and one TMA store per 64 columns - a thread owns a whole output row, so direct stores put 32
        // different rows into every store instruction.  D=64 (half the bytes; measured 4 % slower with the staging)
        // and packed variable-length outputs (a tile must not spill into the next sequence) store directly.
        if (!ok) break;
        if (!(ok = wait_bar<false>(bar_pv, (sc - 1) & 1, abort_s, P.status, 33))) break;   // the last P.V has landed
        tc_fence_after();
        const float inv = (l == 0.f || l != l) ? 0.f : 1.0f / l;
        const float2 inv2 = make_float2(inv, inv);
        if (kTmaStore) {
          uint8_t* stage = smem + L::ostage + t * (D / 64) * L::kOStage;
          const uint32_t bar_e = bars + Bars::epi + 8 * t;
          // the stores of the previous work item must have left the staging tile
          if (row == 0) bulk_wait_read0();
          mbar_arrive(bar_e);
          if (!(ok = wait_bar<false>(bar_e, ne & 1, abort_s, P.status, 35))) break;
          ++ne;
          uint32_t oa[16], ob[16];
          tmem_ld16(tm_O, oa);
#pragma unroll
          for (int ch = 0; ch < D / 16; ++ch) {
            uint32_t (&o)[16] = (ch & 1) ? ob : oa;
            uint32_t (&on)[16] = (ch & 1) ? oa : ob;
            tmem_wait_ld();
            if (ch + 1 < D / 16) tmem_ld16(tm_O + (ch + 1) * 16, on);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint4 v;
              float2 x;
              x = ffma2(make_float2(__uint_as_float(o[8 * h + 0]), __uint_as_float(o[8 * h + 1])), inv2, make_float2(0.f, 0.f));
              v.x = pack_bf16(x.x, x.y);
              x = ffma2(make_float2(__uint_as_float(o[8 * h + 2]), __uint_as_float(o[8 * h + 3])), inv2, make_float2(0.f, 0.f));
              v.y = pack_bf16(x.x, x.y);
              x = ffma2(make_float2(__uint_as_float(o[8 * h + 4]), __uint_as_float(o[8 * h + 5])), inv2, make_float2(0.f, 0.f));
              v.z = pack_bf16(x.x, x.y);
              x = ffma2(make_float2(__uint_as_float(o[8 * h + 6]), __uint_as_float(o[8 * h + 7])), inv2, make_float2(0.f, 0.f));
              v.w = pack_bf16(x.x, x.y);
              const int i = 2 * ch + h;                          // 16-byte chunk of the 256-byte output row
              *reinterpret_cast<uint4*>(stage + (i >> 3) * L::kOStage + row * 128 + (((i & 7) ^ (row & 7)) << 4)) = v;
            }
          }
          // O_t is in registers / shared memory: the first P.V of the next work item may overwrite it
          tc_fence_before();
          mbar_arrive(bars + Bars::o_free + 8 * t);
          fence_proxy_async_smem();
          mbar_arrive(bar_e);
          if (!(ok = wait_bar<false>(bar_e, ne & 1, abort_s, P.status, 36))) break;
          ++ne;
          if (row == 0) {
#pragma unroll
            for (int hcol = 0; hcol < D / 64; ++hcol)
              tma_store_4d(&tm_o, sbase + L::ostage + (t * (D / 64) + hcol) * L::kOStage, 64 * hcol,
                           P.o_token_first ? q0 : wk.hq, P.o_token_first ? wk.hq : q0, wk.b);
            bulk_commit_group();
          }
        } else {
          const bool live = qpos < SEQ_NQ;
          uint32_t oa[16], ob[16];
          tmem_ld16(tm_O, oa);
#pragma unroll
          for (int ch = 0; ch < D / 16; ++ch) {
            uint32_t (&o)[16] = (ch & 1) ? ob : oa;
            uint32_t (&on)[16] = (ch & 1) ? oa : ob;
            tmem_wait_ld();
            if (ch + 1 < D / 16) tmem_ld16(tm_O + (ch + 1) * 16, on);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[8 * h + 0]) * inv, __uint_as_float(o[8 * h + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(o[8 * h + 2]) * inv, __uint_as_float(o[8 * h + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(o[8 * h + 4]) * inv, __uint_as_float(o[8 * h + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(o[8 * h + 6]) * inv, __uint_as_float(o[8 * h + 7]) * inv);
              if (live && (2 * ch + h) * 8 < P.d_out) reinterpret_cast<uint4*>(orow)[2 * ch + h] = v;
            }
          }
          tc_fence_before();
          mbar_arrive(bars + Bars::o_free + 8 * t);
        }
        if (qpos < SEQ_NQ) {
          if (P.lse) {
            // natural-log sum of exp(sm_scale * s) over the row (l carries the factor 2688 / 2^kLazyLog2)
            const int64_t li = ((int64_t)wk.b * P.Hq + wk.hq) * P.Nq + qpos;
            float v = (l == 0.f) ? -INFINITY : (m_ref * c + log2f(l) + kLog2InvTop) * (1.0f / kLog2e);
            if (P.lse_add != nullptr) v = fmaf(P.lse_add[li], c * (1.0f / kLog2e), v);
            P.lse[li] = v;
          }
        }
      }
      if (kTmaStore && row == 0) bulk_wait_read0();   // the last output tiles have left shared memory before the CTA ends
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------
// host: tensor maps + launch
// ------------------------------------------------------------------------------------------------
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

// bf16 output [B][Hq][Nq][D] with arbitrary element strides, box = 128 rows x 64 columns (128 bytes, swizzled).
// Tensor-map strides must grow with the dimension, so tokens and heads are ordered by their stride ("HND": D, N,
// H, B; "NHD": D, H, N, B); *n_dim tells the kernel which coordinate is the token.
bool make_out_map(CUtensorMap* m, const void* base, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn,
                  int* n_dim) {   // D = columns the rows really have: the 64-column boxes are clipped to it
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  // a dimension of extent 1 never advances; give it a stride that keeps the order valid
  const bool n_first = (H == 1) || (N > 1 && sn <= sh);
  *n_dim = n_first ? 1 : 2;
  cuuint64_t dims[4] = {(cuuint64_t)D, 0, 0, (cuuint64_t)B};
  cuuint64_t strides[3];
  cuuint32_t box[4] = {64, 1, 1, 1};
  const cuuint64_t s_n = (cuuint64_t)sn * 2, s_h = (cuuint64_t)sh * 2;
  if (n_first) {
    dims[1] = N; dims[2] = H; box[1] = 128;
    strides[0] = N > 1 ? s_n : (cuuint64_t)D * 2;
    strides[1] = H > 1 ? s_h : strides[0] * N;
  } else {
    dims[1] = H; dims[2] = N; box[2] = 128;
    strides[0] = s_h;
    strides[1] = N > 1 ? s_n : strides[0] * H;
  }
  strides[2] = B > 1 ? (cuuint64_t)sb * 2 : strides[1] * dims[2];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool kCausal, bool kPacked>
cudaError_t launch(const AttnArgs& a, cudaStream_t stream) {
  using L = Smem<D>;
  const int Tq = (a.Nq + 127) / 128, Tk = (a.Nk + 127) / 128;
  CUtensorMap tq, tk, tv;
  const CUtensorMapSwizzle swz = D == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  if (!make_map(&tq, a.q_codes, (uint64_t)a.B * a.Hq * Tq * 128, D / 2, 128, swz)) return cudaErrorInvalidValue;
  if (!make_map(&tk, a.k_codes, (uint64_t)a.B * a.Hkv * Tk * 128, D / 2, 128, swz)) return cudaErrorInvalidValue;
  if (!make_map(&tv, a.vt_codes, (uint64_t)a.B * a.Hkv * Tk * D, 64, D, CU_TENSOR_MAP_SWIZZLE_64B))
    return cudaErrorInvalidValue;
  const int d_out = (a.d_out > 0 && a.d_out <= D) ? a.d_out : D;
  CUtensorMap to = tq;                       // only D=128 dense batches store through it
  int o_ndim = 1;
  if (!SAGE3_VARLEN_BUILD && D == 128 &&
      !make_out_map(&to, a.out, a.B, a.Hq, a.Nq, d_out, a.o_sb, a.o_sh, a.o_sn, &o_ndim))
    return cudaErrorInvalidValue;
  KParams P;
  P.q_sf = (const uint8_t*)a.q_sf; P.k_sf = (const uint8_t*)a.k_sf; P.vt_sf = (const uint8_t*)a.vt_sf;
  P.ds = (const __nv_bfloat16*)a.ds; P.out = (__nv_bfloat16*)a.out; P.lse = a.lse; P.lse_add = a.lse_add; P.status = a.status;
  P.o_sb = a.o_sb; P.o_sh = a.o_sh; P.o_sn = a.o_sn;
  P.B = a.B; P.Hq = a.Hq; P.Hkv = a.Hkv; P.Nq = a.Nq; P.Nk = a.Nk; P.Tq = Tq; P.Tk = Tk; P.ds_rows = a.ds_rows;
  P.scale_log2 = a.sm_scale * kLog2e;
  P.o_token_first = o_ndim == 1;
  P.lam = a.k_lambda;
  P.slot_first = kPacked && a.slot_first != 0;
  P.d_out = d_out;
  // K-packing mode: Nk counts key slots; 16 slots hold 15 tokens, a partial group one slot more than its tokens
  P.Nk_log = kPacked ? (a.Nk / 16) * 15 + (a.Nk % 16 == 0 ? 0 : a.Nk % 16 - 1) : a.Nk;
#if SAGE3_VARLEN_BUILD
  P.cu_q = a.cu_q; P.cu_k = a.cu_k;
#endif
  auto kern = attn_fwd_kernel<D, kCausal, kPacked>;
  // persistent CTAs: one per SM (registers and tensor memory allow exactly one), each walks the work list
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  // once per device and instantiation: opt in to the shared memory, and make sure the register hand-over inside
  // the kernel stays within the pool this build of it is launched with (it would block forever otherwise)
  static unsigned char ready[64] = {};
  if (dev < 0 || dev >= 64 || !__atomic_load_n(&ready[dev], __ATOMIC_ACQUIRE)) {
    cudaFuncAttributes fa;
    if ((e = cudaFuncGetAttributes(&fa, kern)) != cudaSuccess) return e;
    if (fa.numRegs * kAttnThreads < 256 * RegSplit<D>::softmax + 128 * RegSplit<D>::role) return cudaErrorLaunchOutOfResources;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total + 1024)) != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) __atomic_store_n(&ready[dev], 1, __ATOMIC_RELEASE);
  }
  const int64_t work = (int64_t)a.B * a.Hq * ((Tq + 1) / 2);
  const int64_t ctas = sms - a.sm_margin > 1 ? sms - a.sm_margin : 1;
  const int64_t grid = work < ctas ? work : ctas;
  kern<<<(unsigned)grid, kAttnThreads, L::total + 1024, stream>>>(tq, tk, tv, to, P);
  return cudaGetLastError();
}

}  // namespace

#if SAGE3_VARLEN_BUILD
cudaError_t launch_attn_fwd_varlen(const AttnArgs& a, cudaStream_t stream) {
  // offsets come in pairs; no K-packing and no LSE for packed batches
  if (a.cu_q == nullptr || a.cu_k == nullptr || a.k_lambda != nullptr || a.lse != nullptr) return cudaErrorInvalidValue;
  if (a.D == 128) return a.causal ? launch<128, true, false>(a, stream) : launch<128, false, false>(a, stream);
  if (a.D == 64) return a.causal ? launch<64, true, false>(a, stream) : launch<64, false, false>(a, stream);
  return cudaErrorInvalidValue;
}
#else
cudaError_t launch_attn_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.D != 128 && a.D != 64) return cudaErrorInvalidValue;
  if (a.k_lambda) {
    if (a.D == 128) return a.causal ? launch<128, true, true>(a, stream) : launch<128, false, true>(a, stream);
    return a.causal ? launch<64, true, true>(a, stream) : launch<64, false, true>(a, stream);
  }
  if (a.D == 128) return a.causal ? launch<128, true, false>(a, stream) : launch<128, false, false>(a, stream);
  return a.causal ? launch<64, true, false>(a, stream) : launch<64, false, false>(a, stream);
}

#endif

}  // namespace sage3
