// Shared device helpers for the sm_100a kernels: numeric conversions that must match the
// reference's instruction forms bit for bit, and thin wrappers over the Blackwell PTX
// (mbarrier, TMA, tcgen05 / TMEM) used by the attention kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sage3 {

// ---------------------------------------------------------------------------------------------
// Numerics.  The reference quantiser (sageattn4/quantization/fp4_quantization_4d.cu:224-251) is
// compiled with --use_fast_math, so `absmax / 6.0f` is div.approx.ftz, `1.0f / SF` is
// rcp.approx.ftz and the products are mul.ftz; the same PTX forms are issued here explicitly so
// that codes and scales come out bit-identical whatever flags this file is built with.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float div_approx_ftz(float a, float b) {
  float r;
  asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float rcp_approx_ftz(float a) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}
__device__ __forceinline__ float mul_ftz(float a, float b) {
  float r;
  asm("mul.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ex2_approx(float a) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}

// fp32 -> E4M3 (round to nearest even, saturate to 448); returns the byte.
__device__ __forceinline__ uint32_t f32_to_e4m3(float x) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
  return r & 0xFFu;
}
// two floats -> two E4M3 bytes, `lo` in bits 0-7
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// E4M3 byte -> fp32 (exact)
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)b));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}

// 8 floats -> 8 E2M1 nibbles in one u32, element 0 in the lowest nibble
// (same operand order as fp32_vec_to_e2m1, fp4_quantization_4d.cu:77-99).
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(float a0, float a1, float a2, float a3,
                                                     float a4, float a5, float a6, float a7) {
  uint32_t v;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(v)
      : "f"(a0), "f"(a1), "f"(a2), "f"(a3), "f"(a4), "f"(a5), "f"(a6), "f"(a7));
  return v;
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ uint32_t habsmax2(uint32_t a, uint32_t b) {   // per-half max(|a|,|b|)
  __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&a);
  __nv_bfloat162 y = *reinterpret_cast<__nv_bfloat162*>(&b);
  __nv_bfloat162 m = __hmax2(__habs2(x), __habs2(y));
  return *reinterpret_cast<uint32_t*>(&m);
}

// Scale byte + reciprocal for one 16-element block whose absmax (a bf16 value) is `amax`
// (fp4_quantization_4d.cu:224-230).
__device__ __forceinline__ void block_scale(float amax, uint32_t& sf_byte, float& inv) {
  float sf = div_approx_ftz(amax, 6.0f);
  sf_byte = f32_to_e4m3(sf);
  float sfq = e4m3_to_f32(sf_byte);
  inv = (sfq == 0.0f) ? 0.0f : rcp_approx_ftz(sfq);
}

// Byte offset of the scale for (row, k16-block) inside a 512-byte "SF atom": 128 rows x 4 scales
// (= 64 elements of the contraction dim).  This is the order tcgen05.cp.32x128b.warpx4 moves
// into tensor memory for a block-scaled MMA: row r sits in lane r%32, 32-bit column r/32,
// byte = block index.
__host__ __device__ __forceinline__ int sf_atom_offset(int row, int blk4) {
  return (row & 31) * 16 + (row >> 5) * 4 + blk4;
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers (sm_100a)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One poll of an mbarrier phase.  kHintNs > 0: try_wait with a suspend-time hint (measured on B200: a failing
// poll returns after about 4 us whatever the hint); 0: try_wait without hint (about 1.5 us); < 0: a plain test
// that never parks (7 ns).  A parked thread resumes as soon as the phase completes.
template <int kHintNs = 0>
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if constexpr (kHintNs > 0) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"((uint32_t)kHintNs) : "memory");
  } else if constexpr (kHintNs == 0) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  }
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports failure instead of hanging the SM.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 26)) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Bounded wait on an mbarrier phase used by the kernels' roles; also gives up as soon as any CTA has reported a
// failure through *status.  A failing poll parks the thread for about 1.5 us (kHinted: about 4 us), so the default
// limit of 2^21 polls is 3 to 8 seconds; which flavour is faster was measured per role: the shorter park costs
// issue slots but reacts sooner.  On giving up it raises the CTA's abort flag, records `code` in *status (first
// writer wins) and returns false - the caller then unwinds instead of hanging the SM.
template <bool kHinted, uint32_t kPolls = (1u << 21)>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_s, int* status, int code) {
  for (uint32_t i = 0; i < kPolls; ++i) {
    if (mbar_try_wait<kHinted ? 20000 : 0>(bar, parity)) return true;
    if ((i & 1023u) == 1023u && (*abort_s != 0 || *reinterpret_cast<volatile int*>(status) != 0)) break;
  }
  *abort_s = 1;
  atomicCAS(status, 0, code);
  return false;
}

// The same with the flavour of the poll chosen at run time (uniform per kernel launch).
template <uint32_t kPolls = (1u << 21)>
__device__ __forceinline__ bool wait_bar_dyn(uint32_t bar, uint32_t parity, const bool hinted, volatile int* abort_s,
                                             int* status, int code) {
  for (uint32_t i = 0; i < kPolls; ++i) {
    if (hinted ? mbar_try_wait<20000>(bar, parity) : mbar_try_wait<0>(bar, parity)) return true;
    if ((i & 1023u) == 1023u && (*abort_s != 0 || *reinterpret_cast<volatile int*>(status) != 0)) break;
  }
  *abort_s = 1;
  atomicCAS(status, 0, code);
  return false;
}

// The same for a whole warp that goes on to warp-wide instructions (tcgen05.ld / st, votes): every lane gets the
// same answer, so the warp never splits on a wait that ran out for some of its lanes only.
template <bool kHinted, uint32_t kPolls = (1u << 21)>
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, volatile int* abort_s, int* status, int code) {
  return __all_sync(0xffffffffu, wait_bar<kHinted, kPolls>(bar, parity, abort_s, status, code));
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// shared -> global tile store through a 4-D tensor map (rows outside the tensor are clipped by the hardware);
// completion is tracked in bulk groups of the issuing thread
__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
               :: "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(src) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
               :: "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all bulk groups of this thread have finished READING shared memory (their source may be reused)
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
// plain bulk copy global -> shared (16-byte aligned addresses and size)
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// --- tensor memory / tcgen05 ---
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 columns of 32-bit values from registers into tensor memory; tmem_wait_st() before a load
// of the same columns
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
         "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// 4 words of this thread's TMEM lane (e.g. 32 FP4 codes of an A operand kept in tensor memory).
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" :: "r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 rows x 16 bytes of scale factors: shared -> tensor memory, replicated into all four
// 32-lane quarters (what block-scaled MMAs expect).
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], E2M1 operands with one UE4M3 scale per 16 elements, K = 64.
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 operands, K = 16.
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// The same three operations taking each 64-bit shared-memory descriptor as (low word, high word):
// the issuing thread then only does 32-bit adds on the low word.
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint32_t lo, uint32_t hi) {
  asm volatile("{\n.reg .b64 d;\nmov.b64 d, {%1, %2};\ntcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n}"
               ::"r"(taddr), "r"(lo), "r"(hi) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %5, [%7], [%8], p;\n}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// The same with the A operand in tensor memory: lane = row, 8 columns per K block of 64, word c of a lane = the row's
// codes 8c ... 8c+7 (low nibble first) - the byte order of the shared-memory operand.
__device__ __forceinline__ void tc_mma_nvf4_ta(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 db;\n"
      "setp.ne.b32 p, %5, 0;\nmov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], [%1], db, %4, [%6], [%7], p;\n}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory matrix descriptor for a K-major operand.
//   swizzle_code: 0 none (8x16B core matrices), 6 = 32B, 4 = 64B, 2 = 128B swizzle
//   sbo_bytes   : distance between consecutive groups of 8 rows
//   lbo_bytes   : distance between the two 16-byte K chunks (unswizzled layouts only)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes, uint32_t lbo_bytes,
                                                   uint32_t swizzle_code) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                          // descriptor version (Blackwell)
  d |= (uint64_t)(swizzle_code & 7) << 61;
  return d;
}

// Instruction descriptor for kind::mxf4nvf4, scale_vec::4X: E2M1 x E2M1 -> fp32, UE4M3 scales,
// both operands K-major, M x N tile, K = 64.
__host__ __device__ constexpr uint32_t make_idesc_nvf4(int M, int N) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | (0u << 23) | ((uint32_t)(M >> 4) << 24);
}
// Instruction descriptor for kind::f16 with bf16 operands, fp32 accumulate, K-major A and B.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 32 consecutive fp32 columns of this thread's TMEM lane -> registers.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

// 8 consecutive fp32 columns of this thread's TMEM lane -> registers.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr) : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane -> registers.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}

}  // namespace sage3
