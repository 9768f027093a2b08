// Measured ceiling of the block-scaled FP4 tensor-core path on the GPU the library runs on: every SM issues
// tcgen05.mma kind::mxf4nvf4.block_scale.scale_vec::4X (M = 128, N = 128 or 256, K = 64) back to back on
// operands and scale factors that stay resident in shared / tensor memory - no loads, no softmax, no epilogue.
// The rate this reaches is the denominator of the attention kernel's tensor roofline (bench.py); the reference
// has no counterpart (its own reports quote the data-sheet figure of the RTX 5090,
// sageattention3_blackwell/README.md).
//
// One CTA per SM (the shared-memory request keeps a second one out), one issuing thread; the operands are
// pseudo-random bytes (all-zero operands would draw less power and flatter the clock).  Every `kBurst` MMAs the
// thread commits and waits (bounded) for the tensor pipe, which also bounds the depth of the issue queue.
#include "common.cuh"
#include "kernels.h"

namespace sage3 {

namespace {

constexpr int kBurst = 64;

template <int N>
__global__ void __launch_bounds__(128, 1) fp4_mma_peak_kernel(int bursts, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  // A: 128 rows x 32 bytes (K = 64 FP4), two K blocks; B: N rows likewise; 64-byte swizzled rows like the
  // attention kernel's Q / K tiles (row = 64 bytes = K 128)
  constexpr uint32_t oA = 0, oB = 8192, oSF = oB + N * 64, oBar = oSF + 4096;
  const uint32_t bar = sbase + oBar, slot = sbase + oBar + 8;
  const int t = threadIdx.x, warp = t >> 5;
  uint32_t x = 0x9E3779B9u * (blockIdx.x * 128 + t + 1);
  for (uint32_t i = t; i < (oSF + 4096) / 4; i += 128) {
    x = x * 1664525u + 1013904223u;
    uint32_t v = x;
    if (i * 4 >= oSF) v = (x & 0x3f3f3f3fu) | 0x20202020u;      // scale bytes: finite, positive E4M3 near 1
    reinterpret_cast<uint32_t*>(smem)[i] = v;
  }
  if (t == 0) { mbar_init(bar, 1); fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + oBar + 8);
  if (t == 0) {
    constexpr uint32_t idesc = make_idesc_nvf4(128, N);
    constexpr uint32_t HI = (512u >> 4) | (1u << 14) | (4u << 29);     // 64-byte swizzle, 8-row groups 512 B apart
    constexpr uint32_t HI_SF = (128u >> 4) | (1u << 14);
    const uint32_t a_lo = ((sbase + oA) >> 4) | (1u << 16), b_lo = ((sbase + oB) >> 4) | (1u << 16);
    // tensor memory: accumulators in columns [0, 256) (two of 128 columns or one of 256), scale factors behind
    const uint32_t tm_sfa = tmem + 256, tm_sfb = tmem + 264;
    // scale factors once: A 2 K-blocks x 4 columns, B 2 K-blocks x 4 (N = 128) or 8 (N = 256) columns
    for (int kb = 0; kb < 2; ++kb) tc_cp_sf(tm_sfa + 4 * kb, ((sbase + oSF) >> 4) + kb * 32, HI_SF);
    for (int kb = 0; kb < 2 * (N / 128); ++kb) tc_cp_sf(tm_sfb + 4 * kb, ((sbase + oSF + 1024) >> 4) + kb * 32, HI_SF);
    bool ok = true;
    for (int b = 0; ok && b < bursts; ++b) {
#pragma unroll 8
      for (int i = 0; i < kBurst; ++i) {
        // (two accumulators in turn,) two K blocks in turn: the same operand mix as one Q.K^T tile
        const uint32_t acc = tmem + (N == 128 ? (uint32_t)(i & 1) * 128u : 0u);
        const uint32_t kb = (uint32_t)((i >> 1) & 1);
        tc_mma_nvf4(acc, a_lo + kb * 2, HI, b_lo + kb * 2, HI, idesc, tm_sfa + 4 * kb, tm_sfb + 4 * kb * (N / 128),
                    i >= 2 ? 1u : 0u);         // every burst starts its accumulators afresh
      }
      tc_commit(bar);
      ok = mbar_wait(bar, b & 1, 1u << 22);
    }
    if (!ok) atomicCAS(status, 0, 60);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

// Enqueues `launches` launches of the kernel; each SM issues bursts * 64 MMAs of 2 * 128 * N * 64 flops per launch.
cudaError_t launch_fp4_mma_peak(int n_cols, int bursts, int* status, cudaStream_t stream, int* ctas) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  *ctas = sms;
  const int smem = 160 * 1024;            // more than half an SM's shared memory: one CTA per SM
  if (n_cols == 256) {
    if ((e = cudaFuncSetAttribute(fp4_mma_peak_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
    fp4_mma_peak_kernel<256><<<sms, 128, smem, stream>>>(bursts, status);
  } else {
    if ((e = cudaFuncSetAttribute(fp4_mma_peak_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return e;
    fp4_mma_peak_kernel<128><<<sms, 128, smem, stream>>>(bursts, status);
  }
  return cudaGetLastError();
}

}  // namespace sage3
