// Tabulates, on the GPU, the two approximate operations the reference quantiser relies on when it
// is built with --use_fast_math (quantization/fp4_quantization_4d.cu:224-230):
//   sf_of_absmax[i] = e4m3( div.approx.ftz(absmax_i, 6) )  for every non-negative bf16 absmax_i
//   inv_of_sf[c]    = rcp.approx.ftz( e4m3_value(c) )      for every E4M3 code c
// The CPU oracle looks these up ("device" mode) so that it reproduces the CUDA result bit for bit.
#include <stdio.h>
#include "../../sageattention_b200/csrc/common.cuh"

__global__ void tables_kernel(uint8_t* sf_of_absmax, float* inv_of_sf) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < 32768) {
    float amax = __uint_as_float((uint32_t)i << 16);
    uint32_t sfb; float inv;
    sage3::block_scale(amax, sfb, inv);
    sf_of_absmax[i] = (uint8_t)sfb;
  }
  if (i < 128) {
    float sfq = sage3::e4m3_to_f32(i);
    inv_of_sf[i] = (sfq == 0.0f) ? 0.0f : sage3::rcp_approx_ftz(sfq);
  }
}

int main(int argc, char** argv) {
  uint8_t* a; float* b;
  cudaMalloc(&a, 32768); cudaMalloc(&b, 128 * sizeof(float));
  tables_kernel<<<128, 256>>>(a, b);
  static uint8_t ha[32768]; static float hb[128];
  if (cudaMemcpy(ha, a, 32768, cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
  if (cudaMemcpy(hb, b, sizeof(hb), cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
  FILE* f = fopen(argc > 1 ? argv[1] : "device_tables.bin", "wb");
  fwrite(ha, 1, 32768, f); fwrite(hb, 4, 128, f); fclose(f);
  return 0;
}
