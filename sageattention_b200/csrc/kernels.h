// Internal launch interfaces between the C-ABI layer (cabi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sage3 {

struct QuantArgs {
  const void *q, *k, *v;                  // bf16, last dim contiguous; any of them may be null (skipped)
  int64_t q_sb, q_sh, q_sn, k_sb, k_sh, k_sn, v_sb, v_sh, v_sn;   // element strides
  int B, Hq, Hkv, Nq, Nk, D;
  int q_mean_mode;                        // 0 none, 1 per 128-token block, 2 whole sequence
  const void* km;                         // bf16 [B,Hkv,D] or null (no K smoothing)
  const void* q_mean_seq;                 // bf16 [B,Hq,D]   (mode 2)
  const void* qm_override;                // fp32 [B,Hq,Tq,D] or null (mode 1)
  void *q_codes, *q_sf, *k_codes, *k_sf, *vt_codes, *vt_sf, *qm;
  void* q_dot_km = nullptr;               // optional fp32 [B,Hq,Nq]: raw q . km (needs km; dense batches only)
  // variable-length batches: device int32 [B+1] token offsets of the sequences inside packed [tokens, H, D]
  // tensors (then *_sb is ignored and Nq / Nk are the LONGEST sequence, which sizes the output layouts)
  const int* cu_q = nullptr;
  const int* cu_k = nullptr;
  int d_in = 0;                           // channels the input rows really have (0 = D; <= D, multiple of 8): the
                                          // kernels read only those and treat the rest of the head dim as zero
};

size_t quant_scratch_bytes(int B, int H, int N, int D);
cudaError_t launch_channel_mean(const void* x, int64_t sb, int64_t sh, int64_t sn, int B, int H, int N, int D,
                                float divisor, void* scratch, void* mean_out, cudaStream_t stream,
                                const int* cu = nullptr, int d_in = 0);
cudaError_t launch_quant_qkv(const QuantArgs& a, cudaStream_t stream);
cudaError_t launch_channel_mean_static(const void* x, int64_t sb, int64_t sh, int64_t sn, int B, int H, int N, int D,
                                       float divisor, void* mean_out, cudaStream_t stream, bool* too_large);

// K-packing mode: 15 tokens -> 16 slots (group mean + residuals), see pack.cu
struct PackArgs {
  const void *k, *v;                      // bf16, strides below; v may be null
  int64_t k_sb, k_sh, k_sn, v_sb, v_sh, v_sn;
  const void* km;                         // bf16 [B,Hkv,D] K channel means to subtract first, or null
  void *kp, *vp;                          // bf16 [B,Hkv,16*G,D] contiguous, G = ceil(Nk/15); vp may be null
  float* lam;                             // fp32 [B,Hkv,ceil(16*G/128)*128]
  int B, Hkv, Nk, D;
  int split_first = 0;                    // V layout of the reference's v_trick (see pack.cu)
};
cudaError_t launch_pack_kv(const PackArgs& a, cudaStream_t stream);

struct DeltaSArgs {
  const void* qm;                         // bf16 [B,Hq,Tq,D]
  const void* k;                          // bf16 raw K, strides below
  int64_t k_sb, k_sh, k_sn;
  const void* km;                         // bf16 [B,Hkv,D] or null
  void* ds;                               // bf16 [B,Hq,Tq,Nk_pad]
  int B, Hq, Hkv, Tq, Nk, D;
  const int* cu_k = nullptr;              // variable-length batches, see QuantArgs
  void* k_codes = nullptr;                // when given, the kernel also writes the NVFP4 codes and scales of the
  void* k_sf = nullptr;                   //   smoothed K tile it holds (the K role of the quantisation kernel)
  int* status = nullptr;                  // optional device status word for the kernel's bounded wait
  int d_in = 0;                           // as in QuantArgs
};
cudaError_t launch_delta_s(const DeltaSArgs& a, cudaStream_t stream);

struct AttnArgs {
  const void *q_codes, *q_sf, *k_codes, *k_sf, *vt_codes, *vt_sf;
  const void* ds;                         // bf16 [B,Hq,ds_rows,Nk_pad] (raw score units) or null
  int ds_rows;                            // Tq, or 1 when one row serves every query block
  void* out;                              // bf16, strides below
  int64_t o_sb, o_sh, o_sn;
  float* lse;                             // fp32 [B,Hq,Nq] or null
  const float* lse_add = nullptr;         // optional fp32 [B,Hq,Nq]: sm_scale times it is added to the LSE
  int* status;                            // device int, set non-zero if a bounded wait gave up
  int B, Hq, Hkv, Nq, Nk, D;
  float sm_scale;
  int causal;
  const float* k_lambda;                  // K-packing mode: fp32 [B,Hkv,Tk*128]; Nk is then the packed length
  int slot_first = 0;                     // K-packing mode: mean slot = first token's score (else masked)
  int d_out = 0;                          // columns the output rows really have (0 = D; <= D, multiple of 8)
  int sm_margin = 0;                      // SMs left free for kernels running beside the persistent attention kernel
  const int* cu_q = nullptr;              // variable-length batches, see QuantArgs; out is then [tokens, Hq, D]
  const int* cu_k = nullptr;
};
cudaError_t launch_attn_fwd(const AttnArgs& a, cudaStream_t stream);
cudaError_t launch_attn_fwd_varlen(const AttnArgs& a, cudaStream_t stream);   // cu_q / cu_k given

// Back-to-back block-scaled FP4 MMAs on resident operands, one CTA per SM (peak.cu); *ctas = CTAs launched.
cudaError_t launch_fp4_mma_peak(int n_cols, int bursts, int* status, cudaStream_t stream, int* ctas);

// One CTA runs a bounded wait that must give up (selftest.cu); *status receives `code`.
cudaError_t launch_bounded_wait_selftest(int* status, int code, cudaStream_t stream);

}  // namespace sage3
