/*
 * C ABI of libsage3_b200.so: NVFP4 (microscaled FP4) attention for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; no torch / pybind types.  Every function returns a status
 * (0 = ok, see sage3_status_string) and never throws, aborts or exits.  The library allocates
 * nothing on the device: the caller owns inputs, outputs and workspace (sage3_buffer_sizes says
 * how large each one must be).  All work is enqueued on the stream the caller passes
 * (a cudaStream_t cast to void*; NULL = the legacy default stream) on the current device.
 *
 * The entry points stand in for the two CPython extension modules of the reference project
 * (paths relative to sageattention3_blackwell/sageattn4/):
 *
 *   sage3_quant_qkv   <- quantization/fp4_quantization_4d.cu:414-490 scaled_fp4_quant,
 *                        :492-569 scaled_fp4_quant_permute, :571-648 scaled_fp4_quant_trans
 *                        (pybind block :650-654), plus the eager preprocessing of
 *                        api.py:112-205 (K channel-mean removal :184, per-128-token Q mean
 *                        :26-72,:186-191, delta_s :201, zero padding :196-203)
 *   sage3_attn_fwd    <- blackwell/api.cpp:258-395 mha_fwd (pybind name "fwd", :399-405)
 *   sage3_attention   <- api.py:250-288 sageattn4_blackwell without its K-packing steps
 *                        (= the SageAttention3 call sequence), in one call
 *   sage3_pack_kv, sage3_attn_fwd_packed <- the K-packing steps themselves (api.py:122-177, 267-274;
 *                        kernel side fwd_mainloop.cu:796-891)
 *
 * Tensor arguments are bf16 with the last (head_dim) dimension contiguous; batch / head / token
 * strides are given in elements, so both the "HND" [B,H,N,D] and "NHD" [B,N,H,D] layouts of
 * sageattention/core.py:79-88 are expressed by strides.  head_dim must be 64 or 128.
 */
#ifndef SAGE3_B200_H
#define SAGE3_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define SAGE3_API __attribute__((visibility("default")))
#else
#define SAGE3_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SAGE3_OK = 0,
  SAGE3_ERR_ARGUMENT = 1,     /* null pointer, bad size, bad stride, buffer too small            */
  SAGE3_ERR_UNSUPPORTED = 2,  /* head_dim not in {64,128}, Hq not a multiple of Hkv, ...          */
  SAGE3_ERR_CUDA = 3,         /* a CUDA runtime / driver call failed (see sage3_last_cuda_error)  */
  SAGE3_ERR_DEVICE_WAIT = 4,  /* a bounded wait inside a kernel gave up (read back via
                                 sage3_read_device_status)                                        */
  SAGE3_ERR_TOO_LARGE = 5     /* problem exceeds the fixed scratch of sage3_k_mean_static         */
};

typedef struct {
  int32_t B;      /* batch                                   */
  int32_t Hq;     /* query heads                             */
  int32_t Hkv;    /* key/value heads (Hq % Hkv == 0)         */
  int32_t Nq;     /* query tokens                            */
  int32_t Nk;     /* key/value tokens                        */
  int32_t D;      /* head dim, 64 or 128                     */
} sage3_shape;

/* A bf16 [B,H,N,D] view: element strides of the batch, head and token dimensions. */
typedef struct {
  const void* ptr;
  int64_t stride_b, stride_h, stride_n;
} sage3_tensor;

/* Byte sizes of the caller-owned buffers for one problem shape. */
typedef struct {
  size_t q_codes;   /* u8  [B,Hq ,Tq,128,D/2]           E2M1 pairs, element 2i in the low nibble   */
  size_t q_sf;      /* u8  [B,Hq ,Tq,D/64,512]          E4M3 scales in 128-row tcgen05 SF atoms    */
  size_t k_codes;   /* u8  [B,Hkv,Tk,128,D/2]                                                      */
  size_t k_sf;      /* u8  [B,Hkv,Tk,D/64,512]                                                     */
  size_t vt_codes;  /* u8  [B,Hkv,Tk,D,64]              V transposed per 128-token tile            */
  size_t vt_sf;     /* u8  [B,Hkv,Tk,2,512]             scales over 16 consecutive tokens          */
  size_t qm;        /* bf16 [B,Hq,Tq,D]  (per-block mean)  or [B,Hq,1,D] (whole-sequence mean)     */
  size_t km;        /* bf16 [B,Hkv,D]                                                              */
  size_t delta_s;   /* bf16 [B,Hq,Tq or 1,Tk*128]                                                  */
  size_t q_dot_km;  /* fp32 [B,Hq,Nq]: raw q . K channel mean (the LSE term K smoothing removes)  */
  size_t scratch;   /* reduction scratch of the channel-mean kernel                               */
  size_t status;    /* one int32 on the device                                                    */
  size_t workspace; /* all of the above packed (256-byte aligned parts), for sage3_attention      */
} sage3_sizes;        /* Tq = ceil(Nq/128), Tk = ceil(Nk/128)                                        */

typedef struct {
  sage3_shape shape;
  sage3_tensor q, k, v;      /* any ptr may be NULL: that operand is skipped                        */
  int32_t per_block_mean;    /* 1: Q minus its per-128-token mean (api.py:187-188); 0: Q minus its
                                whole-(padded)-sequence mean (:190-191); -1: Q is not smoothed      */
  int32_t smooth_k;          /* 1: K minus its per-channel token mean (api.py:184)                   */
  const void* km_in;         /* optional bf16 [B,Hkv,D]: use these K means instead of computing them */
  const float* qm_in;        /* optional fp32 [B,Hq,Tq,D]: use these Q block means (per_block_mean=1)*/
  void *q_codes, *q_sf, *k_codes, *k_sf, *vt_codes, *vt_sf;
  void* qm;                  /* out: Q means (needed when per_block_mean >= 0)                       */
  void* km;                  /* out: K means (needed when smooth_k and km_in == NULL)                */
  void* delta_s;             /* out, optional: bf16(qm . k_smoothed^T), bf16 [B,Hq,Tq or 1,Tk*128]   */
  void* scratch;             /* >= sage3_sizes.scratch bytes, 256-byte aligned                       */
  size_t scratch_bytes;
  int32_t* device_status;    /* optional device int32: a bounded wait of the delta_s kernel that gives up
                                records a code in it (NOT zeroed by this call; read it back with
                                sage3_read_device_status)                                            */
  float* q_dot_km;           /* out, optional fp32 [B,Hq,Nq]: raw q . km of the row's kv head (needs smooth_k;
                                dense batches) - feed it to sage3_attn_args.lse_add                   */
  int32_t head_dim_in;       /* 0 or shape.D: the rows of q, k, v have shape.D channels.  Otherwise a
                                multiple of 8 below shape.D: the rows have only that many channels and
                                the kernels treat the rest of the head dim as zero - the head-dim
                                padding of sageattention/core.py:925-937 without a padded copy       */
} sage3_quant_args;

typedef struct {
  sage3_shape shape;
  const void *q_codes, *q_sf, *k_codes, *k_sf, *vt_codes, *vt_sf;   /* layouts of sage3_sizes        */
  const void* delta_s;       /* optional bf16 [B,Hq,delta_s_rows,Tk*128], added to the raw scores    */
  int32_t delta_s_rows;      /* Tq, or 1 when one row serves all query blocks                        */
  void* out;                 /* bf16, strides below (elements), last dim contiguous                  */
  int64_t out_stride_b, out_stride_h, out_stride_n;
  float* lse;                /* optional fp32 [B,Hq,Nq]: log-sum-exp (natural log) of the scores the
                                kernel saw (after smoothing); -inf for rows that see no key          */
  float sm_scale;            /* > 0                                                                  */
  int32_t is_causal;         /* bottom-right aligned when Nq != Nk (fwd_mainloop.cu:926)             */
  int32_t* device_status;    /* one int32 on the device; zeroed on the stream before the launch      */
  const float* lse_add;      /* optional fp32 [B,Hq,Nq]: sm_scale * lse_add is added to the LSE - with
                                sage3_quant_args.q_dot_km this undoes the shift K smoothing gives every
                                score of a row (the pattern of sageattention/core.py:993-994)         */
  int32_t out_head_dim;      /* 0 or shape.D: `out` rows have shape.D columns.  Otherwise a multiple of 8
                                below shape.D: only that many columns are written (core.py:990)      */
  int32_t sm_margin;         /* >= 0: SMs to leave to kernels that run at the same time (a collective's).
                                The attention kernel is persistent, one CTA per SM, with a static work
                                list: a CTA that finds its SM taken starts late and finishes late.  It
                                launches min(work items, SMs - sm_margin) CTAs; results do not depend
                                on it.  The reference has no counterpart.                            */
} sage3_attn_args;

typedef struct {
  sage3_shape shape;
  sage3_tensor q, k, v;
  void* out;
  int64_t out_stride_b, out_stride_h, out_stride_n;
  float* lse;                /* optional fp32 [B,Hq,Nq]: log-sum-exp of sm_scale * q.k over the row (the K-mean
                                term that smoothing removes is added back on the device)             */
  void* km_out;              /* optional bf16 [B,Hkv,D]: K channel means (zeros when smooth_k == 0)   */
  float sm_scale;            /* <= 0: head_dim^-0.5                                                  */
  int32_t is_causal;
  int32_t per_block_mean;    /* as in sage3_quant_args                                               */
  int32_t smooth_k;
  void* workspace;           /* >= sage3_sizes.workspace bytes, 256-byte aligned                     */
  size_t workspace_bytes;
  int32_t* device_status;    /* optional device int32 (see sage3_attn_args); NULL: one inside the
                                workspace is used and cannot be read back by the caller              */
  int32_t head_dim;          /* 0 or shape.D, else the real head dim of q, k, v and out (a multiple of 8
                                below shape.D, see sage3_quant_args.head_dim_in); the default softmax
                                scale is then head_dim^-0.5 (core.py:941)                            */
  int32_t sm_margin;         /* as in sage3_attn_args                                                */
} sage3_fwd_args;

/* K-packing mode of the fork ("SageAttention4", api.py:122-177, 193-203): every 15 key tokens become 16 key
 * slots - the FP4-rounded group mean and 15 residuals k - lambda * mean - and V gets a zero row in every
 * mean slot. */
typedef struct {
  sage3_shape shape;         /* B, Hkv, Nk (key tokens), D are used                                  */
  sage3_tensor k, v;         /* v.ptr may be NULL                                                    */
  int32_t smooth_k;          /* 1: remove the K channel means first (api.py:184)                     */
  const void* km_in;         /* optional bf16 [B,Hkv,D]: use these means instead of computing them   */
  void* km;                  /* out: the means, when smooth_k and km_in == NULL                      */
  void* k_packed;            /* out bf16 [B,Hkv,sage3_packed_rows(Nk),D]                             */
  void* v_packed;            /* out bf16, same shape (needed when v.ptr != NULL)                     */
  float* k_lambda;           /* out fp32 [B,Hkv,ceil(sage3_packed_rows(Nk)/128)*128], 0 in mean slots
                                and padding                                                          */
  void* scratch;             /* as in sage3_quant_args (only used when the means are computed here)  */
  size_t scratch_bytes;
  int32_t split_first;       /* V layout: 0 = a zero row in every mean slot; 1 = the reference's v_trick
                                (api.py:158-170): slot 1 holds the group's first V row as the V^T quantiser
                                rounds it, slot 0 the remainder                                        */
} sage3_pack_args;

/* Variable-length batch (the calling convention of sageattn_varlen, sageattention/core.py:334-358): packed
 * bf16 [tokens, heads, D] tensors and int32 prefix sums of the sequence lengths on the device. */
typedef struct {
  sage3_shape shape;          /* B = number of sequences; Nq, Nk = the LONGEST query / key sequence
                                 (max_seqlen_q, max_seqlen_k): they size the workspace                   */
  const void *q, *k, *v;      /* [sum(len_q), Hq, D], [sum(len_k), Hkv, D] x 2                           */
  int64_t q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h;   /* elements        */
  const int32_t* cu_seqlens_q; /* device int32 [B+1], starts at 0                                        */
  const int32_t* cu_seqlens_k;
  void* out;                  /* bf16 [sum(len_q), Hq, D], strides below                                 */
  int64_t out_stride_n, out_stride_h;
  float sm_scale;             /* <= 0: head_dim^-0.5                                                     */
  int32_t is_causal;          /* bottom-right aligned per sequence                                       */
  int32_t smooth_k;           /* K channel means are taken per sequence                                  */
  void* workspace;            /* >= sage3_buffer_sizes(shape, 1).workspace bytes, 256-byte aligned       */
  size_t workspace_bytes;
  int32_t* device_status;     /* optional, as in sage3_fwd_args                                          */
} sage3_varlen_args;

SAGE3_API int sage3_version(void);
SAGE3_API const char* sage3_status_string(int status);
/* cudaError_t of the most recent failing CUDA call made by this thread inside the library. */
SAGE3_API int sage3_last_cuda_error(void);

SAGE3_API int sage3_buffer_sizes(const sage3_shape* shape, int per_block_mean, sage3_sizes* out);

SAGE3_API int sage3_quant_qkv(const sage3_quant_args* args, void* stream);
SAGE3_API int sage3_attn_fwd(const sage3_attn_args* args, void* stream);
SAGE3_API int sage3_attention(const sage3_fwd_args* args, void* stream);
/* sage3_attention for a variable-length batch in ONE pass over the same four kernels: every kernel takes
 * the sequence offsets and lengths from cu_seqlens_*, the operands are laid out as for a [B, longest] batch
 * and tiles beyond a sequence's end cost nothing.  Replaces the per-sequence loop a caller of the dense
 * entry points would write; the reference's own varlen operator (sageattention/core.py:334-448) belongs to
 * its INT8 kernels and only lends the calling convention.  Per-block Q mean, no LSE output. */
SAGE3_API int sage3_attention_varlen(const sage3_varlen_args* args, void* stream);
/* K-packing mode.  sage3_pack_kv replaces quant_pack_k / quant_pack_v and the K centring of api.py:122-177,
 * 184, 193-194 (eager PyTorch in the reference); its outputs go through sage3_quant_qkv with
 * shape.Nk = sage3_packed_rows(Nk) and smooth_k = 0.  sage3_attn_fwd_packed is sage3_attn_fwd with the
 * lambda correction, slot masking and packed causal mask of fwd_mainloop.cu:273-324, 796-891 (per-block-mean
 * variant when mean_slot_first == 0: the mean slot is masked out; the other variant, fwd_mainloop.cu:847-891,
 * when mean_slot_first == 1: the slot takes the score of the group's first token and stays out of the row sum -
 * to be used with split_first V and, as the reference pairs them, a whole-sequence Q mean, delta_s_rows == 1);
 * args->shape.Nk must be sage3_packed_len(Nk), the number of occupied key slots (api.py:267-274). */
SAGE3_API int sage3_packed_rows(int nk);   /* 16 * ceil(nk / 15): rows of the packed tensors                */
SAGE3_API int sage3_packed_len(int nk);    /* occupied slots: 16 per full group, tokens + 1 for a partial one */
SAGE3_API int sage3_pack_kv(const sage3_pack_args* args, void* stream);
SAGE3_API int sage3_attn_fwd_packed(const sage3_attn_args* args, const float* k_lambda, int32_t mean_slot_first,
                                    void* stream);

/* K channel means (bf16 [B,Hkv,D] into km_out; shape->Hq and shape->Nq are ignored) for callers that
 * cannot allocate device memory where they run - for example a server that gave all device memory to
 * its own pool at start-up, or a hook in which cudaMalloc's device-wide synchronisation or its failure
 * under memory pressure cannot be tolerated.  It has no counterpart in the reference.  The result is
 * the one sage3_quant_qkv writes to `km`; the reduction scratch is a fixed array inside the library
 * (about 1 MiB per GPU, held until the process exits) instead of a caller buffer, and the function
 * calls neither cudaMalloc nor cudaFree nor any other allocating routine.
 *   limit      B*Hkv*chunks <= 2048 partial rows and B*Hkv <= 2048, where chunks = ceil(Nk / c) and the
 *              chunk length c is a power of two of at least 256 tokens chosen so that each head has at
 *              most 64 chunks; e.g. B=1 Hkv=40 Nk=32760 uses 40*32 = 1280 rows.  Larger problems
 *              return SAGE3_ERR_TOO_LARGE.
 *   set-up     the first call made with a given device current looks up the array's address on that
 *              device (cudaGetSymbolAddress); make that first call before any stream capture.
 *   sharing    all calls on a device use the same array, which keeps the previous call's contents;
 *              the function zeroes the counters it needs on `stream` first.  Two calls whose kernels
 *              can overlap on the GPU (different streams, no ordering between them) race on it. */
SAGE3_API int sage3_k_mean_static(const sage3_shape* shape, const sage3_tensor* k, void* km_out, void* stream);

/* Synchronises `stream`, copies the device status word back and maps it to a status
 * (SAGE3_OK or SAGE3_ERR_DEVICE_WAIT); *code_out, if given, receives the raw word. */
SAGE3_API int sage3_read_device_status(const int32_t* device_status, void* stream, int32_t* code_out);

/* Self-test of the kernels' bounded waits: enqueues a one-CTA kernel that waits, with a short poll limit (a few
 * milliseconds), on a barrier nothing completes.  The kernel returns normally and leaves code 77 in
 * *device_status, so a following sage3_read_device_status reports SAGE3_ERR_DEVICE_WAIT; the context stays
 * usable.  No counterpart in the reference. */
SAGE3_API int sage3_selftest_bounded_wait(int32_t* device_status, void* stream);

/* Measures the block-scaled FP4 tensor-core ceiling of the current GPU: one CTA per SM issues
 * tcgen05.mma kind::mxf4nvf4 (M = 128, N = n_cols in {128, 256}, K = 64) back to back on operands resident in
 * shared / tensor memory, `bursts` x 64 MMAs per launch, `launches` launches timed with CUDA events after one
 * warm-up launch.  *tflops_out receives the dense rate (2*M*N*K flops per MMA).  Synchronises `stream`.
 * No counterpart in the reference (its reports quote a data-sheet peak); the number is the denominator of the
 * attention kernel's tensor roofline. */
SAGE3_API int sage3_fp4_mma_peak(int n_cols, int bursts, int launches, int32_t* device_status, void* stream,
                                 double* tflops_out);

#ifdef __cplusplus
}
#endif
#endif /* SAGE3_B200_H */
