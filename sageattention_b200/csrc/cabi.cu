// extern "C" boundary of libsage3_b200.so (declared in include/sage3_b200.h): argument checks,
// workspace carving and launch sequencing.  No device allocation happens here.
#include "../../include/sage3_b200.h"

#include <cuda_runtime.h>

#include "kernels.h"

namespace {

thread_local int g_last_cuda_error = 0;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return SAGE3_ERR_CUDA;
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

inline int check_shape(const sage3_shape& s) {
  if (s.B <= 0 || s.Hq <= 0 || s.Hkv <= 0 || s.Nq <= 0 || s.Nk <= 0) return SAGE3_ERR_ARGUMENT;
  if (s.D != 64 && s.D != 128) return SAGE3_ERR_UNSUPPORTED;
  if (s.Hq % s.Hkv != 0) return SAGE3_ERR_UNSUPPORTED;
  // (batch, head) pairs index the second grid dimension of the reduction and delta_s kernels
  if ((int64_t)s.B * s.Hq > 65535) return SAGE3_ERR_UNSUPPORTED;
  // tile indices and TMA row coordinates are 32-bit
  const int64_t Tq = (s.Nq + 127) / 128, Tk = (s.Nk + 127) / 128;
  if ((int64_t)s.B * s.Hq * Tq * 128 >= (1ll << 31) || (int64_t)s.B * s.Hkv * Tk * 128 >= (1ll << 31))
    return SAGE3_ERR_UNSUPPORTED;
  return SAGE3_OK;
}

// real head dim of the caller's rows: 0 means D; otherwise a multiple of 8 (128-bit loads) not above D
inline bool head_dim_ok(int d, int D) { return d == 0 || (d > 0 && d <= D && d % 8 == 0); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int check_tensor(const sage3_tensor& t) {
  if (t.ptr == nullptr) return SAGE3_OK;
  if (!aligned16(t.ptr)) return SAGE3_ERR_ARGUMENT;
  // 128-bit loads: every row must start on a 16-byte boundary
  if ((t.stride_b % 8) || (t.stride_h % 8) || (t.stride_n % 8)) return SAGE3_ERR_ARGUMENT;
  return SAGE3_OK;
}

}  // namespace

extern "C" {

int sage3_version(void) { return 100; }

const char* sage3_status_string(int status) {
  switch (status) {
    case SAGE3_OK: return "ok";
    case SAGE3_ERR_ARGUMENT: return "invalid argument (null pointer, size, stride or alignment)";
    case SAGE3_ERR_UNSUPPORTED: return "unsupported shape (head_dim must be 64 or 128, Hq a multiple of Hkv, B*Hq <= 65535)";
    case SAGE3_ERR_CUDA: return "CUDA call failed (see sage3_last_cuda_error)";
    case SAGE3_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel gave up";
    case SAGE3_ERR_TOO_LARGE: return "problem exceeds the fixed scratch of sage3_k_mean_static (2048 partial rows / 2048 heads)";
    default: return "unknown status";
  }
}

int sage3_last_cuda_error(void) { return g_last_cuda_error; }

int sage3_buffer_sizes(const sage3_shape* shape, int per_block_mean, sage3_sizes* out) {
  if (shape == nullptr || out == nullptr) return SAGE3_ERR_ARGUMENT;
  if (int st = check_shape(*shape)) return st;
  const sage3_shape& s = *shape;
  const size_t Tq = (s.Nq + 127) / 128, Tk = (s.Nk + 127) / 128;
  const size_t bhq = (size_t)s.B * s.Hq, bhk = (size_t)s.B * s.Hkv;
  const size_t ds_rows = per_block_mean == 1 ? Tq : 1;
  out->q_codes = bhq * Tq * 128 * (s.D / 2);
  out->q_sf = bhq * Tq * (s.D / 64) * 512;
  out->k_codes = bhk * Tk * 128 * (s.D / 2);
  out->k_sf = bhk * Tk * (s.D / 64) * 512;
  out->vt_codes = bhk * Tk * s.D * 64;
  out->vt_sf = bhk * Tk * 1024;
  out->qm = bhq * ds_rows * s.D * 2;
  out->km = bhk * s.D * 2;
  out->delta_s = per_block_mean < 0 ? 0 : bhq * ds_rows * Tk * 128 * 2;
  out->q_dot_km = bhq * (size_t)s.Nq * sizeof(float);
  size_t sk = sage3::quant_scratch_bytes(s.B, s.Hkv, s.Nk, s.D);
  size_t sq = sage3::quant_scratch_bytes(s.B, s.Hq, s.Nq, s.D);
  out->scratch = sk > sq ? sk : sq;
  out->status = 4;
  out->workspace = align256(out->q_codes) + align256(out->q_sf) + align256(out->k_codes) + align256(out->k_sf) +
                   align256(out->vt_codes) + align256(out->vt_sf) + align256(out->qm) + align256(out->km) +
                   align256(out->delta_s) + align256(out->q_dot_km) + align256(out->scratch) + 256;
  return SAGE3_OK;
}

static int quant_qkv_impl(const sage3_quant_args* a, const int* cu_q, const int* cu_k, void* stream_) {
  if (a == nullptr) return SAGE3_ERR_ARGUMENT;
  if (int st = check_shape(a->shape)) return st;
  if (int st = check_tensor(a->q)) return st;
  if (int st = check_tensor(a->k)) return st;
  if (int st = check_tensor(a->v)) return st;
  cudaStream_t stream = (cudaStream_t)stream_;
  const sage3_shape& s = a->shape;
  if (a->q.ptr && (!a->q_codes || !a->q_sf)) return SAGE3_ERR_ARGUMENT;
  if (a->k.ptr && (!a->k_codes || !a->k_sf)) return SAGE3_ERR_ARGUMENT;
  if (a->v.ptr && (!a->vt_codes || !a->vt_sf)) return SAGE3_ERR_ARGUMENT;
  if (a->q.ptr && a->per_block_mean >= 0 && !a->qm) return SAGE3_ERR_ARGUMENT;
  if (a->per_block_mean < -1 || a->per_block_mean > 1) return SAGE3_ERR_ARGUMENT;
  if (!head_dim_ok(a->head_dim_in, s.D)) return SAGE3_ERR_ARGUMENT;

  const void* km = nullptr;
  if (a->k.ptr && a->smooth_k) {
    if (a->km_in) {
      km = a->km_in;
    } else {
      if (!a->km || !a->scratch || !aligned16(a->scratch)) return SAGE3_ERR_ARGUMENT;
      if (a->scratch_bytes < sage3::quant_scratch_bytes(s.B, s.Hkv, s.Nk, s.D)) return SAGE3_ERR_ARGUMENT;
      cudaError_t e = sage3::launch_channel_mean(a->k.ptr, a->k.stride_b, a->k.stride_h, a->k.stride_n, s.B, s.Hkv,
                                                 s.Nk, s.D, (float)s.Nk, a->scratch, a->km, stream, cu_k, a->head_dim_in);
      if (e != cudaSuccess) return cuda_fail(e);
      km = a->km;
    }
  }
  const int Tq = (s.Nq + 127) / 128;
  if (a->q.ptr && a->per_block_mean == 0) {
    // mean over the zero-padded length, as the reference pads before taking it (api.py:186,190)
    if (cu_q != nullptr) return SAGE3_ERR_UNSUPPORTED;   // whole-sequence Q mean is not built for packed batches
    if (!a->scratch || !aligned16(a->scratch) ||
        a->scratch_bytes < sage3::quant_scratch_bytes(s.B, s.Hq, s.Nq, s.D))
      return SAGE3_ERR_ARGUMENT;
    cudaError_t e = sage3::launch_channel_mean(a->q.ptr, a->q.stride_b, a->q.stride_h, a->q.stride_n, s.B, s.Hq, s.Nq,
                                               s.D, (float)(Tq * 128), a->scratch, a->qm, stream, nullptr, a->head_dim_in);
    if (e != cudaSuccess) return cuda_fail(e);
  }

  // with delta_s requested, K is quantised by the delta_s kernel, which has the smoothed tile in hand anyway
  if (a->delta_s != nullptr && !aligned16(a->delta_s)) return SAGE3_ERR_ARGUMENT;     // written through a tensor map
  const bool k_in_ds = a->delta_s != nullptr && a->k.ptr != nullptr;
  if (a->delta_s != nullptr && (!a->q.ptr || !a->k.ptr || a->per_block_mean < 0)) return SAGE3_ERR_ARGUMENT;
  sage3::QuantArgs q{};
  q.q = a->q.ptr; q.k = k_in_ds ? nullptr : a->k.ptr; q.v = a->v.ptr;
  q.q_sb = a->q.stride_b; q.q_sh = a->q.stride_h; q.q_sn = a->q.stride_n;
  q.k_sb = a->k.stride_b; q.k_sh = a->k.stride_h; q.k_sn = a->k.stride_n;
  q.v_sb = a->v.stride_b; q.v_sh = a->v.stride_h; q.v_sn = a->v.stride_n;
  q.B = s.B; q.Hq = s.Hq; q.Hkv = s.Hkv; q.Nq = s.Nq; q.Nk = s.Nk; q.D = s.D;
  q.q_mean_mode = a->per_block_mean == 1 ? 1 : (a->per_block_mean == 0 ? 2 : 0);
  q.km = km;
  q.q_mean_seq = a->per_block_mean == 0 ? a->qm : nullptr;
  q.qm_override = a->per_block_mean == 1 ? a->qm_in : nullptr;
  q.q_codes = a->q_codes; q.q_sf = a->q_sf; q.k_codes = a->k_codes; q.k_sf = a->k_sf;
  q.vt_codes = a->vt_codes; q.vt_sf = a->vt_sf; q.qm = a->qm;
  q.cu_q = cu_q; q.cu_k = cu_k;
  q.d_in = a->head_dim_in;
  if (a->q_dot_km != nullptr) {
    if (km == nullptr || cu_q != nullptr || !a->q.ptr) return SAGE3_ERR_ARGUMENT;
    q.q_dot_km = a->q_dot_km;
  }
  cudaError_t e = sage3::launch_quant_qkv(q, stream);
  if (e != cudaSuccess) return cuda_fail(e);

  if (a->delta_s != nullptr) {
    sage3::DeltaSArgs d{};
    d.qm = a->qm; d.k = a->k.ptr; d.k_sb = a->k.stride_b; d.k_sh = a->k.stride_h; d.k_sn = a->k.stride_n;
    d.km = km; d.ds = a->delta_s; d.cu_k = cu_k;
    d.k_codes = a->k_codes; d.k_sf = a->k_sf; d.status = a->device_status; d.d_in = a->head_dim_in;
    d.B = s.B; d.Hq = s.Hq; d.Hkv = s.Hkv; d.Tq = a->per_block_mean == 1 ? Tq : 1; d.Nk = s.Nk; d.D = s.D;
    e = sage3::launch_delta_s(d, stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  return SAGE3_OK;
}

int sage3_quant_qkv(const sage3_quant_args* a, void* stream) { return quant_qkv_impl(a, nullptr, nullptr, stream); }

static int attn_fwd_impl(const sage3_attn_args* a, const float* k_lambda, const int* cu_q, const int* cu_k, void* stream_,
                         int slot_first = 0, bool zero_status = true) {
  if (a == nullptr) return SAGE3_ERR_ARGUMENT;
  if (int st = check_shape(a->shape)) return st;
  if (!a->q_codes || !a->q_sf || !a->k_codes || !a->k_sf || !a->vt_codes || !a->vt_sf || !a->out || !a->device_status)
    return SAGE3_ERR_ARGUMENT;
  if (!aligned16(a->q_codes) || !aligned16(a->k_codes) || !aligned16(a->vt_codes) || !aligned16(a->q_sf) ||
      !aligned16(a->k_sf) || !aligned16(a->vt_sf) || !aligned16(a->out) || (a->delta_s && !aligned16(a->delta_s)))
    return SAGE3_ERR_ARGUMENT;
  if ((a->out_stride_b % 8) || (a->out_stride_h % 8) || (a->out_stride_n % 8)) return SAGE3_ERR_ARGUMENT;
  const sage3_shape& s = a->shape;
  const int Tq = (s.Nq + 127) / 128;
  if (a->delta_s && a->delta_s_rows != 1 && a->delta_s_rows != Tq) return SAGE3_ERR_ARGUMENT;
  if (!(a->sm_scale > 0.f)) return SAGE3_ERR_ARGUMENT;          // the row maximum is tracked in raw score units
  if (!head_dim_ok(a->out_head_dim, s.D)) return SAGE3_ERR_ARGUMENT;
  if (a->sm_margin < 0) return SAGE3_ERR_ARGUMENT;
  cudaStream_t stream = (cudaStream_t)stream_;
  cudaError_t e = cudaSuccess;
  if (zero_status) {
    e = cudaMemsetAsync(a->device_status, 0, sizeof(int32_t), stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  sage3::AttnArgs k{};
  k.q_codes = a->q_codes; k.q_sf = a->q_sf; k.k_codes = a->k_codes; k.k_sf = a->k_sf;
  k.vt_codes = a->vt_codes; k.vt_sf = a->vt_sf; k.ds = a->delta_s; k.ds_rows = a->delta_s ? a->delta_s_rows : 1;
  k.out = a->out; k.o_sb = a->out_stride_b; k.o_sh = a->out_stride_h; k.o_sn = a->out_stride_n;
  k.lse = a->lse; k.lse_add = a->lse_add; k.status = a->device_status;
  k.B = s.B; k.Hq = s.Hq; k.Hkv = s.Hkv; k.Nq = s.Nq; k.Nk = s.Nk; k.D = s.D;
  k.sm_scale = a->sm_scale; k.causal = a->is_causal;
  k.k_lambda = k_lambda;
  k.slot_first = slot_first;
  k.d_out = a->out_head_dim;
  k.sm_margin = a->sm_margin;
  k.cu_q = cu_q; k.cu_k = cu_k;
  e = (cu_q != nullptr || cu_k != nullptr) ? sage3::launch_attn_fwd_varlen(k, stream) : sage3::launch_attn_fwd(k, stream);
  if (e != cudaSuccess) return cuda_fail(e);
  return SAGE3_OK;
}

int sage3_attn_fwd(const sage3_attn_args* a, void* stream) { return attn_fwd_impl(a, nullptr, nullptr, nullptr, stream); }

int sage3_attn_fwd_packed(const sage3_attn_args* a, const float* k_lambda, int32_t mean_slot_first, void* stream) {
  if (k_lambda == nullptr || !aligned16(k_lambda)) return SAGE3_ERR_ARGUMENT;
  return attn_fwd_impl(a, k_lambda, nullptr, nullptr, stream, mean_slot_first != 0);
}

int sage3_packed_rows(int nk) { return nk <= 0 ? 0 : 16 * ((nk + 14) / 15); }

int sage3_packed_len(int nk) { return nk <= 0 ? 0 : (nk / 15) * 16 + (nk % 15 == 0 ? 0 : nk % 15 + 1); }

int sage3_pack_kv(const sage3_pack_args* a, void* stream_) {
  if (a == nullptr || a->k.ptr == nullptr || a->k_packed == nullptr || a->k_lambda == nullptr) return SAGE3_ERR_ARGUMENT;
  const sage3_shape& s = a->shape;
  if (s.B <= 0 || s.Hkv <= 0 || s.Nk <= 0) return SAGE3_ERR_ARGUMENT;
  if (s.D != 64 && s.D != 128) return SAGE3_ERR_UNSUPPORTED;
  if ((int64_t)s.B * s.Hkv > 65535) return SAGE3_ERR_UNSUPPORTED;
  if (int st = check_tensor(a->k)) return st;
  if (int st = check_tensor(a->v)) return st;
  if (a->v.ptr && !a->v_packed) return SAGE3_ERR_ARGUMENT;
  if (!aligned16(a->k_packed) || !aligned16(a->k_lambda) || (a->v_packed && !aligned16(a->v_packed))) return SAGE3_ERR_ARGUMENT;
  cudaStream_t stream = (cudaStream_t)stream_;
  const void* km = nullptr;
  if (a->smooth_k) {
    if (a->km_in) {
      km = a->km_in;
    } else {
      if (!a->km || !a->scratch || !aligned16(a->scratch)) return SAGE3_ERR_ARGUMENT;
      if (a->scratch_bytes < sage3::quant_scratch_bytes(s.B, s.Hkv, s.Nk, s.D)) return SAGE3_ERR_ARGUMENT;
      cudaError_t e = sage3::launch_channel_mean(a->k.ptr, a->k.stride_b, a->k.stride_h, a->k.stride_n, s.B, s.Hkv,
                                                 s.Nk, s.D, (float)s.Nk, a->scratch, a->km, stream);
      if (e != cudaSuccess) return cuda_fail(e);
      km = a->km;
    }
  }
  sage3::PackArgs p{};
  p.k = a->k.ptr; p.k_sb = a->k.stride_b; p.k_sh = a->k.stride_h; p.k_sn = a->k.stride_n;
  p.v = a->v.ptr; p.v_sb = a->v.stride_b; p.v_sh = a->v.stride_h; p.v_sn = a->v.stride_n;
  p.km = km; p.kp = a->k_packed; p.vp = a->v.ptr ? a->v_packed : nullptr; p.lam = a->k_lambda;
  p.B = s.B; p.Hkv = s.Hkv; p.Nk = s.Nk; p.D = s.D;
  p.split_first = a->split_first != 0;
  cudaError_t e = sage3::launch_pack_kv(p, stream);
  if (e != cudaSuccess) return cuda_fail(e);
  return SAGE3_OK;
}

int sage3_attention(const sage3_fwd_args* a, void* stream) {
  if (a == nullptr || a->workspace == nullptr || a->out == nullptr) return SAGE3_ERR_ARGUMENT;
  if (!a->q.ptr || !a->k.ptr || !a->v.ptr) return SAGE3_ERR_ARGUMENT;
  sage3_sizes z;
  if (int st = sage3_buffer_sizes(&a->shape, a->per_block_mean, &z)) return st;
  if (a->workspace_bytes < z.workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) return SAGE3_ERR_ARGUMENT;
  char* w = reinterpret_cast<char*>(a->workspace);
  auto take = [&](size_t n) { char* p = w; w += align256(n); return (void*)p; };
  sage3_quant_args q{};
  q.shape = a->shape; q.q = a->q; q.k = a->k; q.v = a->v;
  q.per_block_mean = a->per_block_mean; q.smooth_k = a->smooth_k;
  q.q_codes = take(z.q_codes); q.q_sf = take(z.q_sf); q.k_codes = take(z.k_codes); q.k_sf = take(z.k_sf);
  q.vt_codes = take(z.vt_codes); q.vt_sf = take(z.vt_sf);
  q.qm = take(z.qm);
  void* km_ws = take(z.km);
  q.km = a->km_out ? a->km_out : km_ws;
  void* ds = take(z.delta_s);
  float* qk = reinterpret_cast<float*>(take(z.q_dot_km));
  q.scratch = take(z.scratch); q.scratch_bytes = z.scratch;
  int32_t* status = reinterpret_cast<int32_t*>(take(4));
  if (a->device_status) status = a->device_status;
  if (a->lse && a->smooth_k) q.q_dot_km = qk;
  if (!head_dim_ok(a->head_dim, a->shape.D)) return SAGE3_ERR_ARGUMENT;
  const int d_real = a->head_dim > 0 ? a->head_dim : a->shape.D;
  const float sm_scale = a->sm_scale > 0.f ? a->sm_scale : 1.0f / sqrtf((float)d_real);
  q.head_dim_in = a->head_dim;
  q.delta_s = a->per_block_mean >= 0 ? ds : nullptr;
  // one status word for the whole call: zeroed here, the preprocessing kernels and the attention kernel report in it
  q.device_status = status;
  {
    cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int32_t), (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  if (a->km_out && !a->smooth_k) {
    // no mean is removed: the caller's LSE correction term must vanish
    cudaError_t e = cudaMemsetAsync(a->km_out, 0, z.km, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  if (int st = sage3_quant_qkv(&q, stream)) return st;
  sage3_attn_args t{};
  t.shape = a->shape;
  t.q_codes = q.q_codes; t.q_sf = q.q_sf; t.k_codes = q.k_codes; t.k_sf = q.k_sf; t.vt_codes = q.vt_codes; t.vt_sf = q.vt_sf;
  t.delta_s = q.delta_s;
  t.delta_s_rows = a->per_block_mean == 1 ? (a->shape.Nq + 127) / 128 : 1;
  t.out = a->out; t.out_stride_b = a->out_stride_b; t.out_stride_h = a->out_stride_h; t.out_stride_n = a->out_stride_n;
  t.lse = a->lse; t.sm_scale = sm_scale; t.is_causal = a->is_causal; t.device_status = status;
  t.lse_add = q.q_dot_km;
  t.out_head_dim = a->head_dim;
  t.sm_margin = a->sm_margin;
  return attn_fwd_impl(&t, nullptr, nullptr, nullptr, stream, 0, /*zero_status=*/false);
}

int sage3_attention_varlen(const sage3_varlen_args* a, void* stream) {
  if (a == nullptr || a->workspace == nullptr || a->out == nullptr) return SAGE3_ERR_ARGUMENT;
  if (!a->q || !a->k || !a->v || !a->cu_seqlens_q || !a->cu_seqlens_k) return SAGE3_ERR_ARGUMENT;
  if ((a->out_stride_h % 8) || (a->out_stride_n % 8)) return SAGE3_ERR_ARGUMENT;
  sage3_sizes z;
  if (int st = sage3_buffer_sizes(&a->shape, 1, &z)) return st;
  if (a->workspace_bytes < z.workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) return SAGE3_ERR_ARGUMENT;
  char* w = reinterpret_cast<char*>(a->workspace);
  auto take = [&](size_t n) { char* p = w; w += align256(n); return (void*)p; };
  sage3_quant_args q{};
  q.shape = a->shape;
  q.q.ptr = a->q; q.q.stride_b = 0; q.q.stride_h = a->q_stride_h; q.q.stride_n = a->q_stride_n;
  q.k.ptr = a->k; q.k.stride_b = 0; q.k.stride_h = a->k_stride_h; q.k.stride_n = a->k_stride_n;
  q.v.ptr = a->v; q.v.stride_b = 0; q.v.stride_h = a->v_stride_h; q.v.stride_n = a->v_stride_n;
  q.per_block_mean = 1; q.smooth_k = a->smooth_k;
  q.q_codes = take(z.q_codes); q.q_sf = take(z.q_sf); q.k_codes = take(z.k_codes); q.k_sf = take(z.k_sf);
  q.vt_codes = take(z.vt_codes); q.vt_sf = take(z.vt_sf);
  q.qm = take(z.qm);
  q.km = take(z.km);
  q.delta_s = take(z.delta_s);
  take(z.q_dot_km);                                   // no LSE for packed batches (the reference returns none)
  q.scratch = take(z.scratch); q.scratch_bytes = z.scratch;
  int32_t* status = reinterpret_cast<int32_t*>(take(4));
  if (a->device_status) status = a->device_status;
  q.device_status = status;
  {
    cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int32_t), (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  if (int st = quant_qkv_impl(&q, a->cu_seqlens_q, a->cu_seqlens_k, stream)) return st;
  sage3_attn_args t{};
  t.shape = a->shape;
  t.q_codes = q.q_codes; t.q_sf = q.q_sf; t.k_codes = q.k_codes; t.k_sf = q.k_sf; t.vt_codes = q.vt_codes; t.vt_sf = q.vt_sf;
  t.delta_s = q.delta_s;
  t.delta_s_rows = (a->shape.Nq + 127) / 128;
  t.out = a->out; t.out_stride_b = 0; t.out_stride_h = a->out_stride_h; t.out_stride_n = a->out_stride_n;
  t.lse = nullptr;
  t.sm_scale = a->sm_scale > 0.f ? a->sm_scale : 1.0f / sqrtf((float)a->shape.D);
  t.is_causal = a->is_causal; t.device_status = status;
  return attn_fwd_impl(&t, nullptr, a->cu_seqlens_q, a->cu_seqlens_k, stream, 0, /*zero_status=*/false);
}

int sage3_k_mean_static(const sage3_shape* shape, const sage3_tensor* k, void* km_out, void* stream) {
  if (shape == nullptr || k == nullptr || k->ptr == nullptr || km_out == nullptr) return SAGE3_ERR_ARGUMENT;
  if (shape->B <= 0 || shape->Hkv <= 0 || shape->Nk <= 0) return SAGE3_ERR_ARGUMENT;
  if (shape->D != 64 && shape->D != 128) return SAGE3_ERR_UNSUPPORTED;
  if (int st = check_tensor(*k)) return st;
  if (!aligned16(km_out)) return SAGE3_ERR_ARGUMENT;
  bool too_large = false;
  cudaError_t e = sage3::launch_channel_mean_static(k->ptr, k->stride_b, k->stride_h, k->stride_n, shape->B, shape->Hkv,
                                                    shape->Nk, shape->D, (float)shape->Nk, km_out, (cudaStream_t)stream,
                                                    &too_large);
  if (too_large) return SAGE3_ERR_TOO_LARGE;
  if (e != cudaSuccess) return cuda_fail(e);
  return SAGE3_OK;
}

int sage3_fp4_mma_peak(int n_cols, int bursts, int launches, int32_t* device_status, void* stream_, double* tflops_out) {
  if ((n_cols != 128 && n_cols != 256) || bursts <= 0 || bursts > (1 << 16) || launches <= 0 || launches > 1024 ||
      device_status == nullptr || tflops_out == nullptr)
    return SAGE3_ERR_ARGUMENT;
  cudaStream_t stream = (cudaStream_t)stream_;
  cudaError_t e = cudaMemsetAsync(device_status, 0, sizeof(int32_t), stream);
  if (e != cudaSuccess) return cuda_fail(e);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if ((e = cudaEventCreate(&e0)) != cudaSuccess) return cuda_fail(e);
  if ((e = cudaEventCreate(&e1)) != cudaSuccess) { cudaEventDestroy(e0); return cuda_fail(e); }
  int ctas = 0;
  e = sage3::launch_fp4_mma_peak(n_cols, bursts, device_status, stream, &ctas);          // warm-up
  if (e == cudaSuccess) e = cudaEventRecord(e0, stream);
  for (int i = 0; e == cudaSuccess && i < launches; ++i)
    e = sage3::launch_fp4_mma_peak(n_cols, bursts, device_status, stream, &ctas);
  if (e == cudaSuccess) e = cudaEventRecord(e1, stream);
  if (e == cudaSuccess) e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (e != cudaSuccess) return cuda_fail(e);
  const double flops = 2.0 * 128.0 * n_cols * 64.0 * 64.0 * bursts * (double)ctas * launches;
  *tflops_out = ms > 0.f ? flops / (ms * 1e-3) / 1e12 : 0.0;
  return sage3_read_device_status(device_status, stream_, nullptr);
}

int sage3_selftest_bounded_wait(int32_t* device_status, void* stream_) {
  if (device_status == nullptr) return SAGE3_ERR_ARGUMENT;
  cudaStream_t stream = (cudaStream_t)stream_;
  cudaError_t e = cudaMemsetAsync(device_status, 0, sizeof(int32_t), stream);
  if (e != cudaSuccess) return cuda_fail(e);
  e = sage3::launch_bounded_wait_selftest(device_status, 77, stream);
  if (e != cudaSuccess) return cuda_fail(e);
  return SAGE3_OK;
}

int sage3_read_device_status(const int32_t* device_status, void* stream, int32_t* code_out) {
  if (device_status == nullptr) return SAGE3_ERR_ARGUMENT;
  int32_t h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, device_status, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e);
  if (code_out) *code_out = h;
  return h == 0 ? SAGE3_OK : SAGE3_ERR_DEVICE_WAIT;
}

}  // extern "C"
