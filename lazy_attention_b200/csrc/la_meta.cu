// Integer and table helpers of the path: the packed block table and the cos/sin
// table.  Both are pure streaming kernels (HBM-bound, a few bytes per element).
#include <cmath>

#include "la_common.cuh"

namespace la {
namespace {

// packed = block << 32 | q_offset << 16 | q_mask, element-wise over the listed rows.
__global__ void pack_kernel(const int32_t* __restrict__ bt, const int32_t* __restrict__ off,
                            const int32_t* __restrict__ msk, int64_t* __restrict__ out,
                            const int32_t* __restrict__ rows, int n_rows, int n_cols,
                            int64_t in_stride, int64_t out_stride) {
  const int64_t total = (int64_t)n_rows * n_cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int ri = (int)(i / n_cols), c = (int)(i - (int64_t)ri * n_cols);
    const int r = rows ? rows[ri] : ri;
    const int64_t src = (int64_t)r * in_stride + c;
    // Same arithmetic as int64 tensors: shift, then OR; fields that do not fit
    // carry exactly as they do in the reference.
    const int64_t v = ((int64_t)bt[src] << 32) | ((int64_t)off[src] << 16) | (int64_t)msk[src];
    out[(int64_t)r * out_stride + c] = v;
  }
}

constexpr int kMaxHalf = 128;
struct InvFreq {
  float v[kMaxHalf];
};

template <typename T>
__global__ void cos_sin_kernel(T* __restrict__ out, int64_t max_pos, int half, InvFreq inv) {
  const int64_t total = max_pos * half;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t pos = i / half;
    const int d = (int)(i - pos * half);
    const float theta = (float)pos * inv.v[d];
    out[pos * 2 * half + d] = from_f32<T>(cosf(theta));
    out[pos * 2 * half + half + d] = from_f32<T>(sinf(theta));
  }
}

// Scatter of the step's new K/V rows into the paged caches.
// One CTA per token; K is written 16 bytes at a time (the cache keeps x = 16 B
// of one token's consecutive dims together), V element by element (the cache
// keeps a dim's 16 tokens together, so one token's dims are BS elements apart).
template <typename T, typename CT>
__device__ __forceinline__ CT to_cache(T v, float scale) {
  if constexpr (sizeof(CT) == 1) {
    return CT(to_f32<T>(v) / scale);  // saturating fp8 conversion of the scaled value
  } else {
    return v;
  }
}

// One token's K and V rows into the caches (all threads of the block take part).
template <typename T, typename CT>
__device__ __forceinline__ void write_token(int64_t tok, const T* __restrict__ key, const T* __restrict__ value,
                                            CT* __restrict__ kc, CT* __restrict__ vc,
                                            const int64_t* __restrict__ slots, int64_t k_st, int64_t k_sh,
                                            int64_t v_st, int64_t v_sh, int64_t kc_sb, int64_t kc_sh,
                                            int64_t vc_sb, int64_t vc_sh, int Hkv, int D, int BS, int x,
                                            const float* k_scale, const float* v_scale) {
  const int64_t slot = slots[tok];
  if (slot < 0) return;  // padding token
  const int64_t blk = slot / BS;
  const int off = (int)(slot - blk * BS);
  const float ik = (sizeof(CT) == 1 && k_scale) ? *k_scale : 1.f;
  const float iv = (sizeof(CT) == 1 && v_scale) ? *v_scale : 1.f;
  const int n = Hkv * D;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int h = i / D, d = i - h * D;
    const T kv = key[tok * k_st + (int64_t)h * k_sh + d];
    const T vv = value[tok * v_st + (int64_t)h * v_sh + d];
    kc[blk * kc_sb + (int64_t)h * kc_sh + (int64_t)(d / x) * BS * x + (int64_t)off * x + (d % x)] =
        to_cache<T, CT>(kv, ik);
    vc[blk * vc_sb + (int64_t)h * vc_sh + (int64_t)d * BS + off] = to_cache<T, CT>(vv, iv);
  }
}

template <typename T, typename CT>
__global__ void write_cache_kernel(const T* __restrict__ key, const T* __restrict__ value, CT* __restrict__ kc,
                                   CT* __restrict__ vc, const int64_t* __restrict__ slots, int64_t k_st,
                                   int64_t k_sh, int64_t v_st, int64_t v_sh, int64_t kc_sb, int64_t kc_sh,
                                   int64_t vc_sb, int64_t vc_sh, int Hkv, int D, int BS, int x,
                                   const float* k_scale, const float* v_scale) {
  write_token<T, CT>(blockIdx.x, key, value, kc, vc, slots, k_st, k_sh, v_st, v_sh, kc_sb, kc_sh, vc_sb, vc_sh, Hkv,
                     D, BS, x, k_scale, v_scale);
}

// The same for the tokens of the requests an attention call serves: block (i, b) takes token
// i of request b.  which = 0: requests with more than one query token, or all when
// skip_decode is off (what the prefill call serves); which = 1: requests with exactly one
// query token (what the decode call serves).
template <typename T, typename CT>
__global__ void write_cache_by_request_kernel(const int32_t* __restrict__ qsl, int which, int skip_decode,
                                              const T* __restrict__ key, const T* __restrict__ value,
                                              CT* __restrict__ kc, CT* __restrict__ vc,
                                              const int64_t* __restrict__ slots, int64_t k_st, int64_t k_sh,
                                              int64_t v_st, int64_t v_sh, int64_t kc_sb, int64_t kc_sh,
                                              int64_t vc_sb, int64_t vc_sh, int Hkv, int D, int BS, int x,
                                              const float* k_scale, const float* v_scale) {
  const int b = blockIdx.y;
  const int s0 = qsl[b], qlen = qsl[b + 1] - s0;
  if ((int)blockIdx.x >= qlen) return;
  if (which == 0 && skip_decode && qlen == 1) return;
  if (which == 1 && qlen != 1) return;
  write_token<T, CT>(s0 + blockIdx.x, key, value, kc, vc, slots, k_st, k_sh, v_st, v_sh, kc_sb, kc_sh, vc_sb, vc_sh,
                     Hkv, D, BS, x, k_scale, v_scale);
}

template <typename T, typename CT>
int launch_write(const LaWriteCacheArgs& a, cudaStream_t s) {
  const int threads = 256;
  write_cache_kernel<T, CT><<<(unsigned)a.num_tokens, threads, 0, s>>>(
      (const T*)a.key, (const T*)a.value, (CT*)a.k_cache, (CT*)a.v_cache, a.slot_mapping, a.k_stride_t,
      a.k_stride_h, a.v_stride_t, a.v_stride_h, a.kc_stride_block, a.kc_stride_head, a.vc_stride_block,
      a.vc_stride_head, a.num_kv_heads, a.head_dim, a.block_size, a.x, a.k_scale, a.v_scale);
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  return LA_OK;
}

template <typename T>
int launch_write_t(const LaWriteCacheArgs& a, cudaStream_t s) {
  if (a.kv_dtype == a.dtype) return launch_write<T, T>(a, s);
  if (a.kv_dtype == LA_DTYPE_FP8_E4M3) return launch_write<T, __nv_fp8_e4m3>(a, s);
  if (a.kv_dtype == LA_DTYPE_FP8_E5M2) return launch_write<T, __nv_fp8_e5m2>(a, s);
  set_error("la_write_paged_cache: cache dtype %d with activation dtype %d unsupported", a.kv_dtype, a.dtype);
  return LA_ERR_UNSUPPORTED;
}

template <typename T, typename CT>
int launch_by_request(const int32_t* qsl, int batch, int max_q, int which, int skip_decode, const void* key,
                      const void* value, void* kc, void* vc, const int64_t* slots, int64_t k_st, int64_t k_sh,
                      int64_t v_st, int64_t v_sh, int64_t kc_sb, int64_t kc_sh, int64_t vc_sb, int64_t vc_sh, int Hkv,
                      int D, int BS, int x, const float* ks, const float* vs, cudaStream_t s) {
  dim3 grid((unsigned)max_q, (unsigned)batch);
  write_cache_by_request_kernel<T, CT><<<grid, 256, 0, s>>>(qsl, which, skip_decode, (const T*)key, (const T*)value,
                                                            (CT*)kc, (CT*)vc, slots, k_st, k_sh, v_st, v_sh, kc_sb,
                                                            kc_sh, vc_sb, vc_sh, Hkv, D, BS, x, ks, vs);
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  return LA_OK;
}

template <typename T>
int launch_by_request_t(int kv_dtype, int dtype, const int32_t* qsl, int batch, int max_q, int which, int skip_decode,
                        const void* key, const void* value, void* kc, void* vc, const int64_t* slots, int64_t k_st,
                        int64_t k_sh, int64_t v_st, int64_t v_sh, int64_t kc_sb, int64_t kc_sh, int64_t vc_sb,
                        int64_t vc_sh, int Hkv, int D, int BS, int x, const float* ks, const float* vs,
                        cudaStream_t s) {
#define LA_BY_REQ(CT)                                                                                              \
  return launch_by_request<T, CT>(qsl, batch, max_q, which, skip_decode, key, value, kc, vc, slots, k_st, k_sh, v_st, \
                                  v_sh, kc_sb, kc_sh, vc_sb, vc_sh, Hkv, D, BS, x, ks, vs, s)
  if (kv_dtype == dtype) LA_BY_REQ(T);
  if (kv_dtype == LA_DTYPE_FP8_E4M3) LA_BY_REQ(__nv_fp8_e4m3);
  if (kv_dtype == LA_DTYPE_FP8_E5M2) LA_BY_REQ(__nv_fp8_e5m2);
#undef LA_BY_REQ
  set_error("fused cache write: cache dtype %d with activation dtype %d unsupported", kv_dtype, dtype);
  return LA_ERR_UNSUPPORTED;
}

}  // namespace

// Cache write of the tokens an attention call serves, as a launch of its own: used where
// the attention kernel that was selected does not write the rows itself.
int write_cache_by_request(int kv_dtype, int dtype, const int32_t* qsl, int batch, int max_q, int which,
                           int skip_decode, const void* key, const void* value, void* kc, void* vc,
                           const int64_t* slots, int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh, int64_t kc_sb,
                           int64_t kc_sh, int64_t vc_sb, int64_t vc_sh, int Hkv, int D, int BS, int x,
                           const float* ks, const float* vs, cudaStream_t s) {
  if (batch <= 0 || max_q <= 0) return LA_OK;
#define LA_BY_REQ_T(T)                                                                                             \
  return launch_by_request_t<T>(kv_dtype, dtype, qsl, batch, max_q, which, skip_decode, key, value, kc, vc, slots,  \
                                k_st, k_sh, v_st, v_sh, kc_sb, kc_sh, vc_sb, vc_sh, Hkv, D, BS, x, ks, vs, s)
  switch (dtype) {
    case LA_DTYPE_F32: LA_BY_REQ_T(float);
    case LA_DTYPE_F16: LA_BY_REQ_T(__half);
    case LA_DTYPE_BF16: LA_BY_REQ_T(__nv_bfloat16);
    default: break;
  }
#undef LA_BY_REQ_T
  set_error("fused cache write: activation dtype %d unsupported", dtype);
  return LA_ERR_UNSUPPORTED;
}

}  // namespace la

extern "C" int la_write_paged_cache(const LaWriteCacheArgs* args, void* stream) {
  using namespace la;
  LA_REQUIRE(args != nullptr, LA_ERR_INVALID_ARGUMENT, "la_write_paged_cache: null args");
  const LaWriteCacheArgs& a = *args;
  if (a.num_tokens <= 0) return LA_OK;
  LA_REQUIRE(a.key && a.value && a.k_cache && a.v_cache && a.slot_mapping, LA_ERR_INVALID_ARGUMENT,
             "la_write_paged_cache: null tensor");
  LA_REQUIRE(a.num_kv_heads > 0 && a.head_dim > 0 && a.block_size > 0, LA_ERR_INVALID_ARGUMENT,
             "la_write_paged_cache: bad geometry");
  LA_REQUIRE(a.x == 16 / dtype_size(a.kv_dtype) && a.head_dim % a.x == 0, LA_ERR_INVALID_ARGUMENT,
             "la_write_paged_cache: x=%d does not match cache dtype %d / head_dim %d", a.x, a.kv_dtype, a.head_dim);
  cudaStream_t s = (cudaStream_t)stream;
  switch (a.dtype) {
    case LA_DTYPE_F32: return launch_write_t<float>(a, s);
    case LA_DTYPE_F16: return launch_write_t<__half>(a, s);
    case LA_DTYPE_BF16: return launch_write_t<__nv_bfloat16>(a, s);
    default:
      set_error("la_write_paged_cache: activation dtype %d unsupported", a.dtype);
      return LA_ERR_UNSUPPORTED;
  }
}

extern "C" int la_pack_block_table(const int32_t* block_table, const int32_t* q_offset,
                                   const int32_t* q_mask, int64_t* packed, const int32_t* rows,
                                   int32_t n_rows, int32_t n_cols, int64_t in_stride,
                                   int64_t packed_stride, void* stream) {
  using namespace la;
  LA_REQUIRE(block_table && q_offset && q_mask && packed, LA_ERR_INVALID_ARGUMENT,
             "la_pack_block_table: null tensor");
  LA_REQUIRE(n_rows >= 0 && n_cols >= 0 && in_stride >= n_cols && packed_stride >= n_cols,
             LA_ERR_INVALID_ARGUMENT, "la_pack_block_table: bad shape (%d x %d, strides %lld/%lld)",
             n_rows, n_cols, (long long)in_stride, (long long)packed_stride);
  if (n_rows == 0 || n_cols == 0) return LA_OK;
  const int64_t total = (int64_t)n_rows * n_cols;
  const int threads = 256;
  int blocks = (int)((total + threads - 1) / threads);
  if (blocks > 148 * 8) blocks = 148 * 8;
  pack_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(block_table, q_offset, q_mask, packed,
                                                            rows, n_rows, n_cols, in_stride,
                                                            packed_stride);
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  return LA_OK;
}

extern "C" int la_build_cos_sin_table(void* out, int32_t out_dtype, int64_t max_position,
                                      int32_t rotary_dim, double base, int32_t rope_type,
                                      double scaling_factor, double low_freq_factor,
                                      double high_freq_factor, int64_t orig_max_position,
                                      void* stream) {
  using namespace la;
  LA_REQUIRE(out != nullptr, LA_ERR_INVALID_ARGUMENT, "la_build_cos_sin_table: null output");
  LA_REQUIRE(rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim / 2 <= kMaxHalf,
             LA_ERR_UNSUPPORTED, "la_build_cos_sin_table: rotary_dim %d unsupported", rotary_dim);
  LA_REQUIRE(max_position >= 0, LA_ERR_INVALID_ARGUMENT, "la_build_cos_sin_table: max_position < 0");
  LA_REQUIRE(rope_type == 0 || rope_type == 1, LA_ERR_UNSUPPORTED,
             "la_build_cos_sin_table: rope_type %d unknown (0 plain, 1 llama3)", rope_type);
  if (max_position == 0) return LA_OK;
  const int half = rotary_dim / 2;
  InvFreq inv;
  // float32 arithmetic throughout, as the reference's torch mirror does.
  const float fbase = (float)base;
  for (int i = 0; i < half; ++i) {
    const float e = (float)(2 * i) / (float)rotary_dim;
    float f = 1.0f / powf(fbase, e);
    if (rope_type == 1) {
      const float orig = (float)orig_max_position;
      const float lo = (float)low_freq_factor, hi = (float)high_freq_factor;
      const float fac = (float)scaling_factor;
      const float wave_len = 2.0f * (float)M_PI / f;
      const float low_wl = orig / lo, high_wl = orig / hi;
      if (wave_len < high_wl) {
        // keep
      } else if (wave_len > low_wl) {
        f = f / fac;
      } else {
        const float smooth = (hi != lo) ? (orig / wave_len - lo) / (hi - lo) : 0.f;
        f = (1.0f - smooth) * f / fac + smooth * f;
      }
    }
    inv.v[i] = f;
  }
  const int64_t total = max_position * half;
  const int threads = 256;
  int64_t blocks64 = (total + threads - 1) / threads;
  const int blocks = (int)(blocks64 > 148 * 16 ? 148 * 16 : blocks64);
  cudaStream_t s = (cudaStream_t)stream;
  switch (out_dtype) {
    case LA_DTYPE_F32:
      cos_sin_kernel<float><<<blocks, threads, 0, s>>>((float*)out, max_position, half, inv);
      break;
    case LA_DTYPE_F16:
      cos_sin_kernel<__half><<<blocks, threads, 0, s>>>((__half*)out, max_position, half, inv);
      break;
    case LA_DTYPE_BF16:
      cos_sin_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((__nv_bfloat16*)out, max_position, half, inv);
      break;
    default:
      set_error("la_build_cos_sin_table: output dtype %d unsupported", out_dtype);
      return LA_ERR_UNSUPPORTED;
  }
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  return LA_OK;
}
