// Shared declarations of the lazy_attention_b200 CUDA sources.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/lazy_attention_b200.h"

namespace la {

// ---- host-side error reporting -------------------------------------------------
void set_error(const char* fmt, ...);
extern std::atomic<int64_t> g_launch_count;
inline void count_launch(int n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }

#define LA_CHECK_CUDA(expr)                                                       \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      la::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),       \
                    __FILE__, __LINE__);                                          \
      return LA_ERR_CUDA;                                                         \
    }                                                                             \
  } while (0)

#define LA_REQUIRE(cond, code, ...)                                               \
  do {                                                                            \
    if (!(cond)) {                                                                \
      la::set_error(__VA_ARGS__);                                                 \
      return (code);                                                              \
    }                                                                             \
  } while (0)

// ---- element helpers --------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_fp8_e5m2>(__nv_fp8_e5m2 v) { return float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// cos/sin table element read with a run-time dtype (F32 / F16 / BF16).
__device__ __forceinline__ float load_cs(const void* base, int64_t idx, int dtype) {
  if (dtype == LA_DTYPE_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == LA_DTYPE_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

inline int dtype_size(int dt) {
  switch (dt) {
    case LA_DTYPE_F32: return 4;
    case LA_DTYPE_F16: return 2;
    case LA_DTYPE_BF16: return 2;
    case LA_DTYPE_FP8_E4M3: return 1;
    case LA_DTYPE_FP8_E5M2: return 1;
    default: return 0;
  }
}

// Argument checks of la_prefill_fwd, for entry points defined in other files.
int validate_prefill_args(const LaPrefillArgs* a);

// Device status word shared by the kernels with bounded waits (0 = fine).
int* device_status_ptr();

// ---- kernel launchers (one per .cu file) ------------------------------------------
// What kind of call the general kernel is serving.
enum GeneralMode : int {
  kPrefillLazy = 0,
  kPrefillMepic = 1,
  kDecodeLazy = 2,
  kDecodeMepic = 3,
};

int launch_general_prefill(const LaPrefillArgs& a, cudaStream_t stream);
int launch_general_decode(const LaDecodeArgs& a, cudaStream_t stream);

// Tensor-core prefill (TMA + tcgen05).  `supported` tells whether the arguments
// fit the kernel's constraints; the launcher assumes they do.
bool tc_prefill_supported(const LaPrefillArgs& a, const char** why);
size_t tc_prefill_workspace_bytes(const LaPrefillArgs& a);
int launch_tc_prefill(const LaPrefillArgs& a, cudaStream_t stream);

// Cache write of the tokens an attention call serves, as a launch of its own (la_meta.cu).
int write_cache_by_request(int kv_dtype, int dtype, const int32_t* qsl, int batch, int max_q, int which,
                           int skip_decode, const void* key, const void* value, void* kc, void* vc,
                           const int64_t* slots, int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh, int64_t kc_sb,
                           int64_t kc_sh, int64_t vc_sb, int64_t vc_sh, int Hkv, int D, int BS, int x,
                           const float* ks, const float* vs, cudaStream_t s);

// Split-KV decode (bulk-copy ring + mma).
bool fast_decode_supported(const LaDecodeArgs& a, const char** why);
size_t fast_decode_workspace_bytes(const LaDecodeArgs& a);
int launch_fast_decode(const LaDecodeArgs& a, cudaStream_t stream);

}  // namespace la
