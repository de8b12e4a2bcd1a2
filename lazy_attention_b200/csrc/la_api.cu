// C ABI entry points: argument validation, kernel selection, error text.
#include <cstring>

#include "la_common.cuh"
#include "la_sm100.cuh"

namespace la {

static thread_local char g_err[512] = {0};
std::atomic<int64_t> g_launch_count{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

__device__ int g_device_status[4];

// Device address of the status word on the current device, looked up once per device.
int* device_status_ptr() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int*> cached[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  int* ptr = cached[dev].load(std::memory_order_acquire);
  if (ptr != nullptr) return ptr;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_device_status) != cudaSuccess) return nullptr;
  cached[dev].store(reinterpret_cast<int*>(sym), std::memory_order_release);
  return reinterpret_cast<int*>(sym);
}

namespace {

bool is_act_dtype(int dt) { return dt == LA_DTYPE_F32 || dt == LA_DTYPE_F16 || dt == LA_DTYPE_BF16; }
bool is_fp8(int dt) { return dt == LA_DTYPE_FP8_E4M3 || dt == LA_DTYPE_FP8_E5M2; }

int validate_prefill(const LaPrefillArgs* a) {
  LA_REQUIRE(a != nullptr, LA_ERR_INVALID_ARGUMENT, "la_prefill_fwd: null args");
  LA_REQUIRE(a->batch >= 0, LA_ERR_INVALID_ARGUMENT, "la_prefill_fwd: batch %d < 0", a->batch);
  if (a->batch == 0 || a->max_query_len <= 0) return LA_OK;
  LA_REQUIRE(a->q && a->k && a->v && a->out, LA_ERR_INVALID_ARGUMENT, "la_prefill_fwd: null q/k/v/out");
  LA_REQUIRE(a->k_cache && a->v_cache && (a->block_table || a->packed_block_table), LA_ERR_INVALID_ARGUMENT,
             "la_prefill_fwd: null cache or block table");
  LA_REQUIRE(a->query_start_loc && a->seq_lens, LA_ERR_INVALID_ARGUMENT,
             "la_prefill_fwd: null query_start_loc / seq_lens");
  LA_REQUIRE(is_act_dtype(a->q_dtype), LA_ERR_INVALID_ARGUMENT, "la_prefill_fwd: q dtype %d", a->q_dtype);
  LA_REQUIRE(a->kv_dtype == a->q_dtype || is_fp8(a->kv_dtype), LA_ERR_INVALID_ARGUMENT,
             "la_prefill_fwd: cache dtype %d does not match activations (%d) and is not fp8",
             a->kv_dtype, a->q_dtype);
  LA_REQUIRE(a->num_kv_heads > 0 && a->num_q_heads > 0 && a->num_q_heads % a->num_kv_heads == 0,
             LA_ERR_INVALID_ARGUMENT, "la_prefill_fwd: heads %d / %d", a->num_q_heads, a->num_kv_heads);
  LA_REQUIRE(a->head_dim > 0 && a->rotary_dim == a->head_dim, LA_ERR_UNSUPPORTED,
             "la_prefill_fwd: rotary_dim %d must equal head_dim %d", a->rotary_dim, a->head_dim);
  LA_REQUIRE(a->x == 16 / dtype_size(a->kv_dtype), LA_ERR_INVALID_ARGUMENT,
             "la_prefill_fwd: x=%d does not match 16 bytes of cache dtype %d", a->x, a->kv_dtype);
  LA_REQUIRE(a->rot_mode == LA_ROT_LAZY || a->rot_mode == LA_ROT_MEPIC, LA_ERR_INVALID_ARGUMENT,
             "la_prefill_fwd: rot_mode %d", a->rot_mode);
  const bool needs_table = a->rot_mode == LA_ROT_MEPIC || a->is_lazy != nullptr;
  if (needs_table) {
    LA_REQUIRE(a->cos_sin_cache != nullptr && a->cos_sin_rows > 0, LA_ERR_INVALID_ARGUMENT,
               "la_prefill_fwd: rotation requested without a cos/sin table");
    LA_REQUIRE(is_act_dtype(a->cos_sin_dtype), LA_ERR_INVALID_ARGUMENT,
               "la_prefill_fwd: cos/sin dtype %d", a->cos_sin_dtype);
    LA_REQUIRE(a->q_mask != nullptr || a->packed_block_table != nullptr, LA_ERR_INVALID_ARGUMENT,
               "la_prefill_fwd: q_mask is null");
    LA_REQUIRE(a->q_offset != nullptr || a->packed_block_table != nullptr ||
                   (a->rot_mode == LA_ROT_MEPIC && a->is_mepic),
               LA_ERR_INVALID_ARGUMENT, "la_prefill_fwd: q_offset is null");
  }
  return LA_OK;
}

int validate_decode(const LaDecodeArgs* a) {
  LA_REQUIRE(a != nullptr, LA_ERR_INVALID_ARGUMENT, "la_decode_fwd: null args");
  LA_REQUIRE(a->num_seqs >= 0, LA_ERR_INVALID_ARGUMENT, "la_decode_fwd: num_seqs %d < 0", a->num_seqs);
  if (a->num_seqs == 0) return LA_OK;
  LA_REQUIRE(a->q && a->out && a->k_cache && a->v_cache, LA_ERR_INVALID_ARGUMENT,
             "la_decode_fwd: null q/out/cache");
  LA_REQUIRE(a->query_start_loc && a->seq_lens, LA_ERR_INVALID_ARGUMENT,
             "la_decode_fwd: null query_start_loc / seq_lens");
  LA_REQUIRE(is_act_dtype(a->q_dtype), LA_ERR_INVALID_ARGUMENT, "la_decode_fwd: q dtype %d", a->q_dtype);
  LA_REQUIRE(a->kv_dtype == a->q_dtype || is_fp8(a->kv_dtype), LA_ERR_INVALID_ARGUMENT,
             "la_decode_fwd: cache dtype %d does not match activations (%d) and is not fp8",
             a->kv_dtype, a->q_dtype);
  LA_REQUIRE(a->num_kv_heads > 0 && a->num_q_heads > 0 && a->num_q_heads % a->num_kv_heads == 0,
             LA_ERR_INVALID_ARGUMENT, "la_decode_fwd: heads %d / %d", a->num_q_heads, a->num_kv_heads);
  LA_REQUIRE(a->head_dim > 0 && a->rotary_dim == a->head_dim, LA_ERR_UNSUPPORTED,
             "la_decode_fwd: rotary_dim %d must equal head_dim %d", a->rotary_dim, a->head_dim);
  LA_REQUIRE(a->x == 16 / dtype_size(a->kv_dtype), LA_ERR_INVALID_ARGUMENT,
             "la_decode_fwd: x=%d does not match 16 bytes of cache dtype %d", a->x, a->kv_dtype);
  if (a->rot_mode == LA_ROT_LAZY) {
    LA_REQUIRE(a->packed_block_table != nullptr, LA_ERR_INVALID_ARGUMENT,
               "la_decode_fwd: lazy mode needs the packed block table");
    if (a->is_lazy)
      LA_REQUIRE((a->cos_sin_cache != nullptr && a->cos_sin_rows > 0) || a->compute_cos_sin, LA_ERR_INVALID_ARGUMENT,
                 "la_decode_fwd: rotation requested without a cos/sin table or RoPE parameters");
  } else if (a->rot_mode == LA_ROT_MEPIC) {
    LA_REQUIRE(a->block_table != nullptr && a->q_mask != nullptr, LA_ERR_INVALID_ARGUMENT,
               "la_decode_fwd: per-token mode needs block_table and q_mask");
    LA_REQUIRE(a->cos_sin_cache != nullptr && a->cos_sin_rows > 0, LA_ERR_INVALID_ARGUMENT,
               "la_decode_fwd: rotation requested without a cos/sin table");
  } else {
    set_error("la_decode_fwd: rot_mode %d", a->rot_mode);
    return LA_ERR_INVALID_ARGUMENT;
  }
  return LA_OK;
}

}  // namespace
}  // namespace la

namespace la {
int validate_prefill_args(const LaPrefillArgs* a) { return validate_prefill(a); }
}  // namespace la

using namespace la;

extern "C" int la_prefill_fwd(const LaPrefillArgs* args, void* stream) {
  int rc = validate_prefill(args);
  if (rc != LA_OK) return rc;
  if (args->batch == 0 || args->max_query_len <= 0) return LA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const char* why = "";
  // The general kernel does not store the new K/V rows itself: where it serves the call,
  // the fused cache write runs as a launch of its own just before it.
  auto general = [&]() -> int {
    const LaPrefillArgs& a = *args;
    if (a.slot_mapping != nullptr) {
      int wrc = write_cache_by_request(a.kv_dtype, a.q_dtype, a.query_start_loc, a.batch, a.max_query_len, 0,
                                       a.skip_decode, a.k, a.v, const_cast<void*>(a.k_cache),
                                       const_cast<void*>(a.v_cache), a.slot_mapping, a.k_stride_t, a.k_stride_h,
                                       a.v_stride_t, a.v_stride_h, a.kc_stride_block, a.kc_stride_head,
                                       a.vc_stride_block, a.vc_stride_head, a.num_kv_heads, a.head_dim, a.block_size,
                                       a.x, a.k_scale, a.v_scale, s);
      if (wrc != LA_OK) return wrc;
    }
    return launch_general_prefill(a, s);
  };
  if (args->kernel == LA_KERNEL_GENERAL) {
    LA_REQUIRE(args->peer.num_peers == 0, LA_ERR_UNSUPPORTED, "la_prefill_fwd: the general kernel has no fused output gather");
    LA_REQUIRE(args->q_positions == nullptr, LA_ERR_UNSUPPORTED, "la_prefill_fwd: the general kernel has no fused rotary op");
    return general();
  }
  const bool tc_ok = tc_prefill_supported(*args, &why);
  LA_REQUIRE(tc_ok || args->q_positions == nullptr, LA_ERR_UNSUPPORTED,
             "la_prefill_fwd: the fused rotary op needs the tensor-core kernel, unavailable here: %s", why);
  if (args->kernel == LA_KERNEL_TENSOR) {
    LA_REQUIRE(tc_ok, LA_ERR_UNSUPPORTED, "la_prefill_fwd: tensor-core kernel unavailable: %s", why);
    return launch_tc_prefill(*args, s);
  }
  // Automatic selection: the tensor-core kernel whenever the arguments fit it.  A missing
  // or short workspace is then an error of the call (launch_tc_prefill reports the size
  // needed), never a reason to run the far slower general kernel unasked.
  if (tc_ok) return launch_tc_prefill(*args, s);
  LA_REQUIRE(args->peer.num_peers == 0, LA_ERR_UNSUPPORTED,
             "la_prefill_fwd: the fused output gather needs the tensor-core kernel (%s)", why);
  return general();
}

extern "C" int la_decode_fwd(const LaDecodeArgs* args, void* stream) {
  int rc = validate_decode(args);
  if (rc != LA_OK) return rc;
  if (args->num_seqs == 0) return LA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const char* why = "";
  if (args->slot_mapping != nullptr)
    LA_REQUIRE(args->key != nullptr && args->value != nullptr, LA_ERR_INVALID_ARGUMENT,
               "la_decode_fwd: slot_mapping given without the step's key / value rows");
  // as in la_prefill_fwd: the general kernel leaves the cache write to a launch of its own
  auto general = [&]() -> int {
    const LaDecodeArgs& a = *args;
    if (a.slot_mapping != nullptr) {
      int wrc = write_cache_by_request(a.kv_dtype, a.q_dtype, a.query_start_loc, a.num_seqs, 1, 1, 0, a.key, a.value,
                                       const_cast<void*>(a.k_cache), const_cast<void*>(a.v_cache), a.slot_mapping,
                                       a.k_stride_t, a.k_stride_h, a.v_stride_t, a.v_stride_h, a.kc_stride_block,
                                       a.kc_stride_head, a.vc_stride_block, a.vc_stride_head, a.num_kv_heads,
                                       a.head_dim, a.block_size, a.x, a.k_scale, a.v_scale, s);
      if (wrc != LA_OK) return wrc;
    }
    return launch_general_decode(a, s);
  };
  if (args->kernel == LA_KERNEL_GENERAL) {
    LA_REQUIRE(args->peer.num_peers == 0, LA_ERR_UNSUPPORTED, "la_decode_fwd: the general kernel has no fused output gather");
    LA_REQUIRE(args->q_positions == nullptr && !(args->compute_cos_sin && args->cos_sin_cache == nullptr),
               LA_ERR_UNSUPPORTED, "la_decode_fwd: the general kernel has no fused rotary op / in-kernel cos/sin");
    return general();
  }
  const bool fast_ok = fast_decode_supported(*args, &why);
  LA_REQUIRE(fast_ok || (args->q_positions == nullptr && !(args->compute_cos_sin && args->cos_sin_cache == nullptr)),
             LA_ERR_UNSUPPORTED,
             "la_decode_fwd: the fused rotary op / in-kernel cos/sin need the split-KV kernel, unavailable here: %s", why);
  if (args->kernel == LA_KERNEL_TENSOR) {
    LA_REQUIRE(fast_ok, LA_ERR_UNSUPPORTED, "la_decode_fwd: split-KV kernel unavailable: %s", why);
    return launch_fast_decode(*args, s);
  }
  // As above: a missing or short workspace is reported, not papered over by the general kernel.
  if (fast_ok) return launch_fast_decode(*args, s);
  LA_REQUIRE(args->peer.num_peers == 0, LA_ERR_UNSUPPORTED,
             "la_decode_fwd: the fused output gather needs the split-KV kernel (%s)", why);
  return general();
}

extern "C" size_t la_prefill_workspace_bytes(const LaPrefillArgs* args) {
  if (!args || args->kernel == LA_KERNEL_GENERAL) return 0;
  const char* why = "";
  if (!tc_prefill_supported(*args, &why)) return 0;
  return tc_prefill_workspace_bytes(*args);
}

extern "C" size_t la_decode_workspace_bytes(const LaDecodeArgs* args) {
  if (!args || args->kernel == LA_KERNEL_GENERAL) return 0;
  const char* why = "";
  if (!fast_decode_supported(*args, &why)) return 0;
  return fast_decode_workspace_bytes(*args);
}

extern "C" const char* la_last_error(void) { return la::g_err; }
extern "C" int la_version(void) { return LA_VERSION; }
extern "C" int64_t la_launch_count(void) { return la::g_launch_count.load(); }
extern "C" size_t la_sizeof_prefill_args(void) { return sizeof(LaPrefillArgs); }
extern "C" size_t la_sizeof_decode_args(void) { return sizeof(LaDecodeArgs); }
extern "C" int la_device_status(void) {
  int host[4] = {0, 0, 0, 0};
  LA_CHECK_CUDA(cudaDeviceSynchronize());
  LA_CHECK_CUDA(cudaMemcpyFromSymbol(host, la::g_device_status, sizeof(host)));
  if (host[0] != 0) {
    int zero[4] = {0, 0, 0, 0};
    LA_CHECK_CUDA(cudaMemcpyToSymbol(la::g_device_status, zero, sizeof(zero)));
  }
  return host[0];
}

extern "C" int la_check_device(void) {
  const int code = la_device_status();
  if (code < 0) return code;  // the query itself failed
  LA_REQUIRE(code == 0, LA_ERR_DEVICE_STATUS,
             "a kernel gave up on a bounded wait (code %d): results of calls since the last check are invalid", code);
  return LA_OK;
}

// ---- buffers of the fused output gather, shared across processes with CUDA IPC ---------------
extern "C" int la_peer_alloc(size_t bytes, void** out) {
  LA_REQUIRE(out != nullptr && bytes > 0, LA_ERR_INVALID_ARGUMENT, "la_peer_alloc: null result or zero size");
  *out = nullptr;
  void* ptr = nullptr;
  LA_CHECK_CUDA(cudaMalloc(&ptr, bytes));
  cudaError_t e = cudaMemset(ptr, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(ptr);
    la::set_error("la_peer_alloc: cudaMemset failed: %s", cudaGetErrorString(e));
    return LA_ERR_CUDA;
  }
  *out = ptr;
  return LA_OK;
}

extern "C" int la_peer_export(const void* buffer, unsigned char handle[LA_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == LA_IPC_HANDLE_BYTES, "IPC handle size");
  LA_REQUIRE(buffer != nullptr && handle != nullptr, LA_ERR_INVALID_ARGUMENT, "la_peer_export: null argument");
  cudaIpcMemHandle_t h;
  LA_CHECK_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(buffer)));
  std::memcpy(handle, &h, sizeof(h));
  return LA_OK;
}

extern "C" int la_peer_open(const unsigned char handle[LA_IPC_HANDLE_BYTES], void** out) {
  LA_REQUIRE(handle != nullptr && out != nullptr, LA_ERR_INVALID_ARGUMENT, "la_peer_open: null argument");
  *out = nullptr;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* ptr = nullptr;
  LA_CHECK_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  *out = ptr;
  return LA_OK;
}

extern "C" int la_peer_close(void* mapped) {
  if (mapped == nullptr) return LA_OK;
  LA_CHECK_CUDA(cudaIpcCloseMemHandle(mapped));
  return LA_OK;
}

// ---- end-of-step barrier of the fused gather -------------------------------------------------
// Signal buffer of a rank (LA_PEER_SIGNAL_BYTES, zero at allocation): word r = the last round
// rank r has announced to this rank, word kRoundWord = this rank's own round counter.
namespace la {
namespace {
constexpr int kRoundWord = 32;
constexpr uint64_t kBarrierLimitNs = 10000ull * 1000 * 1000;  // ranks are processes: allow for host-side skew
struct PeerSignals {
  uint32_t* ptr[LA_MAX_PEERS];
};

__global__ void peer_barrier_kernel(PeerSignals s, int world, int rank, uint64_t limit_ns, int* status) {
  const int lane = threadIdx.x;
  uint32_t* mine = s.ptr[rank];
  const uint32_t round = *reinterpret_cast<volatile uint32_t*>(mine + kRoundWord) + 1u;
  __syncwarp();
  if (lane == 0) *reinterpret_cast<volatile uint32_t*>(mine + kRoundWord) = round;
  if (lane >= world) return;
  // The kernels launched before this one on the stream have completed, so their stores into
  // the peers' buffers have been performed; the fence orders this thread's announcement
  // after them for an observer on another GPU.
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(s.ptr[lane] + rank), "r"(round) : "memory");
  const uint32_t* from = mine + lane;
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while (true) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(from) : "memory");
    // a rank can be one round ahead (it has passed this barrier and reached the next)
    if ((int32_t)(seen - round) >= 0) break;
    if ((++polls & 63u) == 0) {
      const uint64_t now = sm100::global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, 300 + lane);  // rank `lane` never arrived
        break;
      }
    }
  }
}
}  // namespace
}  // namespace la

extern "C" int la_peer_barrier(void* const* signals, int32_t world, int32_t rank, void* stream) {
  LA_REQUIRE(signals != nullptr, LA_ERR_INVALID_ARGUMENT, "la_peer_barrier: null signals");
  LA_REQUIRE(world >= 1 && world <= LA_MAX_PEERS && rank >= 0 && rank < world, LA_ERR_INVALID_ARGUMENT,
             "la_peer_barrier: rank %d of %d (at most %d ranks)", rank, world, LA_MAX_PEERS);
  la::PeerSignals s;
  for (int r = 0; r < LA_MAX_PEERS; ++r) s.ptr[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    LA_REQUIRE(signals[r] != nullptr && (reinterpret_cast<uintptr_t>(signals[r]) & 3) == 0, LA_ERR_INVALID_ARGUMENT,
               "la_peer_barrier: signal buffer of rank %d is null or unaligned", r);
    s.ptr[r] = reinterpret_cast<uint32_t*>(signals[r]);
  }
  uint64_t limit_ns = la::kBarrierLimitNs;
  if (const char* e = getenv("LAZY_ATTN_B200_BARRIER_LIMIT_MS")) {  // tests of the expiry path
    const long ms = atol(e);
    if (ms >= 1 && ms <= 60000) limit_ns = (uint64_t)ms * 1000000ull;
  }
  la::peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, world, rank, limit_ns, la::device_status_ptr());
  LA_CHECK_CUDA(cudaGetLastError());
  la::count_launch();
  return LA_OK;
}

extern "C" int la_peer_free(void* buffer) {
  if (buffer == nullptr) return LA_OK;
  LA_CHECK_CUDA(cudaFree(buffer));
  return LA_OK;
}
