// General SIMT kernel of the deferred-RoPE paged attention path.
//
// One kernel serves the four reference kernels (prefill / decode, per-page
// "lazy" rotation / per-token "mepic" rotation) for every element type, cache
// type, head size that is a multiple of 32, page size that divides 32, with
// sliding window and (decode only) alibi.  It is the path for shapes and
// options the tensor-core kernels do not take, and the cross-check they are
// developed against.  K is always rotated forward on load in float32 (the
// reference decode rotates Q the other way instead; the two are the same dot
// product).
//
// Work split: a CTA owns up to 32 "rows" = (query token, query head of one KV
// group); it walks the cached pages 32 tokens at a time: all threads stage the
// chunk's K (dequantised, rotated) and V in shared memory as float32, then
// each of the 4 warps runs an online softmax for its 8 rows with one lane per
// token for the scores and one lane per 1/32 of the head dim for P.V.
#include "la_common.cuh"

namespace la {
namespace {

struct GenParams {
  int mode;
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_st, q_sh, k_st, k_sh, v_st, v_sh, o_st, o_sh;
  const void* kc;
  const void* vc;
  int64_t kc_sb, kc_sh, vc_sb, vc_sh;
  const int32_t* block_table;
  const int32_t* q_offset;
  const int32_t* q_mask;
  int64_t table_stride;
  const int64_t* packed;
  int64_t packed_stride;
  const int32_t* qsl;
  const int32_t* seq_lens;
  const uint8_t* is_lazy;
  const float* alibi;
  const float* k_scale;
  const float* v_scale;
  const void* cs;
  int64_t cs_rows;
  int cs_dtype;
  int Hq, Hkv, G, BS, x, tok_tile;
  int sliding_window, skip_decode, is_mepic, ignore_q_mask;
  float sm_scale;
};

constexpr int kChunk = 32;  // tokens staged per step
constexpr int kRows = 32;   // rows per CTA
constexpr int kRowsPerWarp = 8;
constexpr int kThreads = 128;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename QT, typename KT, int DPL>
__global__ void __launch_bounds__(kThreads) general_kernel(GenParams p) {
  constexpr int D = 32 * DPL;
  constexpr int HALF = D / 2;
  constexpr int LD = D + 1;  // padded row stride of the staged K / V
  extern __shared__ float smem[];
  float* Qs = smem;                 // [kRows][D]
  float* Ks = Qs + kRows * D;       // [kChunk][LD]
  float* Vs = Ks + kChunk * LD;     // [kChunk][LD]
  int* tok_state = reinterpret_cast<int*>(Vs + kChunk * LD);  // [kChunk] 0 absent, 1 masked, 2 valid
  int* tok_pos = tok_state + kChunk;                          // [kChunk] rotation row (<= 0: none)
  int* tok_blk = tok_pos + kChunk;                            // [kChunk] physical page

  const int b = blockIdx.z, kvh = blockIdx.y, tile = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mode = p.mode;
  const bool decode = mode >= kDecodeLazy;
  const bool mepic = (mode == kPrefillMepic) || (mode == kDecodeMepic);
  const int s0 = p.qsl[b];
  const int qlen = p.qsl[b + 1] - s0;
  const int seq_len = p.seq_lens[b];
  if (decode) {
    if (qlen != 1) return;
  } else {
    if (qlen <= 0 || (p.skip_decode && qlen == 1)) return;
  }
  const int tok0 = tile * p.tok_tile;
  if (tok0 >= qlen) return;
  const int G = p.G, BS = p.BS, x = p.x;
  const int ntok = min(p.tok_tile, qlen - tok0);
  const int nrows = ntok * G;
  const int ctx = decode ? seq_len : seq_len - qlen;
  const bool lazy = mepic ? true : (p.is_lazy != nullptr && p.is_lazy[b] != 0);
  // The scales only apply to fp8 caches (the reference dequantises nothing else).
  constexpr bool kFp8 = sizeof(KT) == 1;
  const float k_scale = (kFp8 && p.k_scale) ? *p.k_scale : 1.f;
  const float v_scale = (kFp8 && p.v_scale) ? *p.v_scale : 1.f;
  const int sw = p.sliding_window > 0 ? p.sliding_window : 0;
  const float NEG_INF = -INFINITY;

  // ---- stage Q -------------------------------------------------------------------
  {
    const QT* q = reinterpret_cast<const QT*>(p.q);
    for (int idx = tid; idx < kRows * D; idx += kThreads) {
      const int r = idx / D, d = idx - r * D;
      float val = 0.f;
      if (r < nrows) {
        const int tq = tok0 + r / G, h = kvh * G + r % G;
        val = to_f32<QT>(q[(int64_t)(s0 + tq) * p.q_st + (int64_t)h * p.q_sh + d]);
      }
      Qs[idx] = val;
    }
  }

  float m_i[kRowsPerWarp], l_i[kRowsPerWarp], acc[kRowsPerWarp][DPL];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    m_i[r] = NEG_INF;
    l_i[r] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[r][i] = 0.f;
  }

  const int ctx_pages = (ctx + BS - 1) / BS;
  const int ctx_chunks = (ctx_pages * BS + kChunk - 1) / kChunk;
  const int self_chunks = decode ? 0 : (tok0 + ntok + kChunk - 1) / kChunk;
  int carry_rot = 1;  // decode/lazy: rotation in force (1 = none); warp 0 only

  for (int c = 0; c < ctx_chunks + self_chunks; ++c) {
    const bool self = c >= ctx_chunks;
    const int base_n = (self ? c - ctx_chunks : c) * kChunk;
    __syncthreads();  // previous chunk fully consumed (and Q staged)
    // ---- per-token bookkeeping: page, rotation row, validity (warp 0) -----------
    if (warp == 0) {
      const int n = base_n + lane;
      int state = 0, pos = 0, blk = 0;
      if (!self) {
        const int j = n / BS, lip = n - j * BS;
        int rot = 0;
        if (j < ctx_pages) {
          int pad = 0;
          if (mode == kDecodeLazy || (p.packed != nullptr && mode != kDecodeMepic)) {
            const int64_t pk = p.packed[(int64_t)b * p.packed_stride + j];
            blk = (int)(pk >> 32);
            rot = (int)((pk >> 16) & 0xFFFF);
            pad = (int)(pk & 0xFFFF);
            if (p.ignore_q_mask) pad = 0;
          } else {
            blk = p.block_table[(int64_t)b * p.table_stride + j];
            if (lazy && p.q_mask) pad = p.q_mask[(int64_t)b * p.table_stride + j];
            if (lazy && p.q_offset && mode != kDecodeMepic)
              rot = p.q_offset[(int64_t)b * p.table_stride + j];
          }
          if (!lazy) { pad = 0; rot = 0; }
          const int bound = min(ctx, (j + 1) * BS - pad);
          state = (n < bound) ? 2 : 1;
          if (mode == kPrefillLazy) {
            pos = rot != 0 ? rot - 1 : 0;
          } else if (mode == kPrefillMepic) {
            pos = p.is_mepic ? n : ((rot != 0 ? rot - 1 : j * BS) + lip);
          } else if (mode == kDecodeMepic) {
            pos = n;
          }
        }
        if (mode == kDecodeLazy) {
          // 0 keeps the rotation of the page before; scan "last non-zero" over
          // the lanes, then fall back on the value carried from earlier chunks.
          int eff = (state != 0 && lazy) ? rot : 0;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, eff, o);
            if (lane >= o && eff == 0) eff = up;
          }
          if (eff == 0) eff = carry_rot;
          carry_rot = __shfl_sync(0xffffffffu, eff, 31);
          pos = lazy ? eff - 1 : 0;
        }
      } else {
        if (n < qlen) {
          state = 2;
          if (mode == kPrefillMepic) pos = ctx + n;
        }
      }
      if (pos > 0 && p.cs_rows > 0 && pos >= p.cs_rows) pos = (int)p.cs_rows - 1;
      tok_state[lane] = state;
      tok_pos[lane] = pos;
      tok_blk[lane] = blk;
    }
    __syncthreads();
    // ---- stage K (dequantise, rotate) and V -----------------------------------------
    if (!self) {
      const KT* kc = reinterpret_cast<const KT*>(p.kc);
      const KT* vc = reinterpret_cast<const KT*>(p.vc);
      const int per_page = HALF * BS;
      for (int idx = tid; idx < kChunk * HALF; idx += kThreads) {
        const int pc = idx / per_page;
        int rem = idx - pc * per_page;
        const int g = rem / (BS * x);
        rem -= g * BS * x;
        const int lip = rem / x, dx = rem - lip * x;
        const int t = pc * BS + lip, d = g * x + dx;
        float r1 = 0.f, r2 = 0.f;
        if (t < kChunk && tok_state[t] != 0) {
          const KT* base = kc + (int64_t)tok_blk[t] * p.kc_sb + (int64_t)kvh * p.kc_sh;
          const float k1 = to_f32<KT>(base[(int64_t)g * BS * x + lip * x + dx]) * k_scale;
          const int d2 = d + HALF, g2 = d2 / x, dx2 = d2 - g2 * x;
          const float k2 = to_f32<KT>(base[(int64_t)g2 * BS * x + lip * x + dx2]) * k_scale;
          const int pos = tok_pos[t];
          if (pos > 0) {
            const float cv = load_cs(p.cs, (int64_t)pos * D + d, p.cs_dtype);
            const float sv = load_cs(p.cs, (int64_t)pos * D + HALF + d, p.cs_dtype);
            r1 = k1 * cv - k2 * sv;
            r2 = k1 * sv + k2 * cv;
          } else {
            r1 = k1;
            r2 = k2;
          }
        }
        if (t < kChunk) {
          Ks[t * LD + d] = r1;
          Ks[t * LD + d + HALF] = r2;
        }
      }
      const int v_per_page = D * BS;
      for (int idx = tid; idx < kChunk * D; idx += kThreads) {
        const int pc = idx / v_per_page;
        const int rem = idx - pc * v_per_page;
        const int d = rem / BS, lip = rem - d * BS;
        const int t = pc * BS + lip;
        float val = 0.f;
        if (tok_state[t] != 0)
          val = to_f32<KT>(vc[(int64_t)tok_blk[t] * p.vc_sb + (int64_t)kvh * p.vc_sh +
                              (int64_t)d * BS + lip]) * v_scale;
        Vs[t * LD + d] = val;
      }
    } else {
      const QT* kn = reinterpret_cast<const QT*>(p.k);
      const QT* vn = reinterpret_cast<const QT*>(p.v);
      for (int idx = tid; idx < kChunk * HALF; idx += kThreads) {
        const int t = idx / HALF, d = idx - t * HALF;
        float r1 = 0.f, r2 = 0.f, v1 = 0.f, v2 = 0.f;
        if (tok_state[t] != 0) {
          const int n = base_n + t;
          const QT* kr = kn + (int64_t)(s0 + n) * p.k_st + (int64_t)kvh * p.k_sh;
          const QT* vr = vn + (int64_t)(s0 + n) * p.v_st + (int64_t)kvh * p.v_sh;
          const float k1 = to_f32<QT>(kr[d]), k2 = to_f32<QT>(kr[d + HALF]);
          v1 = to_f32<QT>(vr[d]);
          v2 = to_f32<QT>(vr[d + HALF]);
          const int pos = tok_pos[t];
          if (pos > 0) {
            const float cv = load_cs(p.cs, (int64_t)pos * D + d, p.cs_dtype);
            const float sv = load_cs(p.cs, (int64_t)pos * D + HALF + d, p.cs_dtype);
            r1 = k1 * cv - k2 * sv;
            r2 = k1 * sv + k2 * cv;
          } else {
            r1 = k1;
            r2 = k2;
          }
        }
        Ks[t * LD + d] = r1;
        Ks[t * LD + d + HALF] = r2;
        Vs[t * LD + d] = v1;
        Vs[t * LD + d + HALF] = v2;
      }
    }
    __syncthreads();
    // ---- scores, online softmax, P.V -----------------------------------------------
    const int st = tok_state[lane];
    const int n = base_n + lane;
    const float* krow = Ks + lane * LD;
#pragma unroll
    for (int rr = 0; rr < kRowsPerWarp; ++rr) {
      const int r = warp * kRowsPerWarp + rr;
      if (r >= nrows) continue;  // warp-uniform
      const int tq = tok0 + r / G;
      const float* qrow = Qs + r * D;
      float dot = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) dot = fmaf(qrow[d], krow[d], dot);
      float s;
      if (!self) {
        if (decode) {
          s = (st == 2 ? 0.f : NEG_INF) + p.sm_scale * dot;
          const int ctx_len = seq_len - 1;
          if (sw > 0 && !((ctx_len - n) < sw)) s = -10000.f;
          if (p.alibi) s += p.alibi[kvh * G + r % G] * (float)(n - ctx_len);
        } else {
          s = (st == 2) ? dot : NEG_INF;
          s *= p.sm_scale;
          if (sw > 0 && !((ctx + tq) - n < sw)) s = -10000.f;
        }
        if (st == 0) s = NEG_INF;
      } else {
        s = dot * p.sm_scale;
        if (!(tq >= n) || st == 0) s = NEG_INF;
        if (sw > 0 && !((tq - n) < sw)) s = -10000.f;
        if (st == 0) s = NEG_INF;
      }
      const float m_new = fmaxf(m_i[rr], warp_max(s));
      float pr = 0.f, alpha = 1.f;
      if (m_new != NEG_INF) {
        pr = expf(s - m_new);
        alpha = expf(m_i[rr] - m_new);
      }
      l_i[rr] = l_i[rr] * alpha + warp_sum(pr);
      m_i[rr] = m_new;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[rr][i] *= alpha;
#pragma unroll 4
      for (int t = 0; t < kChunk; ++t) {
        const float pt = __shfl_sync(0xffffffffu, pr, t);
        const float* vrow = Vs + t * LD + lane;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[rr][i] = fmaf(pt, vrow[32 * i], acc[rr][i]);
      }
    }
  }

  // ---- write out ---------------------------------------------------------------------
  QT* out = reinterpret_cast<QT*>(p.out);
#pragma unroll
  for (int rr = 0; rr < kRowsPerWarp; ++rr) {
    const int r = warp * kRowsPerWarp + rr;
    if (r >= nrows) continue;
    const int tq = tok0 + r / G, h = kvh * G + r % G;
    const float inv = l_i[rr] > 0.f ? 1.f / l_i[rr] : 0.f;
    QT* orow = out + (int64_t)(s0 + tq) * p.o_st + (int64_t)h * p.o_sh;
#pragma unroll
    for (int i = 0; i < DPL; ++i) orow[lane + 32 * i] = from_f32<QT>(acc[rr][i] * inv);
  }
}

template <typename QT, typename KT>
int launch_dpl(const GenParams& p, int D, dim3 grid, cudaStream_t stream) {
  const size_t smem = (size_t)(kRows * D + 2 * kChunk * (D + 1)) * sizeof(float) + 3 * kChunk * sizeof(int);
#define LA_GEN_CASE(DPL)                                                                      \
  case DPL: {                                                                                 \
    auto kern = general_kernel<QT, KT, DPL>;                                                  \
    if (smem > 48 * 1024)                                                                     \
      LA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                         (int)smem));                                         \
    kern<<<grid, kThreads, smem, stream>>>(p);                                                \
    break;                                                                                    \
  }
  switch (D / 32) {
    LA_GEN_CASE(1)
    LA_GEN_CASE(2)
    LA_GEN_CASE(3)
    LA_GEN_CASE(4)
    LA_GEN_CASE(6)
    LA_GEN_CASE(8)
    default:
      set_error("general kernel: head_dim %d unsupported (need 32, 64, 96, 128, 192 or 256)", D);
      return LA_ERR_UNSUPPORTED;
  }
#undef LA_GEN_CASE
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  return LA_OK;
}

template <typename QT>
int launch_kv(const GenParams& p, int D, int kv_dtype, int q_dtype, dim3 grid, cudaStream_t stream) {
  if (kv_dtype == q_dtype) return launch_dpl<QT, QT>(p, D, grid, stream);
  if (kv_dtype == LA_DTYPE_FP8_E4M3) return launch_dpl<QT, __nv_fp8_e4m3>(p, D, grid, stream);
  if (kv_dtype == LA_DTYPE_FP8_E5M2) return launch_dpl<QT, __nv_fp8_e5m2>(p, D, grid, stream);
  set_error("general kernel: cache dtype %d with activation dtype %d unsupported", kv_dtype, q_dtype);
  return LA_ERR_UNSUPPORTED;
}

int launch_q(const GenParams& p, int D, int q_dtype, int kv_dtype, dim3 grid, cudaStream_t stream) {
  switch (q_dtype) {
    case LA_DTYPE_F32: return launch_kv<float>(p, D, kv_dtype, q_dtype, grid, stream);
    case LA_DTYPE_F16: return launch_kv<__half>(p, D, kv_dtype, q_dtype, grid, stream);
    case LA_DTYPE_BF16: return launch_kv<__nv_bfloat16>(p, D, kv_dtype, q_dtype, grid, stream);
    default:
      set_error("general kernel: activation dtype %d unsupported", q_dtype);
      return LA_ERR_UNSUPPORTED;
  }
}

int check_common(int D, int BS, int x, int Hq, int Hkv) {
  LA_REQUIRE(D % 32 == 0 && D >= 32 && D <= 256, LA_ERR_UNSUPPORTED,
             "general kernel: head_dim %d must be a multiple of 32 in [32, 256]", D);
  LA_REQUIRE(BS >= 1 && BS <= 32 && (32 % BS) == 0, LA_ERR_UNSUPPORTED,
             "general kernel: block_size %d must divide 32", BS);
  LA_REQUIRE(x >= 1 && (D / 2) % x == 0, LA_ERR_UNSUPPORTED,
             "general kernel: x=%d must divide head_dim/2=%d", x, D / 2);
  LA_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 32, LA_ERR_UNSUPPORTED,
             "general kernel: %d query heads per KV head unsupported", Hkv ? Hq / Hkv : 0);
  return LA_OK;
}

}  // namespace

int launch_general_prefill(const LaPrefillArgs& a, cudaStream_t stream) {
  int rc = check_common(a.head_dim, a.block_size, a.x, a.num_q_heads, a.num_kv_heads);
  if (rc != LA_OK) return rc;
  GenParams p{};
  p.mode = a.rot_mode == LA_ROT_MEPIC ? kPrefillMepic : kPrefillLazy;
  p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out;
  p.q_st = a.q_stride_t; p.q_sh = a.q_stride_h;
  p.k_st = a.k_stride_t; p.k_sh = a.k_stride_h;
  p.v_st = a.v_stride_t; p.v_sh = a.v_stride_h;
  p.o_st = a.o_stride_t; p.o_sh = a.o_stride_h;
  p.kc = a.k_cache; p.vc = a.v_cache;
  p.kc_sb = a.kc_stride_block; p.kc_sh = a.kc_stride_head;
  p.vc_sb = a.vc_stride_block; p.vc_sh = a.vc_stride_head;
  p.block_table = a.block_table; p.q_offset = a.q_offset; p.q_mask = a.q_mask;
  p.table_stride = a.table_stride;
  p.packed = a.packed_block_table; p.packed_stride = a.packed_stride;
  p.qsl = a.query_start_loc; p.seq_lens = a.seq_lens; p.is_lazy = a.is_lazy;
  p.k_scale = a.k_scale; p.v_scale = a.v_scale;
  p.cs = a.cos_sin_cache; p.cs_rows = a.cos_sin_rows; p.cs_dtype = a.cos_sin_dtype;
  p.Hq = a.num_q_heads; p.Hkv = a.num_kv_heads; p.G = a.num_q_heads / a.num_kv_heads;
  p.BS = a.block_size; p.x = a.x;
  p.tok_tile = kRows / p.G;
  p.sliding_window = a.sliding_window; p.skip_decode = a.skip_decode; p.is_mepic = a.is_mepic;
  p.sm_scale = a.sm_scale;
  if (a.batch <= 0 || a.max_query_len <= 0) return LA_OK;
  dim3 grid((a.max_query_len + p.tok_tile - 1) / p.tok_tile, a.num_kv_heads, a.batch);
  return launch_q(p, a.head_dim, a.q_dtype, a.kv_dtype, grid, stream);
}

int launch_general_decode(const LaDecodeArgs& a, cudaStream_t stream) {
  int rc = check_common(a.head_dim, a.block_size, a.x, a.num_q_heads, a.num_kv_heads);
  if (rc != LA_OK) return rc;
  GenParams p{};
  p.mode = a.rot_mode == LA_ROT_MEPIC ? kDecodeMepic : kDecodeLazy;
  p.q = a.q; p.out = a.out;
  p.q_st = a.q_stride_t; p.q_sh = a.q_stride_h;
  p.o_st = a.o_stride_t; p.o_sh = a.o_stride_h;
  p.kc = a.k_cache; p.vc = a.v_cache;
  p.kc_sb = a.kc_stride_block; p.kc_sh = a.kc_stride_head;
  p.vc_sb = a.vc_stride_block; p.vc_sh = a.vc_stride_head;
  p.block_table = a.block_table; p.q_mask = a.q_mask; p.table_stride = a.table_stride;
  p.packed = a.packed_block_table; p.packed_stride = a.packed_stride;
  p.qsl = a.query_start_loc; p.seq_lens = a.seq_lens; p.is_lazy = a.is_lazy;
  p.alibi = a.alibi_slopes;
  p.k_scale = a.k_scale; p.v_scale = a.v_scale;
  p.cs = a.cos_sin_cache; p.cs_rows = a.cos_sin_rows; p.cs_dtype = a.cos_sin_dtype;
  p.Hq = a.num_q_heads; p.Hkv = a.num_kv_heads; p.G = a.num_q_heads / a.num_kv_heads;
  p.BS = a.block_size; p.x = a.x;
  p.tok_tile = 1;
  p.sliding_window = a.sliding_window; p.ignore_q_mask = a.ignore_q_mask;
  p.sm_scale = a.sm_scale;
  if (a.num_seqs <= 0) return LA_OK;
  dim3 grid(1, a.num_kv_heads, a.num_seqs);
  return launch_q(p, a.head_dim, a.q_dtype, a.kv_dtype, grid, stream);
}

}  // namespace la
