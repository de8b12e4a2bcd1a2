// Split-KV paged decode kernel for sm_100a (HBM-bound path).
//
// One CTA owns a contiguous run of pages of one (sequence, KV head).  Each warp
// streams its own 2-page tiles (K and V pages of 16 tokens) from the paged cache
// into a private shared-memory ring with bulk async copies (one contiguous
// D*16*e-byte chunk per page and tensor), and consumes them with warp-level
// tensor-core MMAs in the "tokens on M" orientation:
//     S^T[16 tok x 8 heads] = K[16 tok x D] * Q^T[D x 8 heads]     (D/16 MMAs per page)
//     O^T[D x 8 heads]     += V^T[D x 16 tok] * P^T[16 tok x 8 heads] (D/16 MMAs per page)
// so the K and V fragments are read straight from the cache's page layouts
// ([D/x][16][x] and [D][16]) with one 4- or 8-byte shared load each, and an fp8
// cache is dequantised in registers (e4m3/e5m2 -> f16, exact) with the scales
// folded into the score scale and the final normalisation.  The rotation of the
// "lazy" variant is applied to Q (inverse rotation by the page's offset, rebuilt
// from the original Q whenever the offset changes), as the reference decode does.
// Partial results of the splits are merged by a second small kernel.
#include <cstdlib>

#include <atomic>

#include "la_common.cuh"
#include "la_sm100.cuh"

namespace la {
namespace {

using namespace sm100;

struct DecParams {
  const void* q;
  void* out;
  int64_t q_st, q_sh, o_st, o_sh;
  const uint8_t* kc;
  const uint8_t* vc;
  int64_t kc_sb, kc_sh, vc_sb, vc_sh;  // bytes
  int64_t num_blocks;
  const int64_t* packed;
  int64_t packed_stride;
  const int32_t* block_table;  // per-token mode: plain tables
  const int32_t* q_mask;
  int64_t table_stride;
  const int32_t* qsl;
  const int32_t* seq_lens;
  const uint8_t* is_lazy;
  const float* k_scale;
  const float* v_scale;
  const void* cs;
  int64_t cs_rows;
  int Hq, Hkv, G;
  int chunk_pages, n_splits, ignore_q_mask;
  float sm_scale;
  LaPeerOut peer;  // fused output gather: result rows go to every rank's buffer instead of `out`
  // fused cache write of the new token's K/V row (slots == nullptr: off)
  const void* key;
  const void* value;
  int64_t k_st, k_sh, v_st, v_sh;
  const int64_t* slots;
  const int64_t* q_pos;  // fused rotary op on the query (nullptr: the query arrives rotated)
  // in-kernel cos/sin (compute_cs != 0): parameters of the inverse frequencies
  int compute_cs, rope_type, rope_orig;
  float rope_base, rope_factor, rope_low, rope_high;
  float* part_o;   // [num_seqs][Hq][n_splits][D]
  float* part_ml;  // [num_seqs][Hq][n_splits][2]
  int* status;
};

template <int D, int KV>
struct DecCfg {
  static constexpr int kElem = KV == 0 ? 2 : 1;
  static constexpr int kPageBytes = D * 16 * kElem;
  // pages per tile: as many as make a tile of 8 KB (K pages, then V pages) -- one 4 KB page
  // (16-bit, head_dim 128), two 2 KB pages, four 1 KB pages (8-bit, head_dim 64: 0.633 -> 0.593 ms
  // on the 256-sequence workload against two) -- so that every configuration runs as small CTAs
  static constexpr int kPPT = kPageBytes > 2048 ? 1 : (kPageBytes > 1024 ? 2 : 4);
  static constexpr int kTileBytes = 2 * kPPT * kPageBytes;
  // Small CTAs of 4 warps with a 64 KB ring, three of them per SM, so that one
  // CTA's prologue and merge overlap the others' streaming (measured on the fp8
  // decode configuration: 8 warps x 3 stages x 1 CTA 4.7 TB/s, 12 x 2 x 1 5.2,
  // 4 x 2 x 3 6.15).
  static constexpr int kWarps = 4;
  static constexpr int kStages = 65536 / (kWarps * kTileBytes);
  static constexpr int kMinBlocks = 3;
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kMaxChunkPages = 512;
  static constexpr int kRingBytes = kWarps * kStages * kTileBytes;
  static constexpr int kMergeBytes = kWarps * 8 * (D + 2) * 4;
  static constexpr int kSmemBytes = (kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes) + 128;
};

// token held by MMA row r (r < 8) of a page; row r + 8 holds sigma(r) ^ 2
__device__ __forceinline__ int sigma(int r) { return 4 * (r >> 1) + (r & 1) + ((r >> 2) << 1); }

template <bool BF16MMA>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  if constexpr (BF16MMA) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

template <bool BF16MMA>
__device__ __forceinline__ uint32_t pack_mma(float a, float b) {
  if constexpr (BF16MMA) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
template <bool BF16>
__device__ __forceinline__ float2 unpack_q(uint32_t u) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}
// four fp8 values (one 32-bit word) -> two f16x2 registers: lo = values 0,1; hi = values 2,3
template <int KV>
__device__ __forceinline__ void fp8x4_to_h2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  if constexpr (KV == 1) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(w));
  } else {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e5m2x2 %0, l;\n\tcvt.rn.f16x2.e5m2x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(w));
  }
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// n consecutive activations (BF16 or f16 bits) -> cache elements at dst: copied as they are for
// a 16-bit cache, converted like la_write_paged_cache does (saturating fp8 of value / scale)
// for an 8-bit one.
template <int KV, bool BF16>
__device__ __forceinline__ void to_cache_elems(const uint16_t* src, int n, uint8_t* dst, float scale) {
  for (int i = 0; i < n; ++i) {
    if constexpr (KV == 0) {
      reinterpret_cast<uint16_t*>(dst)[i] = src[i];
    } else {
      float f;
      if constexpr (BF16) f = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&src[i]));
      else f = __half2float(*reinterpret_cast<const __half*>(&src[i]));
      if constexpr (KV == 1) {
        const __nv_fp8_e4m3 c(f / scale);
        dst[i] = *reinterpret_cast<const uint8_t*>(&c);
      } else {
        const __nv_fp8_e5m2 c(f / scale);
        dst[i] = *reinterpret_cast<const uint8_t*>(&c);
      }
    }
  }
}

// Inverse RoPE frequency of dimension pair i of D/2, float32, with the llama3 wavelength
// smoothing when rope_type == 1 (lazy_attn/lazy/model_executor/rope/cos_sin.py:38-59).
template <int D>
__device__ __forceinline__ float rope_inv_freq(const DecParams& p, int i) {
  const float inv = 1.0f / powf(p.rope_base, (float)(2 * i) / (float)D);
  if (p.rope_type != 1) return inv;
  const float wave_len = 6.283185307179586f / inv;
  const float low_wl = (float)p.rope_orig / p.rope_low, high_wl = (float)p.rope_orig / p.rope_high;
  if (wave_len < high_wl) return inv;
  if (wave_len > low_wl) return inv / p.rope_factor;
  const float smooth = ((float)p.rope_orig / wave_len - p.rope_low) / (p.rope_high - p.rope_low);
  return (1.f - smooth) * inv / p.rope_factor + smooth * inv;
}

// cos / sin of position x inverse frequency for dims d0 and d0 + 1, in float32 (the reference's
// COMPUTE_COS_SIN branch, ops/models/llama_v1.py:212-214).  Out of line: the range reduction of
// sincosf is long, and inlined at every rotation change it weighed on the whole tile loop.
template <int D>
__device__ __noinline__ void rope_cos_sin_pair(const DecParams& p, int pos, int d0, float2& cc, float2& ss) {
  const float t0 = (float)pos * rope_inv_freq<D>(p, d0);
  const float t1 = (float)pos * rope_inv_freq<D>(p, d0 + 1);
  float s0, c0, s1, c1;
  sincosf(t0, &s0, &c0);
  sincosf(t1, &s1, &c1);
  cc = make_float2(c0, c1);
  ss = make_float2(s0, s1);
}

// Forward rotation of two packed key pairs (dims d, d+1 and their partners D/2 further) in the
// MMA's own 16-bit type: k1' = k1*c - k2*s, k2' = k1*s + k2*c, two roundings per result as the
// reference's 16-bit evaluation has (old_ops/chunked_prefill_paged_decode.py:228-229).
template <bool BF16MMA>
__device__ __forceinline__ void rotate_pair(uint32_t& k1, uint32_t& k2, uint32_t c, uint32_t s) {
  const uint32_t nk2 = k2 ^ 0x80008000u;
  if constexpr (BF16MMA) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&k1), b = *reinterpret_cast<const __nv_bfloat162*>(&k2);
    const __nv_bfloat162 nb = *reinterpret_cast<const __nv_bfloat162*>(&nk2);
    const __nv_bfloat162 cc = *reinterpret_cast<const __nv_bfloat162*>(&c), ss = *reinterpret_cast<const __nv_bfloat162*>(&s);
    const __nv_bfloat162 r1 = __hfma2(nb, ss, __hmul2(a, cc));
    const __nv_bfloat162 r2 = __hfma2(a, ss, __hmul2(b, cc));
    k1 = *reinterpret_cast<const uint32_t*>(&r1);
    k2 = *reinterpret_cast<const uint32_t*>(&r2);
  } else {
    const __half2 a = *reinterpret_cast<const __half2*>(&k1), b = *reinterpret_cast<const __half2*>(&k2);
    const __half2 nb = *reinterpret_cast<const __half2*>(&nk2);
    const __half2 cc = *reinterpret_cast<const __half2*>(&c), ss = *reinterpret_cast<const __half2*>(&s);
    const __half2 r1 = __hfma2(nb, ss, __hmul2(a, cc));
    const __half2 r2 = __hfma2(a, ss, __hmul2(b, cc));
    k1 = *reinterpret_cast<const uint32_t*>(&r1);
    k2 = *reinterpret_cast<const uint32_t*>(&r2);
  }
}

// One output element: to `out`, or with the fused gather to the same place of every rank's buffer.
template <bool BF16>
__device__ __forceinline__ void store_result(const DecParams& p, int row_q, int head, int d, float val) {
  uint16_t bits;
  if constexpr (BF16) {
    const __nv_bfloat16 h = __float2bfloat16_rn(val);
    bits = *reinterpret_cast<const uint16_t*>(&h);
  } else {
    const __half h = __float2half_rn(val);
    bits = *reinterpret_cast<const uint16_t*>(&h);
  }
  if (p.peer.num_peers == 0) {
    *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(p.out) +
                                 ((int64_t)row_q * p.o_st + (int64_t)head * p.o_sh + d) * 2) = bits;
    return;
  }
  const int64_t prow = p.peer.rows ? p.peer.rows[row_q] : row_q;
  const int64_t off = (prow * p.peer.stride_t + (int64_t)(p.peer.head_offset + head) * p.peer.stride_h + d) * 2;
  for (int q = 0; q < p.peer.num_peers; ++q)
    *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(p.peer.out[q]) + off) = bits;
}

// EXTRA: the optional fusions (cache write of the new token, rotary op on the query, cos/sin
// computed in the kernel) are compiled into a second instance of the kernel, so that the
// plain call keeps the register budget and instruction count its bandwidth depends on.
template <int D, int KV, bool BF16, bool MEPIC, int EXTRA>
__global__ void __launch_bounds__(DecCfg<D, KV>::kThreads, DecCfg<D, KV>::kMinBlocks) decode_split_kernel(DecParams p) {
  using Cfg = DecCfg<D, KV>;
  constexpr bool BF16MMA = (KV == 0) && BF16;  // fp8 caches go through f16
  constexpr int KSTEPS = D / 16;
  constexpr int W = Cfg::kWarps, S = Cfg::kStages;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  __shared__ __align__(8) uint64_t bar_full[W * S];
  __shared__ int2 ent[Cfg::kMaxChunkPages];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = lane >> 2, c = lane & 3;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int row_q = p.qsl[seq];
  if (p.qsl[seq + 1] - row_q != 1) return;
  const int seq_len = p.seq_lens[seq];
  const int npages = (seq_len + 15) >> 4;
  const int first_page = split * p.chunk_pages;
  if (first_page >= npages) return;
  // The plan (chunk size, split count) comes from the caller's max_seq_len.  A
  // sequence longer than that bound is still covered in full: the last split
  // walks on, chunk by chunk, to the sequence's real last page.
  const int end_page = (split == p.n_splits - 1) ? npages : min(npages, first_page + p.chunk_pages);
  const bool lazy = !MEPIC && p.is_lazy != nullptr && p.is_lazy[seq] != 0;
  const int64_t* prow = MEPIC ? nullptr : p.packed + (int64_t)seq * p.packed_stride;
  // fused rotary op: the token's position, fetched here so that only the table row's loads remain
  // when the query is prepared
  int64_t q_position = 0;
  if (EXTRA && p.q_pos != nullptr) q_position = p.q_pos[row_q];

  if (tid == 0) {
    for (int i = 0; i < W * S; ++i) mbar_init(&bar_full[i], 1);
    mbar_fence_init();
  }
  // ---- Q fragments (B operand: head = lane/4, four consecutive dims per k-step).  The plain
  // call fetches them first; with the fused rotary op they are prepared after the first copies
  // have been issued, so that the table row's latency runs under them (for the plain call that
  // order measured 0.5 % slower).
  uint32_t qfull[KSTEPS][2], qcur[KSTEPS][2];
  auto load_query = [&]() {
    const int h = r;
    const uint8_t* qrow = reinterpret_cast<const uint8_t*>(p.q) +
                          ((int64_t)row_q * p.q_st + (int64_t)(kvh * p.G + h) * p.q_sh) * 2;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint2 v = make_uint2(0, 0);
      if (h < p.G) v = *reinterpret_cast<const uint2*>(qrow + (ks * 16 + c * 4) * 2);
      qfull[ks][0] = v.x;
      qfull[ks][1] = v.y;
    }
    if (EXTRA && p.q_pos != nullptr) {
      // Fused rotary op: the query arrives without rotary embedding; rotate it forward at its
      // position (NeoX halves: dims d and d + D/2 sit in k-steps ks and ks + KSTEPS/2 of this
      // thread) and round to the query's dtype, as the stand-alone op leaves it.
      int64_t pos = q_position;
      if (p.cs != nullptr && pos >= p.cs_rows) pos = p.cs_rows - 1;
      const uint8_t* crow = reinterpret_cast<const uint8_t*>(p.cs) + pos * D * 2;
#pragma unroll
      for (int ks = 0; ks < KSTEPS / 2; ++ks) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float2 cc, ss;
          if (EXTRA != 2 || p.cs != nullptr) {
            cc = unpack_q<BF16>(*reinterpret_cast<const uint32_t*>(crow + (ks * 16 + c * 4 + 2 * j) * 2));
            ss = unpack_q<BF16>(*reinterpret_cast<const uint32_t*>(crow + D + (ks * 16 + c * 4 + 2 * j) * 2));
          } else {
            rope_cos_sin_pair<D>(p, (int)pos, ks * 16 + c * 4 + 2 * j, cc, ss);
          }
          const float2 q1 = unpack_q<BF16>(qfull[ks][j]), q2 = unpack_q<BF16>(qfull[ks + KSTEPS / 2][j]);
          qfull[ks][j] = pack_mma<BF16>(q1.x * cc.x - q2.x * ss.x, q1.y * cc.y - q2.y * ss.y);
          qfull[ks + KSTEPS / 2][j] = pack_mma<BF16>(q2.x * cc.x + q1.x * ss.x, q2.y * cc.y + q1.y * ss.y);
        }
      }
    }
    };
  auto set_rotation = [&](int eff) {
    if (eff <= 1) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const float2 a = unpack_q<BF16>(qfull[ks][0]), b = unpack_q<BF16>(qfull[ks][1]);
        qcur[ks][0] = pack_mma<BF16MMA>(a.x, a.y);
        qcur[ks][1] = pack_mma<BF16MMA>(b.x, b.y);
      }
      return;
    }
    int pos = eff - 1;
    if (EXTRA != 2 && pos >= p.cs_rows) pos = (int)p.cs_rows - 1;
    const uint8_t* crow = reinterpret_cast<const uint8_t*>(p.cs) + (int64_t)pos * D * 2;
#pragma unroll
    for (int ks = 0; ks < KSTEPS / 2; ++ks) {
      // dims d = 16ks + 4c + {0..3} pair with d + D/2, which sit in k-step ks + KSTEPS/2
      constexpr bool compute_cs = EXTRA == 2;
      uint32_t cw[2] = {0, 0}, sw[2] = {0, 0};
      if (!compute_cs) {
        const uint2 cv = __ldg(reinterpret_cast<const uint2*>(crow + (ks * 16 + c * 4) * 2));
        const uint2 sv = __ldg(reinterpret_cast<const uint2*>(crow + D + (ks * 16 + c * 4) * 2));
        cw[0] = cv.x; cw[1] = cv.y; sw[0] = sv.x; sw[1] = sv.y;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float2 q1 = unpack_q<BF16>(qfull[ks][j]), q2 = unpack_q<BF16>(qfull[ks + KSTEPS / 2][j]);
        float2 cc, ss;
        if (compute_cs) {
          // float32, not rounded to the table's dtype
          rope_cos_sin_pair<D>(p, eff - 1, ks * 16 + c * 4 + 2 * j, cc, ss);
        } else {
          cc = unpack_q<BF16>(cw[j]);
          ss = unpack_q<BF16>(sw[j]);
        }
        // inverse rotation; rounded to the query's storage type as the reference does
        float n1x = q1.x * cc.x + q2.x * ss.x, n1y = q1.y * cc.y + q2.y * ss.y;
        float n2x = q2.x * cc.x - q1.x * ss.x, n2y = q2.y * cc.y - q1.y * ss.y;
        if constexpr (BF16 && !BF16MMA) {
          n1x = __bfloat162float(__float2bfloat16_rn(n1x)); n1y = __bfloat162float(__float2bfloat16_rn(n1y));
          n2x = __bfloat162float(__float2bfloat16_rn(n2x)); n2y = __bfloat162float(__float2bfloat16_rn(n2y));
        }
        qcur[ks][j] = pack_mma<BF16MMA>(n1x, n1y);
        qcur[ks + KSTEPS / 2][j] = pack_mma<BF16MMA>(n2x, n2y);
      }
    }
  };
  int cur_eff = 1;
  if constexpr (EXTRA == 0) {
    load_query();
    set_rotation(1);
  }

  const float k_scale = (KV != 0 && p.k_scale) ? *p.k_scale : 1.f;
  const float v_scale = (KV != 0 && p.v_scale) ? *p.v_scale : 1.f;
  const float scale_log2 = p.sm_scale * k_scale * 1.4426950408889634f;

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[KSTEPS][4];
#pragma unroll
  for (int mt = 0; mt < KSTEPS; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
  const int tok_lo = sigma(r), tok_hi = tok_lo ^ 2;
  bool ok = true;
  int git = 0;  // tiles this warp has issued and consumed so far (ring stage and phase)
  constexpr int PPT = Cfg::kPPT;
  uint8_t* ring = smem + (size_t)warp * S * Cfg::kTileBytes;
  uint64_t* my_bar = bar_full + warp * S;

  if (EXTRA && p.slots != nullptr && first_page <= npages - 1 && npages - 1 < end_page) {
    // Fused cache write: the CTA whose run of pages holds the sequence's last page stores the new
    // token's K/V row (in cache format) into that page before any of its copies is issued, so
    // that this call attends to it like the calls to come.  Order: the stores, a device-wide
    // fence by the storing threads, the CTA barrier below, a proxy fence by the thread that
    // issues the bulk copies (which read global memory through the asynchronous proxy).
    const int64_t slot = p.slots[row_q];
    if (slot >= 0) {
      constexpr int X = 16 / Cfg::kElem;  // elements per 16-byte group
      const int64_t blk = slot >> 4;
      const int off_g = (int)(slot & 15);
      uint8_t* kp_g = const_cast<uint8_t*>(p.kc) + blk * p.kc_sb + (int64_t)kvh * p.kc_sh;
      uint8_t* vp_g = const_cast<uint8_t*>(p.vc) + blk * p.vc_sb + (int64_t)kvh * p.vc_sh;
      const uint16_t* krow = reinterpret_cast<const uint16_t*>(p.key) + (int64_t)row_q * p.k_st + (int64_t)kvh * p.k_sh;
      const uint16_t* vrow = reinterpret_cast<const uint16_t*>(p.value) + (int64_t)row_q * p.v_st + (int64_t)kvh * p.v_sh;
      const float ksc = (KV != 0 && p.k_scale) ? *p.k_scale : 1.f;
      const float vsc = (KV != 0 && p.v_scale) ? *p.v_scale : 1.f;
      for (int g = tid; g < D / X; g += Cfg::kThreads) {  // K page [D/X][16][X]
        uint8_t grp[16];
        to_cache_elems<KV, BF16>(krow + g * X, X, grp, ksc);
        *reinterpret_cast<uint4*>(kp_g + (g * 16 + off_g) * 16) = *reinterpret_cast<const uint4*>(grp);
      }
      for (int d = tid; d < D; d += Cfg::kThreads) {      // V page [D][16]
        uint8_t el[2];
        to_cache_elems<KV, BF16>(vrow + d, 1, el, vsc);
        for (int bb = 0; bb < Cfg::kElem; ++bb) vp_g[(d * 16 + off_g) * Cfg::kElem + bb] = el[bb];
      }
      __threadfence();
    }
  }
  for (int page0 = first_page; page0 < end_page && ok; page0 += p.chunk_pages) {
  const int n = min(p.chunk_pages, end_page - page0);
  // ---- page entries of this chunk: physical page, rotation in force, pad count.
  // All threads fetch the packed entries; warp 0 then resolves "offset 0 keeps the
  // rotation in force" with a scan, seeded by a backward search before the chunk.
  for (int i = tid; i < n; i += Cfg::kThreads) {
    if constexpr (MEPIC) {
      int blk = p.block_table[(int64_t)seq * p.table_stride + page0 + i];
      if (p.num_blocks > 0) blk = max(0, min(blk, (int)p.num_blocks - 1));
      const int pad = min(max(p.q_mask[(int64_t)seq * p.table_stride + page0 + i], 0), 16);
      ent[i] = make_int2(blk, (1 << 16) | pad);
      continue;
    }
    const int64_t pk = prow[page0 + i];
    int blk = (int)(pk >> 32);
    if (p.num_blocks > 0) blk = max(0, min(blk, (int)p.num_blocks - 1));
    const int rot = lazy ? (int)((pk >> 16) & 0xFFFF) : 1;
    const int pad = (lazy && !p.ignore_q_mask) ? min((int)(pk & 0xFFFF), 16) : 0;
    ent[i] = make_int2(blk, (int)(((uint32_t)rot << 16) | (uint32_t)pad));
  }
  __syncthreads();
  if (warp == 0 && lazy) {
    int carry = 1;
    if (page0 > 0) {
      for (int base = page0 - 32;; base -= 32) {
        const int idx = base + lane;
        int rot = 0;
        if (idx >= 0 && idx < page0) rot = (int)((prow[idx] >> 16) & 0xFFFF);
        const unsigned m = __ballot_sync(0xffffffffu, rot != 0);
        if (m) {
          carry = __shfl_sync(0xffffffffu, rot, 31 - __clz(m));
          break;
        }
        if (base <= 0) break;
      }
    }
    for (int g0 = 0; g0 < n; g0 += 32) {
      const int i = g0 + lane;
      int2 e = make_int2(0, 0);
      if (i < n) e = ent[i];
      int eff = (int)((uint32_t)e.y >> 16);  // the rotation field fills the top 16 bits: no sign extension
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, eff, o);
        if (lane >= o && eff == 0) eff = up;
      }
      if (eff == 0) eff = carry;
      carry = __shfl_sync(0xffffffffu, eff, 31);
      if (i < n) ent[i] = make_int2(e.x, (int)(((uint32_t)eff << 16) | ((uint32_t)e.y & 0xFFFFu)));
    }
  }

  // ---- this warp's tiles: tile tl covers chunk pages 2*tl, 2*tl+1; warp w takes tl = w, w+W, ...
  const int n_tiles = (n + PPT - 1) / PPT;
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + W - 1) / W : 0;
  auto issue = [&](int it) {  // lane 0 only
    const int tl = warp + it * W;
    const int st = (git + it) % S;
    uint8_t* dst = ring + st * Cfg::kTileBytes;
    const int pg = PPT * tl;
    const int np = min(PPT, n - pg);
    mbar_arrive_expect_tx(&my_bar[st], (uint32_t)(2 * np * Cfg::kPageBytes));
    for (int i = 0; i < np; ++i) {
      const int64_t blk = ent[pg + i].x;
      bulk_load(dst + i * Cfg::kPageBytes, p.kc + blk * p.kc_sb + (int64_t)kvh * p.kc_sh, Cfg::kPageBytes,
                &my_bar[st]);
      bulk_load(dst + (PPT + i) * Cfg::kPageBytes, p.vc + blk * p.vc_sb + (int64_t)kvh * p.vc_sh, Cfg::kPageBytes,
                &my_bar[st]);
    }
  };
  if (lane == 0) {
    if (EXTRA) asm volatile("fence.proxy.async;" ::: "memory");  // after the fused cache write above
    for (int it = 0; it < min(S, my_tiles); ++it) issue(it);
  }
  if (EXTRA != 0 && page0 == first_page) {
    load_query();
    set_rotation(1);
  }
  __syncthreads();  // the rotation scan of warp 0 is complete

  for (int it = 0; it < my_tiles; ++it) {
    const int tl = warp + it * W;
    const int st = (git + it) % S;
    const uint8_t* tile = ring + st * Cfg::kTileBytes;
    ok = mbar_wait(&my_bar[st], (uint32_t)((git + it) / S) & 1u, p.status, 501);
    ok = __all_sync(0xffffffffu, ok) != 0;
    if (!ok) break;
    const int pg = PPT * tl;
    const int np = min(PPT, n - pg);
    float s[PPT][4];
    bool vlo[PPT], vhi[PPT];
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      vlo[i] = vhi[i] = false;
      if (i < np) {
        const int2 e = ent[pg + i];
        const int eff = (int)((uint32_t)e.y >> 16), pad = e.y & 0xFFFF;
        if (eff != cur_eff) {
          set_rotation(eff);
          cur_eff = eff;
        }
        const uint8_t* kp = tile + i * Cfg::kPageBytes;
        if constexpr (MEPIC) {
          // per-token mode: every cached key is rotated forward at its slot position
          // before the dot product; dims d and d + D/2 sit in k-steps ks and ks + KSTEPS/2
          // of the same thread, so the rotation is thread-local.
          const int tb = (page0 + pg + i) * 16;
          int pos_lo = tb + tok_lo, pos_hi = tb + tok_hi;
          if (pos_lo >= p.cs_rows) pos_lo = (int)p.cs_rows - 1;
          if (pos_hi >= p.cs_rows) pos_hi = (int)p.cs_rows - 1;
          const uint8_t* c_lo = reinterpret_cast<const uint8_t*>(p.cs) + (int64_t)pos_lo * D * 2;
          const uint8_t* c_hi = reinterpret_cast<const uint8_t*>(p.cs) + (int64_t)pos_hi * D * 2;
#pragma unroll
          for (int ks = 0; ks < KSTEPS / 2; ++ks) {
            uint32_t k1[4], k2[4];  // order a0, a1, a2, a3: (lo tok, dims 0-1), (hi tok, 0-1), (lo, 2-3), (hi, 2-3)
            if constexpr (KV == 0) {
              const uint8_t* b1 = kp + (2 * ks + (c >> 1)) * 256 + (c & 1) * 8;
              const uint8_t* b2 = kp + (2 * (ks + KSTEPS / 2) + (c >> 1)) * 256 + (c & 1) * 8;
              const uint2 l1 = *reinterpret_cast<const uint2*>(b1 + tok_lo * 16);
              const uint2 h1 = *reinterpret_cast<const uint2*>(b1 + tok_hi * 16);
              const uint2 l2 = *reinterpret_cast<const uint2*>(b2 + tok_lo * 16);
              const uint2 h2 = *reinterpret_cast<const uint2*>(b2 + tok_hi * 16);
              k1[0] = l1.x; k1[2] = l1.y; k1[1] = h1.x; k1[3] = h1.y;
              k2[0] = l2.x; k2[2] = l2.y; k2[1] = h2.x; k2[3] = h2.y;
            } else {
              const uint8_t* b1 = kp + ks * 256 + c * 4;
              const uint8_t* b2 = kp + (ks + KSTEPS / 2) * 256 + c * 4;
              fp8x4_to_h2x2<KV>(*reinterpret_cast<const uint32_t*>(b1 + tok_lo * 16), k1[0], k1[2]);
              fp8x4_to_h2x2<KV>(*reinterpret_cast<const uint32_t*>(b1 + tok_hi * 16), k1[1], k1[3]);
              fp8x4_to_h2x2<KV>(*reinterpret_cast<const uint32_t*>(b2 + tok_lo * 16), k2[0], k2[2]);
              fp8x4_to_h2x2<KV>(*reinterpret_cast<const uint32_t*>(b2 + tok_hi * 16), k2[1], k2[3]);
            }
            const uint2 cl = __ldg(reinterpret_cast<const uint2*>(c_lo + (ks * 16 + c * 4) * 2));
            const uint2 sl = __ldg(reinterpret_cast<const uint2*>(c_lo + D + (ks * 16 + c * 4) * 2));
            const uint2 ch = __ldg(reinterpret_cast<const uint2*>(c_hi + (ks * 16 + c * 4) * 2));
            const uint2 sh = __ldg(reinterpret_cast<const uint2*>(c_hi + D + (ks * 16 + c * 4) * 2));
            const uint32_t cw[4] = {cl.x, ch.x, cl.y, ch.y}, sw[4] = {sl.x, sh.x, sl.y, sh.y};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint32_t cv = cw[e], sv = sw[e];
              if constexpr (BF16 && !BF16MMA) {  // bf16 table, keys and MMAs in f16 (fp8 cache)
                const float2 cc = unpack_q<true>(cv), ss = unpack_q<true>(sv);
                cv = pack_mma<false>(cc.x, cc.y);
                sv = pack_mma<false>(ss.x, ss.y);
              }
              rotate_pair<BF16MMA>(k1[e], k2[e], cv, sv);
            }
            mma16816<BF16MMA>(s[i], k1[0], k1[1], k1[2], k1[3], qcur[ks][0], qcur[ks][1]);
            mma16816<BF16MMA>(s[i], k2[0], k2[1], k2[2], k2[3], qcur[ks + KSTEPS / 2][0], qcur[ks + KSTEPS / 2][1]);
          }
        } else
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          uint32_t a0, a1, a2, a3;
          if constexpr (KV == 0) {
            const uint8_t* base = kp + (2 * ks + (c >> 1)) * 256 + (c & 1) * 8;
            const uint2 lo = *reinterpret_cast<const uint2*>(base + tok_lo * 16);
            const uint2 hi = *reinterpret_cast<const uint2*>(base + tok_hi * 16);
            a0 = lo.x; a2 = lo.y; a1 = hi.x; a3 = hi.y;
          } else {
            const uint8_t* base = kp + ks * 256 + c * 4;
            const uint32_t lo = *reinterpret_cast<const uint32_t*>(base + tok_lo * 16);
            const uint32_t hi = *reinterpret_cast<const uint32_t*>(base + tok_hi * 16);
            fp8x4_to_h2x2<KV>(lo, a0, a2);
            fp8x4_to_h2x2<KV>(hi, a1, a3);
          }
          mma16816<BF16MMA>(s[i], a0, a1, a2, a3, qcur[ks][0], qcur[ks][1]);
        }
        const int tbase = (page0 + pg + i) * 16;
        vlo[i] = (tbase + tok_lo < seq_len) && (tok_lo < 16 - pad);
        vhi[i] = (tbase + tok_hi < seq_len) && (tok_hi < 16 - pad);
      }
    }
    // ---- online softmax over the tile's 32 tokens (log2 domain), two heads per thread
    float mx[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float v = -INFINITY;
#pragma unroll
      for (int i = 0; i < PPT; ++i) {
        s[i][hh] = vlo[i] ? s[i][hh] * scale_log2 : -INFINITY;
        s[i][2 + hh] = vhi[i] ? s[i][2 + hh] * scale_log2 : -INFINITY;
        v = fmaxf(v, fmaxf(s[i][hh], s[i][2 + hh]));
      }
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
      v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
      mx[hh] = v;
    }
    float alpha[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const float m_new = fmaxf(m_run[hh], mx[hh]);
      const float m_eff = m_new == -INFINITY ? 0.f : m_new;
      alpha[hh] = ex2(m_run[hh] - m_eff);  // m_run == -inf gives 0
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < PPT; ++i) {
        s[i][hh] = ex2(s[i][hh] - m_eff);
        s[i][2 + hh] = ex2(s[i][2 + hh] - m_eff);
        sum += s[i][hh] + s[i][2 + hh];
      }
      l_run[hh] = l_run[hh] * alpha[hh] + sum;
      m_run[hh] = m_new;
    }
#pragma unroll
    for (int mt = 0; mt < KSTEPS; ++mt) {
      o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1]; o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
    }
    // ---- O^T += V^T * P^T, one page at a time
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      if (i < np) {
        const uint32_t lo_pack = pack_mma<BF16MMA>(s[i][0], s[i][1]);
        const uint32_t hi_pack = pack_mma<BF16MMA>(s[i][2], s[i][3]);
        const int src_a = (2 * c) * 4 + (r >> 1), src_b = (2 * c + 1) * 4 + (r >> 1);
        const uint32_t x0 = __shfl_sync(0xffffffffu, lo_pack, src_a), x1 = __shfl_sync(0xffffffffu, lo_pack, src_b);
        const uint32_t y0 = __shfl_sync(0xffffffffu, hi_pack, src_a), y1 = __shfl_sync(0xffffffffu, hi_pack, src_b);
        const uint32_t sel = (r & 1) ? 0x7632u : 0x5410u;
        const uint32_t px = __byte_perm(x0, x1, sel), py = __byte_perm(y0, y1, sel);
        const uint32_t b0 = c < 2 ? px : py, b1 = c < 2 ? py : px;
        const uint8_t* vp = tile + (PPT + i) * Cfg::kPageBytes;
#pragma unroll
        for (int mt = 0; mt < KSTEPS; ++mt) {
          uint32_t a0, a1, a2, a3;
          if constexpr (KV == 0) {
            const uint8_t* base = vp + (mt * 16 + r) * 32 + c * 8;
            const uint2 lo = *reinterpret_cast<const uint2*>(base);
            const uint2 hi = *reinterpret_cast<const uint2*>(base + 8 * 32);
            a0 = lo.x; a2 = lo.y; a1 = hi.x; a3 = hi.y;
          } else {
            const uint8_t* base = vp + (mt * 16 + r) * 16 + c * 4;
            const uint32_t lo = *reinterpret_cast<const uint32_t*>(base);
            const uint32_t hi = *reinterpret_cast<const uint32_t*>(base + 8 * 16);
            fp8x4_to_h2x2<KV>(lo, a0, a2);
            fp8x4_to_h2x2<KV>(hi, a1, a3);
          }
          mma16816<BF16MMA>(o[mt], a0, a1, a2, a3, b0, b1);
        }
      }
    }
    // ---- refill this stage
    __syncwarp();
    if (lane == 0 && it + S < my_tiles) {
      fence_proxy_async_smem();  // order the generic-proxy reads above before the async refill
      issue(it + S);
    }
  }
  git += my_tiles;
  // every warp is done with this chunk's entries; a warp whose wait expired stops the whole CTA
  ok = __syncthreads_and(ok) != 0;
  }  // chunks of this split

  // ---- merge the warps of the CTA, then write the result or the split's partial
  __syncthreads();  // every warp has consumed all it issued: the ring can be reused
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
  }
  float* mrg = reinterpret_cast<float*>(smem) + (size_t)warp * 8 * (D + 2);
#pragma unroll
  for (int mt = 0; mt < KSTEPS; ++mt) {
    mrg[(2 * c) * (D + 2) + mt * 16 + r] = o[mt][0];
    mrg[(2 * c + 1) * (D + 2) + mt * 16 + r] = o[mt][1];
    mrg[(2 * c) * (D + 2) + mt * 16 + r + 8] = o[mt][2];
    mrg[(2 * c + 1) * (D + 2) + mt * 16 + r + 8] = o[mt][3];
  }
  if (r == 0) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      mrg[(2 * c + hh) * (D + 2) + D] = ok ? m_run[hh] : -INFINITY;
      mrg[(2 * c + hh) * (D + 2) + D + 1] = ok ? l_run[hh] : 0.f;
    }
  }
  __syncthreads();
  const float* all = reinterpret_cast<const float*>(smem);
  for (int idx = tid; idx < p.G * D; idx += Cfg::kThreads) {
    const int h = idx / D, d = idx - h * D;
    float m_star = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; ++w) m_star = fmaxf(m_star, all[(w * 8 + h) * (D + 2) + D]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float mw = all[(w * 8 + h) * (D + 2) + D];
      if (mw == -INFINITY) continue;
      const float wgt = ex2(mw - m_star);
      acc += wgt * all[(w * 8 + h) * (D + 2) + d];
      l += wgt * all[(w * 8 + h) * (D + 2) + D + 1];
    }
    const int head = kvh * p.G + h;
    if (p.n_splits == 1) {
      const float val = l > 0.f ? acc / l * v_scale : 0.f;
      store_result<BF16>(p, row_q, head, d, val);
    } else {
      const int64_t slot = ((int64_t)seq * p.Hq + head) * p.n_splits + split;
      p.part_o[slot * D + d] = acc;
      if (d == 0) {
        p.part_ml[slot * 2] = m_star;
        p.part_ml[slot * 2 + 1] = l;
      }
    }
  }
}

template <int D, bool BF16>
__global__ void decode_merge_kernel(DecParams p, float v_scale_on) {
  const int head = blockIdx.x, seq = blockIdx.y;
  const int row_q = p.qsl[seq];
  if (p.qsl[seq + 1] - row_q != 1) return;
  const int npages = (p.seq_lens[seq] + 15) >> 4;
  const int used = min(p.n_splits, (npages + p.chunk_pages - 1) / p.chunk_pages);
  const int d = threadIdx.x;
  const int64_t slot0 = ((int64_t)seq * p.Hq + head) * p.n_splits;
  float m_star = -INFINITY;
  for (int s = 0; s < used; ++s) m_star = fmaxf(m_star, p.part_ml[(slot0 + s) * 2]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < used; ++s) {
    const float m = p.part_ml[(slot0 + s) * 2];
    if (m == -INFINITY) continue;
    const float w = exp2f(m - m_star);
    acc += w * p.part_o[(slot0 + s) * D + d];
    l += w * p.part_ml[(slot0 + s) * 2 + 1];
  }
  const float v_scale = (v_scale_on != 0.f && p.v_scale) ? *p.v_scale : 1.f;
  const float val = l > 0.f ? acc / l * v_scale : 0.f;
  store_result<BF16>(p, row_q, head, d, val);
}

struct DecPlan {
  int chunk_pages, n_splits;
};

DecPlan make_dec_plan(const LaDecodeArgs& a, int quantum) {  // quantum: pages of one tile per warp
  const int64_t max_pages = a.max_seq_len > 0 ? ((int64_t)a.max_seq_len + 15) / 16 : 1;
  const int64_t items = (int64_t)a.num_seqs * a.num_kv_heads;
  const int64_t target = 148 * 8;
  int64_t chunk = (max_pages * items + target - 1) / target;
  chunk = ((chunk + quantum - 1) / quantum) * quantum;
  if (chunk < 2 * quantum) chunk = 2 * quantum;
  // Runs longer than ~224 pages gain nothing (the per-CTA prologue is amortised long before)
  // and cost balance at the end of the launch: on the 256-sequence fp8 workload a cap of 192..256
  // pages ties with 512 on the whole batch and is 3-6 % faster on a half or a quarter of it.
  if (chunk > 224) chunk = 224;
  if (const char* e = getenv("LAZY_ATTN_B200_DECODE_CHUNK")) {  // experiments only
    const int v = atoi(e);
    if (v >= quantum && v <= 512) chunk = (v / quantum) * quantum;
  }
  DecPlan pl;
  pl.chunk_pages = (int)chunk;
  pl.n_splits = (int)((max_pages + chunk - 1) / chunk);
  if (pl.n_splits < 1) pl.n_splits = 1;
  return pl;
}

// pages that the warps of a CTA consume per round: DecCfg::kWarps * DecCfg::kPPT
int quantum_for(const LaDecodeArgs& a) {
  const int page_bytes = a.head_dim * 16 * (a.kv_dtype == a.q_dtype ? 2 : 1);
  return 4 * (page_bytes > 2048 ? 1 : (page_bytes > 1024 ? 2 : 4));
}

template <int D, int KV, bool BF16, bool MEPIC, int EXTRA>
int launch_dec_m(const LaDecodeArgs& a, DecParams& p, cudaStream_t stream) {
  using Cfg = DecCfg<D, KV>;
  auto kern = decode_split_kernel<D, KV, BF16, MEPIC, EXTRA>;
  // the attribute is per device: remember on which devices this kernel has been prepared
  static std::atomic<uint64_t> prepared{0};
  int dev = 0;
  LA_CHECK_CUDA(cudaGetDevice(&dev));
  if (((prepared.load(std::memory_order_acquire) >> (dev & 63)) & 1ull) == 0) {
    LA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    prepared.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  dim3 grid(p.n_splits, a.num_kv_heads, a.num_seqs);
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  if (p.n_splits > 1) {
    dim3 mgrid(a.num_q_heads, a.num_seqs);
    decode_merge_kernel<D, BF16><<<mgrid, D, 0, stream>>>(p, KV != 0 ? 1.f : 0.f);
    count_launch();
    LA_CHECK_CUDA(cudaGetLastError());
  }
  return LA_OK;
}

template <int D, int KV, bool BF16>
int launch_dec(const LaDecodeArgs& a, DecParams& p, cudaStream_t stream) {
  // 0: the plain call; 1: with the fused cache write and / or the rotary op on the query (table
  // rows); 2: cos/sin evaluated in the kernel as well (per-page rotation mode only)
  const bool extra = a.slot_mapping != nullptr || a.q_positions != nullptr;
  if (a.rot_mode == LA_ROT_MEPIC)
    return extra ? launch_dec_m<D, KV, BF16, true, 1>(a, p, stream) : launch_dec_m<D, KV, BF16, true, 0>(a, p, stream);
  if (a.compute_cos_sin != 0) return launch_dec_m<D, KV, BF16, false, 2>(a, p, stream);
  return extra ? launch_dec_m<D, KV, BF16, false, 1>(a, p, stream) : launch_dec_m<D, KV, BF16, false, 0>(a, p, stream);
}

}  // namespace

bool fast_decode_supported(const LaDecodeArgs& a, const char** why) {
  const int G = a.num_kv_heads > 0 ? a.num_q_heads / a.num_kv_heads : 0;
  if (a.rot_mode == LA_ROT_MEPIC && (a.cos_sin_cache == nullptr || a.cos_sin_dtype != a.q_dtype)) { *why = "cos/sin table dtype must equal the query dtype"; return false; }
  if (a.q_dtype != LA_DTYPE_BF16 && a.q_dtype != LA_DTYPE_F16) { *why = "query must be bf16 or fp16"; return false; }
  if (a.kv_dtype != a.q_dtype && a.kv_dtype != LA_DTYPE_FP8_E4M3 && a.kv_dtype != LA_DTYPE_FP8_E5M2) { *why = "cache dtype"; return false; }
  if (a.head_dim != 64 && a.head_dim != 128) { *why = "head_dim must be 64 or 128"; return false; }
  if (a.block_size != 16) { *why = "block_size must be 16"; return false; }
  if (G < 1 || G > 8) { *why = "at most 8 query heads per KV head"; return false; }
  if (a.alibi_slopes != nullptr) { *why = "alibi"; return false; }
  if (a.sliding_window > 0) { *why = "sliding window"; return false; }
  if (a.is_lazy != nullptr && a.cos_sin_cache != nullptr && a.cos_sin_dtype != a.q_dtype) { *why = "cos/sin table dtype must equal the query dtype"; return false; }
  if (a.compute_cos_sin && a.rot_mode != LA_ROT_LAZY) { *why = "in-kernel cos/sin is for the per-page rotation mode"; return false; }
  if (a.compute_cos_sin && (a.rope_base <= 1.f || (a.rope_type == 1 && (a.rope_high_freq_factor == a.rope_low_freq_factor || a.rope_scaling_factor <= 0.f)))) { *why = "bad RoPE parameters"; return false; }
  if (a.q_positions != nullptr && a.cos_sin_cache == nullptr && !a.compute_cos_sin) { *why = "the fused rotary op needs the cos/sin table or the RoPE parameters"; return false; }
  if (a.q_positions != nullptr && a.cos_sin_cache != nullptr && a.cos_sin_dtype != a.q_dtype) { *why = "cos/sin table dtype must equal the query dtype"; return false; }
  if (a.q_stride_t % 4 || a.q_stride_h % 4) { *why = "query strides must be multiples of 4 elements"; return false; }
  const int e = a.kv_dtype == a.q_dtype ? 2 : 1;
  if ((a.kc_stride_block * e) % 16 || (a.kc_stride_head * e) % 16 || (a.vc_stride_block * e) % 16 || (a.vc_stride_head * e) % 16) { *why = "cache strides must be multiples of 16 bytes"; return false; }
  if ((reinterpret_cast<uintptr_t>(a.k_cache) | reinterpret_cast<uintptr_t>(a.v_cache)) & 15) { *why = "cache pointers must be 16-byte aligned"; return false; }
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.cos_sin_cache)) & 7) { *why = "query / table pointers must be 8-byte aligned"; return false; }
  if (a.peer.num_peers < 0 || a.peer.num_peers > LA_MAX_PEERS) { *why = "peer count out of range"; return false; }
  for (int q = 0; q < a.peer.num_peers; ++q)
    if (a.peer.out[q] == nullptr) { *why = "null peer output pointer"; return false; }
  return true;
}

size_t fast_decode_workspace_bytes(const LaDecodeArgs& a) {
  const DecPlan pl = make_dec_plan(a, quantum_for(a));
  if (pl.n_splits <= 1) return 0;
  return (size_t)a.num_seqs * a.num_q_heads * pl.n_splits * (a.head_dim + 2) * sizeof(float) + 256;
}

int launch_fast_decode(const LaDecodeArgs& a, cudaStream_t stream) {
  const DecPlan pl = make_dec_plan(a, quantum_for(a));
  LA_REQUIRE(a.num_seqs <= 65535 && a.num_kv_heads <= 65535, LA_ERR_UNSUPPORTED,
             "la_decode_fwd: %d sequences or %d KV heads exceed the launch grid (at most 65535 each)", a.num_seqs,
             a.num_kv_heads);
  const int e = a.kv_dtype == a.q_dtype ? 2 : 1;
  DecParams p{};
  p.q = a.q; p.out = a.out;
  p.q_st = a.q_stride_t; p.q_sh = a.q_stride_h; p.o_st = a.o_stride_t; p.o_sh = a.o_stride_h;
  p.kc = reinterpret_cast<const uint8_t*>(a.k_cache);
  p.vc = reinterpret_cast<const uint8_t*>(a.v_cache);
  p.kc_sb = a.kc_stride_block * e; p.kc_sh = a.kc_stride_head * e;
  p.vc_sb = a.vc_stride_block * e; p.vc_sh = a.vc_stride_head * e;
  p.num_blocks = a.num_blocks;
  p.packed = a.packed_block_table; p.packed_stride = a.packed_stride;
  p.block_table = a.block_table; p.q_mask = a.q_mask; p.table_stride = a.table_stride;
  p.qsl = a.query_start_loc; p.seq_lens = a.seq_lens; p.is_lazy = a.is_lazy;
  p.k_scale = a.k_scale; p.v_scale = a.v_scale;
  p.peer = a.peer;
  p.key = a.key; p.value = a.value; p.slots = a.slot_mapping;
  p.q_pos = a.q_positions;
  p.compute_cs = a.compute_cos_sin; p.rope_type = a.rope_type; p.rope_orig = a.rope_orig_max_position;
  p.rope_base = a.rope_base; p.rope_factor = a.rope_scaling_factor;
  p.rope_low = a.rope_low_freq_factor; p.rope_high = a.rope_high_freq_factor;
  p.k_st = a.k_stride_t; p.k_sh = a.k_stride_h; p.v_st = a.v_stride_t; p.v_sh = a.v_stride_h;
  p.cs = a.cos_sin_cache; p.cs_rows = a.cos_sin_rows;
  p.Hq = a.num_q_heads; p.Hkv = a.num_kv_heads; p.G = a.num_q_heads / a.num_kv_heads;
  p.chunk_pages = pl.chunk_pages; p.n_splits = pl.n_splits; p.ignore_q_mask = a.ignore_q_mask;
  p.sm_scale = a.sm_scale;
  if (pl.n_splits > 1) {
    LA_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= fast_decode_workspace_bytes(a), LA_ERR_WORKSPACE,
               "la_decode_fwd: split-KV needs %zu bytes of workspace", fast_decode_workspace_bytes(a));
    const size_t slots = (size_t)a.num_seqs * a.num_q_heads * pl.n_splits;
    uintptr_t base = (reinterpret_cast<uintptr_t>(a.workspace) + 255) & ~uintptr_t(255);
    p.part_o = reinterpret_cast<float*>(base);
    p.part_ml = p.part_o + slots * a.head_dim;
  }
  p.status = device_status_ptr();
  LA_REQUIRE(p.status != nullptr, LA_ERR_CUDA, "la_decode_fwd: device status word unavailable");
  const bool bf16 = a.q_dtype == LA_DTYPE_BF16;
  const int kv = a.kv_dtype == a.q_dtype ? 0 : (a.kv_dtype == LA_DTYPE_FP8_E4M3 ? 1 : 2);
#define LA_DEC_CASE(DD, KK)                                                                   \
  if (a.head_dim == DD && kv == KK)                                                           \
    return bf16 ? launch_dec<DD, KK, true>(a, p, stream) : launch_dec<DD, KK, false>(a, p, stream);
  LA_DEC_CASE(128, 0)
  LA_DEC_CASE(128, 1)
  LA_DEC_CASE(128, 2)
  LA_DEC_CASE(64, 0)
  LA_DEC_CASE(64, 1)
  LA_DEC_CASE(64, 2)
#undef LA_DEC_CASE
  set_error("la_decode_fwd: no split-KV kernel for head_dim %d", a.head_dim);
  return LA_ERR_UNSUPPORTED;
}

}  // namespace la
