// Tensor-core prefix-prefill kernel for sm_100a: TMA page loads, rotate-on-load,
// tcgen05 MMAs with accumulators in tensor memory, online softmax, split-KV.
//
// One CTA owns 256 "rows" of one (request, KV head): row R = token * G + head
// within the KV group, split into two 128-row tiles.  It walks 128-key tiles:
// first the cached pages (8 pages of 16 tokens per tile, gathered through the
// block table by one TMA copy per page), then the new tokens (causal).
//
// Warp roles (14 warps):
//   0-3   softmax of row tile 0: one thread per row, the row's 128 scores taken
//         from tensor memory in four 32-column chunks (the next chunk is in
//         flight while the current one is exponentiated); S/P/O live in tensor
//         memory; these warps also stage the Q tiles at CTA start
//   4-7   softmax of row tile 1
//   8-11  operand staging: rotation of each landed K tile in shared memory by
//         the page's (or token's) position; new-token K/V tiles; with an fp8
//         cache also the copy and conversion of the raw pages
//   12    MMA issue (one thread): S = Q K^T (operands in shared memory),
//         O += P V (P read from tensor memory, V from shared memory)
//   13    TMA issue: K and V pages into their stage rings
//
// Shared-memory operand layout (no swizzle, K-major "core matrices" of
// 8 rows x 16 bytes): the page layouts of the cache map onto it directly:
//   K page [D/8][16 tok][8]  -> TMA box {8, 8 tok, D/8, 2} -> [tok/8][D/8][8 tok][16 B]
//   V page [D][16 tok]       -> TMA box {8 tok, 8, 2, D/8} -> [D/8][tok/8][8 d][16 B]
// so QK^T sees 128 keys x D (row-group stride D*16 B, K-chunk stride 128 B) and
// P.V consumes one page per K=16 step (N-group stride 256 B, K-chunk stride 128 B).
//
// Every wait is bounded (la_sm100.cuh); on expiry the CTA records a code in the
// status word, drains and frees its tensor memory.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include <atomic>
#include <type_traits>

#include "la_common.cuh"
#include "la_sm100.cuh"

namespace la {
namespace {

using namespace sm100;

constexpr int kSoftmaxThreads = 8 * 32;
constexpr int kWarpStage = 8, kWarpMma = 12;  // first staging warp, MMA-issue warp (the TMA warp follows)
// Per-role register budgets (setmaxnreg works on whole warpgroups, so the CTA is padded to 16
// warps; warps 14 and 15 only take part in the budget change and the final barriers).  A raise
// can only take registers the CTA's other warpgroups have released: the budgets must add up to
// at most threads x launch registers, else the raise waits forever.
constexpr int kThreadsTc = 16 * 32;
constexpr int kLaunchRegs = 128;                       // what ptxas reports for 512 threads, one CTA per SM
// Measured on the 65536-token prefill workload (same box, ms per call): no budgets (14 warps x 128) 4.19-4.25,
// 168/112/64 4.19, 176/104/56 4.07-4.10, 184/96/48 4.09-4.12.
constexpr int kRegsSoftmax = 176, kRegsStage = 104, kRegsIssue = 56;
static_assert(kSoftmaxThreads * kRegsSoftmax + 128 * kRegsStage + 128 * kRegsIssue <= kThreadsTc * kLaunchRegs,
              "register budgets exceed what the CTA is launched with");
static_assert(kRegsSoftmax % 8 == 0 && kRegsStage % 8 == 0 && kRegsIssue % 8 == 0, "budgets are multiples of 8");
template <int N> __device__ __forceinline__ void regs_raise() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void regs_lower() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
constexpr int kRowsPerCta = 256;
constexpr int kTileN = 128;
constexpr int kPagesPerTile = 8;
constexpr float kRescaleThreshold = 8.f;  // log2 units

// Optional timeline of CTA (0,0,0) for kernel tuning: compiled in only with -DLA_TRACE
// (clock stamps per tile into a device array read back by la_trace_read).
#ifdef LA_TRACE
constexpr int kTraceRows = 32, kTraceCols = 256;
__device__ long long g_trace[kTraceRows][kTraceCols];
#define LA_STAMP(row, col)                                                                      \
  do {                                                                                          \
    if (trace_on && (col) >= 0 && (col) < kTraceCols) g_trace[(row)][(col)] = clock64();         \
  } while (0)
#else
#define LA_STAMP(row, col) do { } while (0)
#endif

struct TcParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_st, q_sh, k_st, k_sh, v_st, v_sh, o_st, o_sh;
  const int32_t* block_table;
  const int32_t* q_offset;
  const int32_t* q_mask;
  int64_t table_stride;
  const int64_t* packed;  // optional: block << 32 | q_offset << 16 | q_mask per page
  int64_t packed_stride;
  const int32_t* qsl;
  const int32_t* seq_lens;
  const uint8_t* is_lazy;
  const void* cs;
  int64_t cs_rows;
  // fp8 caches are read with plain loads by the staging warps (byte strides)
  const uint8_t* kc;
  const uint8_t* vc;
  int64_t kc_sb, kc_sh, vc_sb, vc_sh, num_blocks;
  const float* k_scale;
  const float* v_scale;
  // fused cache write: slots of the new tokens (nullptr = off), the caches as writable bytes
  const int64_t* slots;
  const int64_t* q_pos;  // fused rotary op on the query (nullptr: the query arrives rotated)
  uint8_t* kcw;
  uint8_t* vcw;
  int64_t kcw_sb, kcw_sh, vcw_sb, vcw_sh;  // bytes
  LaPeerOut peer;  // fused output gather: result rows go to every rank's buffer instead of `out`
  int Hq, Hkv, G, g_shift;
  int rot_mode, is_mepic, skip_decode, n_splits, page_ratio;
  float scale_log2;
  float* part_o;   // [batch][Hkv][rows_cap][n_splits][D]
  float* part_ml;  // [batch][Hkv][rows_cap][n_splits][2]
  int64_t rows_cap;
  int* status;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Same instruction without `volatile`: a pure function the compiler may schedule freely
// (the branch-free exponential pass interleaves it with the packing of earlier values).
__device__ __forceinline__ float ex2_pure(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Tensor-memory column (relative to the row tile's S columns) of the P chunk for keys
// [32c, 32c+32): keys 0..63 over S columns 0..31, keys 64..127 over S columns 96..127.
__device__ __forceinline__ constexpr int p_col(int c) { return c < 2 ? c * 16 : 96 + (c - 2) * 16; }

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Waits for this thread's tensor-memory loads.  The loaded registers are passed through
// the statement so that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
// Orders uses of `r` after the preceding wait (no instruction is emitted).
__device__ __forceinline__ void tie_after_wait(uint32_t (&r)[32]) {
  asm volatile(""
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

__device__ __forceinline__ float row_max32(const uint32_t (&sc)[32]) {
  float mx0 = fmax3(__uint_as_float(sc[0]), __uint_as_float(sc[1]), __uint_as_float(sc[2]));
  float mx1 = fmax3(__uint_as_float(sc[3]), __uint_as_float(sc[4]), __uint_as_float(sc[5]));
#pragma unroll
  for (int i = 6; i + 3 < 32; i += 4) {
    mx0 = fmax3(mx0, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
    mx1 = fmax3(mx1, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
  }
  mx0 = fmax3(mx0, __uint_as_float(sc[30]), __uint_as_float(sc[31]));
  return fmaxf(mx0, mx1);
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// Rotate 8 (k1, k2) pairs held as two 16-byte chunks by the table row chunks, in
// packed 16-bit arithmetic (two roundings per result, as the reference's own
// 16-bit evaluation has):  r1 = k1*c - k2*s,  r2 = k1*s + k2*c.
template <bool BF16>
__device__ __forceinline__ void rotate_chunk(uint4& a, uint4& b, const uint4& cv, const uint4& sv) {
  uint32_t* pa = reinterpret_cast<uint32_t*>(&a);
  uint32_t* pb = reinterpret_cast<uint32_t*>(&b);
  const uint32_t* pc = reinterpret_cast<const uint32_t*>(&cv);
  const uint32_t* ps = reinterpret_cast<const uint32_t*>(&sv);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      const __nv_bfloat162 k1 = *reinterpret_cast<const __nv_bfloat162*>(&pa[i]);
      const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(&pb[i]);
      const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&pc[i]);
      const __nv_bfloat162 sn = *reinterpret_cast<const __nv_bfloat162*>(&ps[i]);
      const uint32_t nk2_bits = pb[i] ^ 0x80008000u;
      const __nv_bfloat162 nk2 = *reinterpret_cast<const __nv_bfloat162*>(&nk2_bits);
      const __nv_bfloat162 r1 = __hfma2(nk2, sn, __hmul2(k1, c));
      const __nv_bfloat162 r2 = __hfma2(k1, sn, __hmul2(k2, c));
      pa[i] = *reinterpret_cast<const uint32_t*>(&r1);
      pb[i] = *reinterpret_cast<const uint32_t*>(&r2);
    } else {
      const __half2 k1 = *reinterpret_cast<const __half2*>(&pa[i]);
      const __half2 k2 = *reinterpret_cast<const __half2*>(&pb[i]);
      const __half2 c = *reinterpret_cast<const __half2*>(&pc[i]);
      const __half2 sn = *reinterpret_cast<const __half2*>(&ps[i]);
      const uint32_t nk2_bits = pb[i] ^ 0x80008000u;
      const __half2 nk2 = *reinterpret_cast<const __half2*>(&nk2_bits);
      const __half2 r1 = __hfma2(nk2, sn, __hmul2(k1, c));
      const __half2 r2 = __hfma2(k1, sn, __hmul2(k2, c));
      pa[i] = *reinterpret_cast<const uint32_t*>(&r1);
      pb[i] = *reinterpret_cast<const uint32_t*>(&r2);
    }
  }
}

// 8 bf16 -> 8 f16 (the fp8-cache path runs its MMAs in f16)
__device__ __forceinline__ uint4 bf16x8_to_f16x8(uint4 v) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2<true>(w[i]);
    w[i] = pack2<false>(f.x, f.y);
  }
  return v;
}
// 8 values of the activation dtype -> 8 f16 of value * s, clamped to the f16 range
template <bool BF16>
__device__ __forceinline__ uint4 to_f16x8_scaled(uint4 v, float s) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2<BF16>(w[i]);
    w[i] = pack2<false>(fminf(fmaxf(f.x * s, -65504.f), 65504.f), fminf(fmaxf(f.y * s, -65504.f), 65504.f));
  }
  return v;
}
// 16 fp8 -> 16 f16 as two 16-byte chunks (values 0-7, 8-15); exact
template <int KVF8>
__device__ __forceinline__ void fp8x16_to_f16(const uint4& raw, uint4& lo, uint4& hi) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(&raw);
  uint32_t* o0 = reinterpret_cast<uint32_t*>(&lo);
  uint32_t* o1 = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t a, b;
    if constexpr (KVF8 == 2) {
      asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e5m2x2 %0, l;\n\tcvt.rn.f16x2.e5m2x2 %1, h;\n\t}"
          : "=r"(a), "=r"(b) : "r"(r[i]));
    } else {
      asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
          : "=r"(a), "=r"(b) : "r"(r[i]));
    }
    uint32_t* dst = i < 2 ? o0 : o1;
    dst[(i & 1) * 2] = a;
    dst[(i & 1) * 2 + 1] = b;
  }
}
// Rotation of 8 (k1, k2) pairs held as f16, in packed f16 arithmetic (one fused
// rounding more than float32 math; the operands come from fp8 values and the
// result is rounded to f16 for the MMA anyway).  Table chunks in the query dtype.
template <bool BF16>
__device__ __forceinline__ void rotate_chunk_f16(uint4& a, uint4& b, const uint4& cv, const uint4& sv) {
  uint32_t* pa = reinterpret_cast<uint32_t*>(&a);
  uint32_t* pb = reinterpret_cast<uint32_t*>(&b);
  const uint32_t* pc = reinterpret_cast<const uint32_t*>(&cv);
  const uint32_t* ps = reinterpret_cast<const uint32_t*>(&sv);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t cw = pc[i], sw = ps[i];
    if constexpr (BF16) {
      const float2 c = unpack2<true>(cw), sn = unpack2<true>(sw);
      cw = pack2<false>(c.x, c.y);
      sw = pack2<false>(sn.x, sn.y);
    }
    const __half2 k1 = *reinterpret_cast<const __half2*>(&pa[i]), k2 = *reinterpret_cast<const __half2*>(&pb[i]);
    const __half2 c = *reinterpret_cast<const __half2*>(&cw), sn = *reinterpret_cast<const __half2*>(&sw);
    const __half2 ra = __hfma2(k1, c, __hneg2(__hmul2(k2, sn)));
    const __half2 rb = __hfma2(k1, sn, __hmul2(k2, c));
    pa[i] = *reinterpret_cast<const uint32_t*>(&ra);
    pb[i] = *reinterpret_cast<const uint32_t*>(&rb);
  }
}

// Fused cache write: 8 consecutive dims [d0, d0+8) of a new token's K (V) row, given in the
// activation dtype, into slot `off` of page `blk` -- the element placement and the fp8
// conversion (saturating, of value / scale) of la_write_paged_cache.
template <bool BF16, int KVF8>
__device__ __forceinline__ void cache_put_k(const TcParams& p, int64_t blk, int off, int kvh, int d0, uint4 v,
                                            float scale) {
  uint8_t* page = p.kcw + blk * p.kcw_sb + (int64_t)kvh * p.kcw_sh;
  if constexpr (KVF8 == 0) {
    *reinterpret_cast<uint4*>(page + ((d0 >> 3) * 16 + off) * 16) = v;  // [D/8][16][8] x 2 bytes
  } else {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
    uint8_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack2<BF16>(w[i]);
      if constexpr (KVF8 == 1) {
        const __nv_fp8_e4m3 a(f.x / scale), b(f.y / scale);
        o[2 * i] = *reinterpret_cast<const uint8_t*>(&a);
        o[2 * i + 1] = *reinterpret_cast<const uint8_t*>(&b);
      } else {
        const __nv_fp8_e5m2 a(f.x / scale), b(f.y / scale);
        o[2 * i] = *reinterpret_cast<const uint8_t*>(&a);
        o[2 * i + 1] = *reinterpret_cast<const uint8_t*>(&b);
      }
    }
    // [D/16][16][16] x 1 byte: 8 dims are half of a 16-byte group
    *reinterpret_cast<uint2*>(page + ((d0 >> 4) * 16 + off) * 16 + (d0 & 15)) = *reinterpret_cast<const uint2*>(o);
  }
}
template <bool BF16, int KVF8>
__device__ __forceinline__ void cache_put_v(const TcParams& p, int64_t blk, int off, int kvh, int d0, uint4 v,
                                            float scale) {
  uint8_t* page = p.vcw + blk * p.vcw_sb + (int64_t)kvh * p.vcw_sh;  // [D][16]
  if constexpr (KVF8 == 0) {
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
    for (int x = 0; x < 8; ++x) *reinterpret_cast<uint16_t*>(page + ((d0 + x) * 16 + off) * 2) = e[x];
  } else {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack2<BF16>(w[i]);
      if constexpr (KVF8 == 1) {
        const __nv_fp8_e4m3 a(f.x / scale), b(f.y / scale);
        page[(d0 + 2 * i) * 16 + off] = *reinterpret_cast<const uint8_t*>(&a);
        page[(d0 + 2 * i + 1) * 16 + off] = *reinterpret_cast<const uint8_t*>(&b);
      } else {
        const __nv_fp8_e5m2 a(f.x / scale), b(f.y / scale);
        page[(d0 + 2 * i) * 16 + off] = *reinterpret_cast<const uint8_t*>(&a);
        page[(d0 + 2 * i + 1) * 16 + off] = *reinterpret_cast<const uint8_t*>(&b);
      }
    }
  }
}

// PAIR: two CTAs of a cluster run every MMA together (M = 256, 128 rows of each row tile
// per CTA).  Each CTA then holds only half of every K tile (64 of its 128 keys) and half of
// every V tile (64 of the D dims of all 128 keys), so a stage is half as large and the ring
// twice as deep.
template <int D, bool PAIR = false>
struct TcCfg {
  static constexpr int kStages = ((D == 128) ? 2 : 4) * (PAIR ? 2 : 1);
  static constexpr int kPageBytes = D * 16 * 2;            // one page of one head, 16-bit elements
  static constexpr int kTileBytes = kPageBytes * kPagesPerTile;
  static constexpr int kKStageBytes = PAIR ? kTileBytes / 2 : kTileBytes;   // this CTA's part of a K tile
  static constexpr int kVPageBytes = PAIR ? kPageBytes / 2 : kPageBytes;    // this CTA's part of a V page
  static constexpr int kVStageBytes = kVPageBytes * kPagesPerTile;
  static constexpr int kQBytes = 2 * 128 * D * 2;
  static constexpr int kRowGroupBytes = D * 16;            // 8 rows x D x 2 B
  static constexpr int kSmemBytes = kQBytes + kStages * (kKStageBytes + kVStageBytes) + 1024;
};

template <int D, bool BF16, int KVF8, bool PAIR>
__device__ __forceinline__ void prefill_tc_body(const CUtensorMap& mapK, const CUtensorMap& mapV, const TcParams& p) {
  using Cfg = TcCfg<D, PAIR>;
  constexpr int KS = Cfg::kStages;
  constexpr int NCH = D / 8;  // 16-byte chunks per row
  constexpr bool MB = BF16 && KVF8 == 0;  // MMA operand type: bf16, else f16 (always f16 with an fp8 cache)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned; align by hand
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kQBytes;
  uint8_t* sV = sK + KS * Cfg::kKStageBytes;
  __shared__ __align__(8) uint64_t bar_k_tma[KS], bar_k_ready[KS], bar_k_empty[KS];
  __shared__ __align__(8) uint64_t bar_v_tma[KS], bar_v_ready[KS], bar_v_empty[KS];
  __shared__ __align__(8) uint64_t bar_s_full[2], bar_p_full[2], bar_o_done, bar_q_ready;
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mb = blockIdx.x, kvh = blockIdx.y;
  const int b = blockIdx.z / p.n_splits, split = blockIdx.z % p.n_splits;
#ifdef LA_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp & 3) == 0;
#endif
  const int s0 = p.qsl[b];
  const int qlen = p.qsl[b + 1] - s0;
  if (qlen <= 0 || (p.skip_decode && qlen == 1)) return;
  const int G = p.G;
  const int nrows = qlen * G;
  const int row0 = mb * kRowsPerCta;
  // In a pair both CTAs take every decision about the tile range from the pair's rows, so
  // that they agree on it: a CTA whose own rows lie past the request's last row still loads
  // and stages its halves of the K/V tiles for its partner.
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;
  const int row0_pair = PAIR ? (mb & ~1) * kRowsPerCta : row0;
  constexpr int kRowsPerUnit = PAIR ? 2 * kRowsPerCta : kRowsPerCta;
  if (row0_pair >= nrows) return;
  const int ctx = p.seq_lens[b] - qlen;
  const int ctx_pages = (ctx + 15) >> 4;
  const int n_ctx = (ctx_pages + kPagesPerTile - 1) / kPagesPerTile;
  const int tok_hi = min(qlen - 1, (row0_pair + kRowsPerUnit - 1) >> p.g_shift);
  const int n_self = tok_hi / kTileN + 1;
  const int total = n_ctx + n_self;
  const int j0 = (int)((int64_t)total * split / p.n_splits);
  const int j1 = (int)((int64_t)total * (split + 1) / p.n_splits);
  const bool lazy = (p.rot_mode == LA_ROT_MEPIC) ? true : (p.is_lazy != nullptr && p.is_lazy[b] != 0);
  // Per-page metadata: one 8-byte entry of the packed table when the caller has one,
  // else the three int32 tables (which share one row stride).
  const int64_t* pk_row = p.packed ? p.packed + (int64_t)b * p.packed_stride : nullptr;
  const int32_t* bt_row = p.block_table ? p.block_table + (int64_t)b * p.table_stride : nullptr;
  const int32_t* off_row = p.q_offset ? p.q_offset + (int64_t)b * p.table_stride : nullptr;
  const int32_t* msk_row = p.q_mask ? p.q_mask + (int64_t)b * p.table_stride : nullptr;
  auto page_block = [&](int page) -> int { return pk_row ? (int)(pk_row[page] >> 32) : bt_row[page]; };
  auto page_offset = [&](int page) -> int {
    return pk_row ? (int)((pk_row[page] >> 16) & 0xFFFF) : (off_row ? off_row[page] : 0);
  };
  auto page_pad = [&](int page) -> int {
    return pk_row ? (int)(pk_row[page] & 0xFFFF) : (msk_row ? msk_row[page] : 0);
  };

  // Barriers the MMA-issuing thread waits on collect the arrivals of both CTAs of a pair
  // (they live in the pair's first CTA, the only one that issues MMAs); the barriers the MMA
  // completions signal exist in both CTAs and are signalled in both.
  constexpr uint32_t kProducers = PAIR ? 2 : 1;
  if (tid == 0) {
    for (int i = 0; i < KS; ++i) {
      mbar_init(&bar_k_tma[i], 1);
      mbar_init(&bar_k_ready[i], 128 * kProducers);
      mbar_init(&bar_k_empty[i], 1);
      mbar_init(&bar_v_tma[i], 1);
      mbar_init(&bar_v_ready[i], 128 * kProducers);
      mbar_init(&bar_v_empty[i], 1);
    }
    mbar_init(&bar_s_full[0], 1);
    mbar_init(&bar_s_full[1], 1);
    mbar_init(&bar_p_full[0], 128 * kProducers);
    mbar_init(&bar_p_full[1], 128 * kProducers);
    mbar_init(&bar_o_done, 1);
    mbar_init(&bar_q_ready, kSoftmaxThreads * kProducers);
    mbar_fence_init();
  }
  if (warp == kWarpMma) {
    if constexpr (PAIR) {
      tmem_alloc_pair(&tmem_base_s, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&tmem_base_s, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  // no thread may touch the partner's barriers before the partner has initialised them
  if constexpr (PAIR) cluster_sync_all();
  tc_fence_after_sync();
  // Arrival on a barrier of the MMA-issuing CTA: local in the single-CTA kernel and in the
  // pair's first CTA, through the cluster window from the second.
  auto arrive_at_leader = [&](uint64_t* bar) {
    if constexpr (PAIR) {
      mbar_arrive_cluster(map_to_cta(smem_u32(bar), 0));
    } else {
      mbar_arrive(bar);
    }
  };
  const uint32_t tmem = tmem_base_s;
  const int ntiles = j1 - j0;
  // fp8 caches: the K scale folds into the score scale of the cached tiles, the V
  // scale into the output (the new tokens' V rows are staged divided by it)
  const float scale_log2_ctx = p.scale_log2 * ((KVF8 != 0 && p.k_scale) ? *p.k_scale : 1.f);
  const float out_scale = (KVF8 != 0 && p.v_scale) ? *p.v_scale : 1.f;

  if (warp < kWarpStage) {
    // =============================== softmax ===============================
    regs_raise<kRegsSoftmax>();
    // One thread per score row.  The row's 128 scores of a tile are consumed in four
    // 32-column chunks: while one chunk is scaled, exponentiated and packed, the
    // tensor-memory load of the next is already in flight.  P (two keys per column) is
    // written over S columns that have been read: keys 0..63 over columns 0..31, keys
    // 64..127 over columns 96..127 (see p_col).
    const int t = warp >> 2;          // row tile
    const int qd = warp & 3;          // lane quarter of tensor memory this warp may touch
    const int r = qd * 32 + lane;     // row within the tile
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const uint32_t tS = tmem + t * 128 + lane_addr;
    const uint32_t tO = tmem + 256 + t * 128 + lane_addr;
    const int R = row0 + t * 128 + r;
    const int tq = R >> p.g_shift;
    // ---- Q tiles: rows R = row0 .. row0+255, chunk-coalesced global reads.  The softmax
    // warps have nothing to do until the first scores exist, so they stage Q while the
    // staging warps already work on the first K tile.
    if (p.q_pos != nullptr) {
      // Fused rotary op: q arrives without rotary embedding; each (chunk, chunk + D/2) pair of
      // a row is rotated forward at the token's position while it is staged (same packed
      // 16-bit arithmetic as the K rotation), q itself stays as it is.
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q);
      const uint8_t* csb = reinterpret_cast<const uint8_t*>(p.cs);
#pragma unroll 2
      for (int idx = tid; idx < kRowsPerCta * (NCH / 2); idx += kSoftmaxThreads) {
        const int row = idx / (NCH / 2), g = idx - row * (NCH / 2);
        const int Rq = row0 + row;
        const int tqq = Rq >> p.g_shift;
        uint4 a = make_uint4(0, 0, 0, 0), bq = make_uint4(0, 0, 0, 0);
        if (tqq < qlen) {
          const int head = kvh * G + (Rq & (G - 1));
          const uint8_t* qrow = qb + ((int64_t)(s0 + tqq) * p.q_st + (int64_t)head * p.q_sh) * 2;
          a = *reinterpret_cast<const uint4*>(qrow + g * 16);
          bq = *reinterpret_cast<const uint4*>(qrow + (g + NCH / 2) * 16);
          int64_t pos = p.q_pos[s0 + tqq];
          if (pos >= p.cs_rows) pos = p.cs_rows - 1;
          if (pos > 0) {
            const uint8_t* crow = csb + pos * D * 2;
            const uint4 cv = __ldg(reinterpret_cast<const uint4*>(crow + g * 16));
            const uint4 sv = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 16));
            rotate_chunk<BF16>(a, bq, cv, sv);
          }
          if constexpr (BF16 && !MB) {
            a = bf16x8_to_f16x8(a);
            bq = bf16x8_to_f16x8(bq);
          }
        }
        uint8_t* dst = sQ + (row >> 3) * Cfg::kRowGroupBytes + (row & 7) * 16;
        *reinterpret_cast<uint4*>(dst + g * 128) = a;
        *reinterpret_cast<uint4*>(dst + (g + NCH / 2) * 128) = bq;
      }
      fence_proxy_async_smem();
      arrive_at_leader(&bar_q_ready);
    } else {
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(p.q);
#pragma unroll 4
      for (int idx = tid; idx < kRowsPerCta * NCH; idx += kSoftmaxThreads) {
        const int row = idx / NCH, g = idx - row * NCH;
        const int Rq = row0 + row;
        const int tqq = Rq >> p.g_shift;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (tqq < qlen) {
          const int head = kvh * G + (Rq & (G - 1));
          val = *reinterpret_cast<const uint4*>(qb + ((int64_t)(s0 + tqq) * p.q_st + (int64_t)head * p.q_sh) * 2 + g * 16);
          if constexpr (BF16 && !MB) val = bf16x8_to_f16x8(val);
        }
        *reinterpret_cast<uint4*>(sQ + (row >> 3) * Cfg::kRowGroupBytes + g * 128 + (row & 7) * 16) = val;
      }
      fence_proxy_async_smem();
      arrive_at_leader(&bar_q_ready);
    }
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    // per-page valid-token counts of a cached tile (lanes 0..7 hold pages 0..7);
    // fetched one tile ahead so that the table read is off the critical path
    auto page_valid = [&](int j) -> int {
      int v = 16;
      if (j < n_ctx && j < j1 && lane < kPagesPerTile) {
        const int page = j * kPagesPerTile + lane;
        v = 0;
        if (page < ctx_pages) {
          const int pad = lazy ? page_pad(page) : 0;
          v = min(ctx, (page + 1) * 16 - pad) - page * 16;
          v = max(0, min(16, v));
        }
      }
      return v;
    };
    // One 32-column chunk of a new-token tile: causal mask, row maximum, lazy rescale,
    // exponentials, P.
    auto do_chunk = [&](uint32_t (&sc)[32], const int c, const int j, const int n0, const float scale_log2) {
      {
        const int lim = tq - (n0 + c * 32);  // columns 0..lim are visible
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i > lim) sc[i] = 0xff800000u;
      }
      float mx0 = fmax3(__uint_as_float(sc[0]), __uint_as_float(sc[1]), __uint_as_float(sc[2]));
      float mx1 = fmax3(__uint_as_float(sc[3]), __uint_as_float(sc[4]), __uint_as_float(sc[5]));
#pragma unroll
      for (int i = 6; i + 3 < 32; i += 4) {
        mx0 = fmax3(mx0, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
      }
      mx0 = fmax3(mx0, __uint_as_float(sc[30]), __uint_as_float(sc[31]));
      const float m_chunk = fmaxf(mx0, mx1) * scale_log2;
      float alpha = 1.f;
      if (j == j0 && c == 0) {
        m_used = m_chunk;
      } else if (m_chunk > m_used + kRescaleThreshold) {
        alpha = ex2f(m_used - m_chunk);  // m_used == -inf gives 0
        m_used = m_chunk;
      }
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
        // Rare (the running maximum grew by more than the threshold): bring what was
        // accumulated under the old maximum to the new one.  Tensor-memory accesses
        // are warp-collective, so the whole warp takes this path together.
        l_sum *= alpha;
        if (j != j0) {
#pragma unroll 1
          for (int oc = 0; oc < D / 32; ++oc) {
            uint32_t o[32];
            tmem_ld32(tO + oc * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + oc * 32, o);
          }
        }
#pragma unroll 1
        for (int pc = 0; pc < c; ++pc) {  // P chunks of this tile formed with the old maximum
          uint32_t pp[16];
          tmem_ld16(tS + p_col(pc), pp);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 f = unpack2<MB>(pp[i]);
            pp[i] = pack2<MB>(f.x * alpha, f.y * alpha);
          }
          tmem_st16(tS + p_col(pc), pp);
        }
        tmem_st_wait();
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(neg_m, neg_m);
      uint32_t pk[16];
      float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
      // three passes over the registers: arguments, exponentials (the 32 MUFU
      // operations back to back), then sums and packing
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), sc2, nm2);
        sc[i] = __float_as_uint(x.x);
        sc[i + 1] = __float_as_uint(x.y);
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) sc[i] = __float_as_uint(ex2f(__uint_as_float(sc[i])));
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 e = make_float2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
        if (i & 2) acc_b = __fadd2_rn(acc_b, e); else acc_a = __fadd2_rn(acc_a, e);
        if constexpr (MB) {
          const uint32_t b0 = sc[i] + 0x8000u;  // round-half-up, then keep the high halves
          const uint32_t b1 = sc[i + 1] + 0x8000u;
          pk[i >> 1] = __byte_perm(b0, b1, 0x7632);
        } else {
          pk[i >> 1] = pack2<false>(e.x, e.y);
        }
      }
      l_sum += (acc_a.x + acc_a.y) + (acc_b.x + acc_b.y);
      tmem_st16(tS + p_col(c), pk);
    };
    int vc_next = page_valid(j0);
    for (int j = j0; j < j1 && ok; ++j) {
      const bool self = j >= n_ctx;
      const int vc = vc_next;
      vc_next = page_valid(j + 1);
      const bool tile_full = self ? false : (__all_sync(0xffffffffu, vc == 16) != 0);
      const int n0 = self ? (j - n_ctx) * kTileN : 0;
      const float scale_log2 = self ? p.scale_log2 : scale_log2_ctx;
      ok = mbar_wait(&bar_s_full[t], (uint32_t)(j - j0) & 1u, p.status, 101 + t);
      if (!ok) break;
      tc_fence_after_sync();
      LA_STAMP(t * 8 + 0, j - j0);
      uint32_t sa[32], sb[32];
      // Cached tiles: two passes over the row, compiled twice.  RAGGED: keys that do not exist
      // (the padding at the end of a document's last page, the slots past the context in its last
      // page) are set to -inf right after each load, by the per-page counts in `vc`; the copy
      // for full tiles carries no trace of it.  (One copy with run-time tests cost the full tiles
      // 3-5 %, this form 1.3 %, and ragged tiles on the chunk-by-chunk path cost a workload of
      // ragged documents 4 %.)
      auto two_pass = [&](auto ragged_tag) {
        constexpr bool RAGGED = decltype(ragged_tag)::value;
        auto mask_chunk = [&](uint32_t (&sc)[32], const int c) {
          if constexpr (RAGGED) {
            const int va = __shfl_sync(0xffffffffu, vc, 2 * c), vb = __shfl_sync(0xffffffffu, vc, 2 * c + 1);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              if (i >= va) sc[i] = 0xff800000u;
              if (i >= vb) sc[16 + i] = 0xff800000u;
            }
          }
        };
        // Pass A: the row maximum of the whole tile, so that the one decision about the
        // running maximum is taken before any exponential is formed.
        tmem_ld32(tS, sa);
        tmem_ld32(tS + 32, sb);
        tmem_ld_wait_for(sa);
        tie_after_wait(sb);
        mask_chunk(sa, 0);
        mask_chunk(sb, 1);
        float mx_a = row_max32(sa), mx_b = row_max32(sb);
        tmem_ld32(tS + 64, sa);
        tmem_ld32(tS + 96, sb);
        tmem_ld_wait_for(sa);
        tie_after_wait(sb);
        mask_chunk(sa, 2);
        mask_chunk(sb, 3);
        mx_a = fmaxf(mx_a, row_max32(sa));
        mx_b = fmaxf(mx_b, row_max32(sb));
        const float m_tile = fmaxf(mx_a, mx_b) * scale_log2;
        LA_STAMP(t * 8 + 1, j - j0);
        float alpha = 1.f;
        if (j == j0) {
          m_used = m_tile;
        } else if (m_tile > m_used + kRescaleThreshold) {
          alpha = ex2f(m_used - m_tile);  // m_used == -inf gives 0
          m_used = m_tile;
        }
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          // rare: bring the accumulator row and the row sum to the new maximum
          l_sum *= alpha;
          if (j != j0) {
#pragma unroll 1
            for (int oc = 0; oc < D / 32; ++oc) {
              uint32_t o[32];
              tmem_ld32(tO + oc * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + oc * 32, o);
            }
            tmem_st_wait();
          }
        }
        // Pass B: exponentials and P, one straight-line block for the four chunks, starting
        // with chunks 2 and 3, which pass A left in registers, while chunks 0 and 1 are
        // fetched again.  bf16 P is formed by truncation of e * (1 + 2^-9) (the factor rides
        // on the subtracted maximum), which is unbiased like rounding and costs one byte
        // permute per pair instead of two integer adds and a permute; the row sum is taken
        // from the same values and scaled back by 1 / (1 + 2^-9).
        constexpr float kBiasLog2 = MB ? 0.0028151247f : 0.f;       // log2(1 + 2^-9)
        constexpr float kUnbias = MB ? 0.998050682f : 1.f;          // 1 / (1 + 2^-9)
        const float neg_m = ((m_used == -INFINITY) ? 0.f : -m_used) + kBiasLog2;
        const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(neg_m, neg_m);
        float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
        auto exp_chunk = [&](uint32_t (&sc)[32], const int c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), sc2, nm2);
            const float2 e = make_float2(ex2_pure(x.x), ex2_pure(x.y));
            if (i & 2) acc_b = __fadd2_rn(acc_b, e); else acc_a = __fadd2_rn(acc_a, e);
            if constexpr (MB) {
              pk[i >> 1] = __byte_perm(__float_as_uint(e.x), __float_as_uint(e.y), 0x7632);
            } else {
              pk[i >> 1] = pack2<false>(e.x, e.y);
            }
          }
          tmem_st16(tS + p_col(c), pk);
        };
        exp_chunk(sa, 2);
        tmem_ld32(tS, sa);
        LA_STAMP(t * 8 + 2, j - j0);
        exp_chunk(sb, 3);
        tmem_ld_wait_for(sa);
        tmem_ld32(tS + 32, sb);
        LA_STAMP(t * 8 + 3, j - j0);
        mask_chunk(sa, 0);
        exp_chunk(sa, 0);
        tmem_ld_wait_for(sb);
        LA_STAMP(t * 8 + 4, j - j0);
        mask_chunk(sb, 1);
        exp_chunk(sb, 1);
        LA_STAMP(t * 8 + 5, j - j0);
        l_sum = fmaf((acc_a.x + acc_a.y) + (acc_b.x + acc_b.y), kUnbias, l_sum);
        tmem_st_wait();
        tc_fence_before_sync();
        arrive_at_leader(&bar_p_full[t]);
        LA_STAMP(t * 8 + 6, j - j0);
      };
      if (tile_full) {
        two_pass(std::false_type{});
        continue;
      }
      if (!self) {
        two_pass(std::true_type{});
        continue;
      }
      // ---- new-token tiles (causal mask per row): chunk by chunk
      tmem_ld32(tS, sa);
      tmem_ld_wait();
      LA_STAMP(t * 8 + 1, j - j0);
      tmem_ld32(tS + 32, sb);
      do_chunk(sa, 0, j, n0, scale_log2);
      LA_STAMP(t * 8 + 2, j - j0);
      tmem_ld_wait();
      tmem_ld32(tS + 64, sa);
      do_chunk(sb, 1, j, n0, scale_log2);
      LA_STAMP(t * 8 + 3, j - j0);
      tmem_ld_wait();
      tmem_ld32(tS + 96, sb);
      tmem_ld_wait();  // P of chunk 2 goes over the columns of chunk 3: have chunk 3 in registers first
      do_chunk(sa, 2, j, n0, scale_log2);
      LA_STAMP(t * 8 + 4, j - j0);
      do_chunk(sb, 3, j, n0, scale_log2);
      LA_STAMP(t * 8 + 5, j - j0);
      tmem_st_wait();
      tc_fence_before_sync();
      arrive_at_leader(&bar_p_full[t]);
      LA_STAMP(t * 8 + 6, j - j0);
    }
    // ---- epilogue: each thread writes its row
    if (ok && ntiles > 0) ok = mbar_wait(&bar_o_done, 0, p.status, 111 + t);
    tc_fence_after_sync();
    const float l_row = l_sum;
    // Tensor-memory loads are warp-collective: every lane of the warp runs them,
    // rows past the request's last token only skip the global stores.
    const bool ok_warp = __all_sync(0xffffffffu, ok) != 0;
    if (ok_warp) {
      const bool row_valid = tq < qlen;
      const int head = kvh * G + (R & (G - 1));
      if (p.n_splits == 1) {
        const float inv = l_row > 0.f ? out_scale / l_row : 0.f;
        uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                        ((int64_t)(s0 + tq) * p.o_st + (int64_t)head * p.o_sh) * 2;
        // Fused gather: the warp's 32 rows go through shared memory (the Q tiles are no longer
        // read once every MMA has completed) so that a row leaves as one contiguous run of
        // 16-byte stores; one row per thread would cross the link as 16-byte pieces.
        constexpr int kRowBytes = D * 2, kRowChunks = kRowBytes / 16;
        const bool to_peers = p.peer.num_peers > 0;
        uint8_t* stage_rows = sQ + (t * 128 + qd * 32) * kRowBytes;
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t o[32];
          tmem_ld32(tO + ch * 32, o);
          tmem_ld_wait();
          uint4 w[4];
          uint32_t* pw = reinterpret_cast<uint32_t*>(w);
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            pw[i >> 1] = pack2<BF16>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
          if (to_peers) {
            // chunk c of row `lane` sits at slot c ^ (lane mod chunks): eight lanes hit eight
            // different 16-byte bank groups on the way in and on the way out
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(stage_rows + lane * kRowBytes +
                                        (((ch * 4 + i) ^ (lane & (kRowChunks - 1))) << 4)) = w[i];
          } else if (row_valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(orow + ch * 64 + i * 16) = w[i];
          }
        }
        if (to_peers) {
          __syncwarp();
          constexpr int kRowsPerPass = 32 / kRowChunks;  // rows one warp-wide store covers
          const int c = lane & (kRowChunks - 1);
#pragma unroll 1
          for (int pass = 0; pass < 32 / kRowsPerPass; ++pass) {
            const int rr = pass * kRowsPerPass + lane / kRowChunks;
            const int Rr = row0 + t * 128 + qd * 32 + rr;
            const int tqr = Rr >> p.g_shift;
            if (tqr < qlen) {
              const uint4 val = *reinterpret_cast<const uint4*>(stage_rows + rr * kRowBytes +
                                                                ((c ^ (rr & (kRowChunks - 1))) << 4));
              const int hr = kvh * G + (Rr & (G - 1));
              const int64_t prow = p.peer.rows ? p.peer.rows[s0 + tqr] : (s0 + tqr);
              const int64_t off =
                  (prow * p.peer.stride_t + (int64_t)(p.peer.head_offset + hr) * p.peer.stride_h) * 2 + c * 16;
              for (int q = 0; q < p.peer.num_peers; ++q)
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer.out[q]) + off) = val;
            }
          }
        }
      } else {
        const int64_t slot = (((int64_t)b * p.Hkv + kvh) * p.rows_cap + R) * p.n_splits + split;
        float* po = p.part_o + slot * D;
        if (ntiles > 0) {
#pragma unroll 1
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t o[32];
            tmem_ld32(tO + ch * 32, o);
            tmem_ld_wait();
            if (row_valid) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(po + ch * 32 + i) =
                    make_float4(__uint_as_float(o[i]) * out_scale, __uint_as_float(o[i + 1]) * out_scale,
                                __uint_as_float(o[i + 2]) * out_scale, __uint_as_float(o[i + 3]) * out_scale);
            }
          }
        }
        if (row_valid) {
          p.part_ml[slot * 2] = ntiles > 0 ? m_used : -INFINITY;
          p.part_ml[slot * 2 + 1] = ntiles > 0 ? l_row : 0.f;
        }
      }
    }
  } else if (warp < kWarpMma) {
    // =============================== operand staging ===============================
    regs_lower<kRegsStage>();
    const int i = tid - kWarpStage * 32;  // 0..127
    bool ok = true;
    const uint8_t* cs = reinterpret_cast<const uint8_t*>(p.cs);
    // Fused cache write: the unit that holds the request's last row stages every new-token
    // tile of the request (each tile in exactly one of its splits) and stores the raw rows.
    const bool put = p.slots != nullptr && row0_pair + kRowsPerUnit >= nrows;
    const float put_ks = (KVF8 != 0 && p.k_scale) ? *p.k_scale : 1.f;
    const float put_vs = (KVF8 != 0 && p.v_scale) ? *p.v_scale : 1.f;
    // fp8 caches: asynchronous copies of tile jn's raw pages into its operand stage
    // (after the stage's previous tile was consumed).  One commit group per call,
    // also when there is nothing to copy, so that the group count stays uniform.
    auto issue_raw_k = [&](int jn) -> bool {
      bool good = true;
      if (jn < j1 && jn < n_ctx) {
        const int stn = (jn - j0) % KS, un = (jn - j0) / KS;
        if (un > 0) good = mbar_wait(&bar_k_empty[stn], (uint32_t)(un - 1) & 1u, p.status, 204);
        if constexpr (PAIR) {
          // This CTA's 64 keys, two threads per key.  Thread `hc` of a key converts the raw pieces
          // g in [hc * NL/4, (hc+1) * NL/4) and their rotation partners g + NL/2; their raw bytes
          // land in the first NL/2 of the chunk slots that this thread alone writes later.
          constexpr int NL = D / 16;
          const int key = i & 63, hc = i >> 6;
          const int page = jn * kPagesPerTile + 4 * (int)cta_rank + (key >> 4);
          if (good && page < ctx_pages) {
            int64_t blk = page_block(page);
            if (blk < 0 || blk >= p.num_blocks) blk = 0;
            const uint8_t* src = p.kc + blk * p.kc_sb + (int64_t)kvh * p.kc_sh + (key & 15) * 16;
            const uint32_t dst =
                smem_u32(sK + stn * Cfg::kKStageBytes + (key >> 3) * Cfg::kRowGroupBytes + (key & 7) * 16);
#pragma unroll
            for (int q = 0; q < NL / 4; ++q) {
              const int g = hc * (NL / 4) + q;
              cp_async_16(dst + (hc * (NL / 2) + q) * 128, src + g * 256);
              cp_async_16(dst + (hc * (NL / 2) + NL / 4 + q) * 128, src + (g + NL / 2) * 256);
            }
          }
        } else {
        const int page = jn * kPagesPerTile + (i >> 4);
        if (good && page < ctx_pages) {
          int64_t blk = page_block(page);
          if (blk < 0 || blk >= p.num_blocks) blk = 0;
          const uint8_t* src = p.kc + blk * p.kc_sb + (int64_t)kvh * p.kc_sh + (i & 15) * 16;
          const uint32_t dst = smem_u32(sK + stn * Cfg::kTileBytes + (i >> 3) * Cfg::kRowGroupBytes + (i & 7) * 16);
#pragma unroll
          for (int g = 0; g < D / 16; ++g) cp_async_16(dst + g * 128, src + g * 256);
        }
        }
      }
      cp_async_commit();
      return good;
    };
    auto issue_raw_v = [&](int jn) -> bool {
      bool good = true;
      if (jn < j1 && jn < n_ctx) {
        const int stn = (jn - j0) % KS, un = (jn - j0) / KS;
        if (un > 0) good = mbar_wait(&bar_v_empty[stn], (uint32_t)(un - 1) & 1u, p.status, 205);
        const int npages = min(kPagesPerTile, ctx_pages - jn * kPagesPerTile);
        if (good) {
          if constexpr (PAIR) {
            // this CTA's half of the head dimension of every page: D/2 rows of 16 tokens per page
#pragma unroll
            for (int it = 0; it < D / 32; ++it) {
              const int idx = i + it * 128;
              const int pg = idx / (D / 2), dl = idx - pg * (D / 2);
              if (pg < npages) {
                int64_t vb = page_block(jn * kPagesPerTile + pg);
                if (vb < 0 || vb >= p.num_blocks) vb = 0;
                cp_async_16(smem_u32(sV + stn * Cfg::kVStageBytes + pg * Cfg::kVPageBytes + (dl >> 3) * 256 + (dl & 7) * 16),
                            p.vc + vb * p.vc_sb + (int64_t)kvh * p.vc_sh + ((int)cta_rank * (D / 2) + dl) * 16);
              }
            }
          } else {
#pragma unroll
          for (int it = 0; it < D / 16; ++it) {  // one (page, dim) row of 16 tokens per piece
            const int idx = i + it * 128;
            const int pg = idx / D, d = idx - pg * D;
            if (pg < npages) {
              int64_t vb = page_block(jn * kPagesPerTile + pg);
              if (vb < 0 || vb >= p.num_blocks) vb = 0;
              cp_async_16(smem_u32(sV + stn * Cfg::kTileBytes + pg * Cfg::kPageBytes + (d >> 3) * 256 + (d & 7) * 16),
                          p.vc + vb * p.vc_sb + (int64_t)kvh * p.vc_sh + d * 16);
            }
          }
          }
        }
      }
      cp_async_commit();
      return good;
    };
    if constexpr (KVF8 != 0) {
      issue_raw_k(j0);
      issue_raw_v(j0);
    }
    // rotation entry of this thread's page, read one tile ahead of its use
    auto page_rot = [&](int jn) -> int {
      const int pg = jn * kPagesPerTile + (i >> 4);
      return (lazy && jn < j1 && pg < ctx_pages) ? page_offset(pg) : 0;
    };
    int rot_next = KVF8 != 0 ? page_rot(j0) : 0;
    for (int j = j0; j < j1 && ok; ++j) {
      const int st = (j - j0) % KS, u = (j - j0) / KS;
      uint8_t* kst = sK + st * Cfg::kKStageBytes;
      uint8_t* vst = sV + st * Cfg::kVStageBytes;
      if constexpr (PAIR) {
        // ---- CTA pair: this CTA stages its 64 keys of the K tile (two threads per key, each
        // rotating half of the row) and, for new-token tiles, its half of the head dimension
        // of V for all 128 keys.
        const int key = i & 63, hc = i >> 6;
        constexpr int NP = NCH / 4;  // (chunk, chunk + NCH/2) pairs per thread
        const int g0 = hc * NP;
        uint8_t* rowp = kst + (key >> 3) * Cfg::kRowGroupBytes + (key & 7) * 16;
        if (j < n_ctx) {
          const int page = j * kPagesPerTile + 4 * (int)cta_rank + (key >> 4);
          int pos = 0;
          if (lazy && page < ctx_pages) {
            const int rot = page_offset(page);
            if (p.rot_mode == LA_ROT_LAZY) {
              pos = rot != 0 ? rot - 1 : 0;
            } else {
              pos = p.is_mepic ? (page * 16 + (key & 15)) : ((rot != 0 ? rot - 1 : page * 16) + (key & 15));
            }
            if (pos >= p.cs_rows) pos = (int)p.cs_rows - 1;
          }
          const uint8_t* crow = cs + (int64_t)pos * D * 2;
          if constexpr (KVF8 != 0) {
            // fp8 cache: this CTA's raw pages of the tile were copied (cp.async, one tile ahead)
            // into the operand stage itself, every 16-byte piece into a chunk slot that only its
            // own thread reads and later overwrites.  Convert to f16 (exact), rotate K, and
            // write the MMA layouts in place.
            constexpr int NL = D / 16;
            const bool present = page < ctx_pages;
            const int npages = min(kPagesPerTile, ctx_pages - j * kPagesPerTile);
            cp_async_wait_group<1>();  // K pieces of tile j have landed
            uint4 kraw[NL / 2];
#pragma unroll
            for (int q = 0; q < NL / 2; ++q)
              kraw[q] = present ? *reinterpret_cast<const uint4*>(rowp + (hc * (NL / 2) + q) * 128)
                                : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int q = 0; q < NL / 4; ++q) {  // dims [16g, 16g+16) and their partners at +D/2
              const int g = hc * (NL / 4) + q;
              uint4 a0, a1, b0, b1;
              fp8x16_to_f16<KVF8>(kraw[q], a0, a1);
              fp8x16_to_f16<KVF8>(kraw[NL / 4 + q], b0, b1);
              if (pos > 0) {
                const uint4 c0 = __ldg(reinterpret_cast<const uint4*>(crow + g * 32));
                const uint4 c1 = __ldg(reinterpret_cast<const uint4*>(crow + g * 32 + 16));
                const uint4 s0v = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 32));
                const uint4 s1v = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 32 + 16));
                rotate_chunk_f16<BF16>(a0, b0, c0, s0v);
                rotate_chunk_f16<BF16>(a1, b1, c1, s1v);
              }
              *reinterpret_cast<uint4*>(rowp + (2 * g) * 128) = a0;
              *reinterpret_cast<uint4*>(rowp + (2 * g + 1) * 128) = a1;
              *reinterpret_cast<uint4*>(rowp + (2 * g + NCH / 2) * 128) = b0;
              *reinterpret_cast<uint4*>(rowp + (2 * g + 1 + NCH / 2) * 128) = b1;
            }
            fence_proxy_async_smem();
            arrive_at_leader(&bar_k_ready[st]);
            ok = issue_raw_k(j + 1);
            if (!ok) break;
            cp_async_wait_group<1>();  // V pieces of tile j have landed
#pragma unroll
            for (int it = 0; it < D / 32; ++it) {
              const int idx = i + it * 128;
              const int pg = idx / (D / 2), dl = idx - pg * (D / 2);
              if (pg < npages) {
                uint8_t* dst = vst + pg * Cfg::kVPageBytes + (dl >> 3) * 256 + (dl & 7) * 16;
                const uint4 raw = *reinterpret_cast<const uint4*>(dst);
                uint4 lo, hi;
                fp8x16_to_f16<KVF8>(raw, lo, hi);
                *reinterpret_cast<uint4*>(dst) = lo;
                *reinterpret_cast<uint4*>(dst + 128) = hi;
              }
            }
            fence_proxy_async_smem();
            arrive_at_leader(&bar_v_ready[st]);
            ok = issue_raw_v(j + 1);
            continue;
          }
          uint4 cv[NP], sv[NP];
          if (pos > 0) {
#pragma unroll
            for (int g = 0; g < NP; ++g) {
              cv[g] = __ldg(reinterpret_cast<const uint4*>(crow + (g0 + g) * 16));
              sv[g] = __ldg(reinterpret_cast<const uint4*>(crow + D + (g0 + g) * 16));
            }
          }
          ok = mbar_wait(&bar_k_tma[st], (uint32_t)u & 1u, p.status, 201);
          if (!ok) break;
          if (pos > 0) {
#pragma unroll
            for (int g = 0; g < NP; ++g) {
              uint4 a = *reinterpret_cast<uint4*>(rowp + (g0 + g) * 128);
              uint4 bq = *reinterpret_cast<uint4*>(rowp + (g0 + g + NCH / 2) * 128);
              rotate_chunk<BF16>(a, bq, cv[g], sv[g]);
              *reinterpret_cast<uint4*>(rowp + (g0 + g) * 128) = a;
              *reinterpret_cast<uint4*>(rowp + (g0 + g + NCH / 2) * 128) = bq;
            }
          }
          fence_proxy_async_smem();
          arrive_at_leader(&bar_k_ready[st]);
          LA_STAMP(20, j - j0);
        } else {
          if (u > 0) ok = mbar_wait(&bar_k_empty[st], (uint32_t)(u - 1) & 1u, p.status, 202);
          if (!ok) break;
          {
            const int n = (j - n_ctx) * kTileN + 64 * (int)cta_rank + key;
            const bool present = n < qlen;
            const uint8_t* krow = reinterpret_cast<const uint8_t*>(p.k) +
                                  ((int64_t)(s0 + n) * p.k_st + (int64_t)kvh * p.k_sh) * 2;
            int pos = 0;
            if (present && p.rot_mode == LA_ROT_MEPIC) {
              pos = ctx + n;
              if (pos >= p.cs_rows) pos = (int)p.cs_rows - 1;
            }
            const uint8_t* crow = cs + (int64_t)pos * D * 2;
#pragma unroll
            for (int g = 0; g < NP; ++g) {
              uint4 a = make_uint4(0, 0, 0, 0), bq = make_uint4(0, 0, 0, 0);
              if (present) {
                a = *reinterpret_cast<const uint4*>(krow + (g0 + g) * 16);
                bq = *reinterpret_cast<const uint4*>(krow + (g0 + g + NCH / 2) * 16);
                if (put) {
                  const int64_t slot = p.slots[s0 + n];
                  if (slot >= 0) {
                    cache_put_k<BF16, KVF8>(p, slot >> 4, (int)(slot & 15), kvh, (g0 + g) * 8, a, put_ks);
                    cache_put_k<BF16, KVF8>(p, slot >> 4, (int)(slot & 15), kvh, (g0 + g + NCH / 2) * 8, bq, put_ks);
                  }
                }
                if (pos > 0) {
                  const uint4 cvv = __ldg(reinterpret_cast<const uint4*>(crow + (g0 + g) * 16));
                  const uint4 svv = __ldg(reinterpret_cast<const uint4*>(crow + D + (g0 + g) * 16));
                  rotate_chunk<BF16>(a, bq, cvv, svv);
                }
                if constexpr (BF16 && !MB) {
                  a = bf16x8_to_f16x8(a);
                  bq = bf16x8_to_f16x8(bq);
                }
              }
              *reinterpret_cast<uint4*>(rowp + (g0 + g) * 128) = a;
              *reinterpret_cast<uint4*>(rowp + (g0 + g + NCH / 2) * 128) = bq;
            }
          }
          fence_proxy_async_smem();
          arrive_at_leader(&bar_k_ready[st]);
          if (u > 0) ok = mbar_wait(&bar_v_empty[st], (uint32_t)(u - 1) & 1u, p.status, 203);
          if (!ok) break;
          {
            // V: thread i holds key i of the tile; this CTA keeps dims [rank * D/2, +D/2), transposed
            const int nv = (j - n_ctx) * kTileN + i;
            const bool presentv = nv < qlen;
            const uint8_t* vrow = reinterpret_cast<const uint8_t*>(p.v) +
                                  ((int64_t)(s0 + nv) * p.v_st + (int64_t)kvh * p.v_sh) * 2 + (int)cta_rank * D;
            uint8_t* base = vst + (i >> 4) * Cfg::kVPageBytes + ((i & 15) >> 3) * 128 + (i & 7) * 2;
#pragma unroll 2
            for (int g = 0; g < NCH / 2; ++g) {
              uint4 val = make_uint4(0, 0, 0, 0);
              if (presentv) {
                val = *reinterpret_cast<const uint4*>(vrow + g * 16);
                if (put) {
                  const int64_t slot = p.slots[s0 + nv];
                  if (slot >= 0)
                    cache_put_v<BF16, KVF8>(p, slot >> 4, (int)(slot & 15), kvh, (int)cta_rank * (D / 2) + g * 8, val, put_vs);
                }
                if constexpr (KVF8 != 0) val = to_f16x8_scaled<BF16>(val, 1.f / out_scale);
              }
              const uint16_t* e = reinterpret_cast<const uint16_t*>(&val);
#pragma unroll
              for (int x = 0; x < 8; ++x) *reinterpret_cast<uint16_t*>(base + g * 256 + x * 16) = e[x];
            }
          }
          fence_proxy_async_smem();
          arrive_at_leader(&bar_v_ready[st]);
        }
        continue;
      }
      int rot;
      if constexpr (KVF8 != 0) {
        rot = rot_next;
        rot_next = page_rot(j + 1);
      } else {
        rot = page_rot(j);
      }
      if (j < n_ctx) {
        const int page = j * kPagesPerTile + (i >> 4);
        int pos = 0;
        if (lazy && page < ctx_pages) {
          if (p.rot_mode == LA_ROT_LAZY) {
            pos = rot != 0 ? rot - 1 : 0;
          } else {
            pos = p.is_mepic ? (page * 16 + (i & 15)) : ((rot != 0 ? rot - 1 : page * 16) + (i & 15));
          }
          if (pos >= p.cs_rows) pos = (int)p.cs_rows - 1;
        }
        if constexpr (KVF8 != 0) {
          // fp8 cache: the raw pages of this tile were copied (cp.async, one tile
          // ahead) into the operand stage itself, every 16-byte piece at a place
          // that only its own thread reads and overwrites.  Convert to f16
          // (exact), rotate K, and write the MMA layouts in place.
          constexpr int NL = D / 16;  // raw 16-byte pieces per thread for K, and for V
          const bool present = page < ctx_pages;
          const int npages = min(kPagesPerTile, ctx_pages - j * kPagesPerTile);
          cp_async_wait_group<1>();  // K pieces of tile j have landed
          uint8_t* rowp = kst + (i >> 3) * Cfg::kRowGroupBytes + (i & 7) * 16;
          uint4 kraw[NL];
#pragma unroll
          for (int g = 0; g < NL; ++g)
            kraw[g] = present ? *reinterpret_cast<const uint4*>(rowp + g * 128) : make_uint4(0, 0, 0, 0);
          const uint8_t* crow = cs + (int64_t)pos * D * 2;
#pragma unroll
          for (int g = 0; g < NL / 2; ++g) {  // dims [16g, 16g+16) and their partners at +D/2
            uint4 a0, a1, b0, b1;
            fp8x16_to_f16<KVF8>(kraw[g], a0, a1);
            fp8x16_to_f16<KVF8>(kraw[g + NL / 2], b0, b1);
            if (pos > 0) {
              const uint4 c0 = __ldg(reinterpret_cast<const uint4*>(crow + g * 32));
              const uint4 c1 = __ldg(reinterpret_cast<const uint4*>(crow + g * 32 + 16));
              const uint4 s0v = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 32));
              const uint4 s1v = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 32 + 16));
              rotate_chunk_f16<BF16>(a0, b0, c0, s0v);
              rotate_chunk_f16<BF16>(a1, b1, c1, s1v);
            }
            *reinterpret_cast<uint4*>(rowp + (2 * g) * 128) = a0;
            *reinterpret_cast<uint4*>(rowp + (2 * g + 1) * 128) = a1;
            *reinterpret_cast<uint4*>(rowp + (2 * g + NCH / 2) * 128) = b0;
            *reinterpret_cast<uint4*>(rowp + (2 * g + 1 + NCH / 2) * 128) = b1;
          }
          fence_proxy_async_smem();
          mbar_arrive(&bar_k_ready[st]);
          ok = issue_raw_k(j + 1);
          if (!ok) break;
          cp_async_wait_group<1>();  // V pieces of tile j have landed
#pragma unroll
          for (int it = 0; it < NL; ++it) {
            const int idx = i + it * 128;
            const int pg = idx / D, d = idx - pg * D;
            if (pg < npages) {
              uint8_t* dst = vst + pg * Cfg::kPageBytes + (d >> 3) * 256 + (d & 7) * 16;
              const uint4 raw = *reinterpret_cast<const uint4*>(dst);
              uint4 lo, hi;
              fp8x16_to_f16<KVF8>(raw, lo, hi);
              *reinterpret_cast<uint4*>(dst) = lo;
              *reinterpret_cast<uint4*>(dst + 128) = hi;
            }
          }
          fence_proxy_async_smem();
          mbar_arrive(&bar_v_ready[st]);
          ok = issue_raw_v(j + 1);
          continue;
        }
        // The table row is known before the page lands: fetch its first half now,
        // so that (per-token mode: one row per thread, L2 latency) the loads
        // overlap the wait for the copy.
        constexpr int NPRE = NCH / 4;
        const uint8_t* crow = cs + (int64_t)pos * D * 2;
        uint4 cpre[NPRE], spre[NPRE];
        if (pos > 0) {
#pragma unroll
          for (int g = 0; g < NPRE; ++g) {
            cpre[g] = __ldg(reinterpret_cast<const uint4*>(crow + g * 16));
            spre[g] = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 16));
          }
        }
        ok = mbar_wait(&bar_k_tma[st], (uint32_t)u & 1u, p.status, 201);
        if (!ok) break;
        LA_STAMP(21, j - j0);
        if (pos > 0) {
          uint8_t* rowp = kst + (i >> 3) * Cfg::kRowGroupBytes + (i & 7) * 16;
          uint4 cpost[NPRE], spost[NPRE];
#pragma unroll
          for (int g = 0; g < NPRE; ++g) {
            cpost[g] = __ldg(reinterpret_cast<const uint4*>(crow + (g + NPRE) * 16));
            spost[g] = __ldg(reinterpret_cast<const uint4*>(crow + D + (g + NPRE) * 16));
          }
#pragma unroll
          for (int g = 0; g < NCH / 2; ++g) {
            uint4 a = *reinterpret_cast<uint4*>(rowp + g * 128);
            uint4 bq = *reinterpret_cast<uint4*>(rowp + (g + NCH / 2) * 128);
            rotate_chunk<BF16>(a, bq, g < NPRE ? cpre[g] : cpost[g - NPRE], g < NPRE ? spre[g] : spost[g - NPRE]);
            *reinterpret_cast<uint4*>(rowp + g * 128) = a;
            *reinterpret_cast<uint4*>(rowp + (g + NCH / 2) * 128) = bq;
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bar_k_ready[st]);
        LA_STAMP(20, j - j0);
      } else {
        // new tokens: K rows into the operand layout (rotated in per-token mode), V transposed
        if (u > 0) ok = mbar_wait(&bar_k_empty[st], (uint32_t)(u - 1) & 1u, p.status, 202);
        if (!ok) break;
        const int n = (j - n_ctx) * kTileN + i;
        const bool present = n < qlen;
        {
          const uint8_t* krow = reinterpret_cast<const uint8_t*>(p.k) +
                                ((int64_t)(s0 + n) * p.k_st + (int64_t)kvh * p.k_sh) * 2;
          uint8_t* rowp = kst + (i >> 3) * Cfg::kRowGroupBytes + (i & 7) * 16;
          int pos = 0;
          if (present && p.rot_mode == LA_ROT_MEPIC) {
            pos = ctx + n;
            if (pos >= p.cs_rows) pos = (int)p.cs_rows - 1;
          }
          const uint8_t* crow = cs + (int64_t)pos * D * 2;
#pragma unroll 2
          for (int g = 0; g < NCH / 2; ++g) {
            uint4 a = make_uint4(0, 0, 0, 0), bq = make_uint4(0, 0, 0, 0);
            if (present) {
              a = *reinterpret_cast<const uint4*>(krow + g * 16);
              bq = *reinterpret_cast<const uint4*>(krow + (g + NCH / 2) * 16);
              if (put) {
                const int64_t slot = p.slots[s0 + n];
                if (slot >= 0) {
                  cache_put_k<BF16, KVF8>(p, slot >> 4, (int)(slot & 15), kvh, g * 8, a, put_ks);
                  cache_put_k<BF16, KVF8>(p, slot >> 4, (int)(slot & 15), kvh, (g + NCH / 2) * 8, bq, put_ks);
                }
              }
              if (pos > 0) {
                const uint4 cv = __ldg(reinterpret_cast<const uint4*>(crow + g * 16));
                const uint4 sv = __ldg(reinterpret_cast<const uint4*>(crow + D + g * 16));
                rotate_chunk<BF16>(a, bq, cv, sv);
              }
              if constexpr (BF16 && !MB) {
                a = bf16x8_to_f16x8(a);
                bq = bf16x8_to_f16x8(bq);
              }
            }
            *reinterpret_cast<uint4*>(rowp + g * 128) = a;
            *reinterpret_cast<uint4*>(rowp + (g + NCH / 2) * 128) = bq;
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bar_k_ready[st]);
        if (u > 0) ok = mbar_wait(&bar_v_empty[st], (uint32_t)(u - 1) & 1u, p.status, 203);
        if (!ok) break;
        {
          const float inv_out_scale = 1.f / out_scale;
          const uint8_t* vrow = reinterpret_cast<const uint8_t*>(p.v) +
                                ((int64_t)(s0 + n) * p.v_st + (int64_t)kvh * p.v_sh) * 2;
          uint8_t* base = vst + (i >> 4) * Cfg::kPageBytes + ((i & 15) >> 3) * 128 + (i & 7) * 2;
#pragma unroll 2
          for (int g = 0; g < NCH; ++g) {
            uint4 val = make_uint4(0, 0, 0, 0);
            if (present) {
              val = *reinterpret_cast<const uint4*>(vrow + g * 16);
              if (put) {
                const int64_t slot = p.slots[s0 + n];
                if (slot >= 0) cache_put_v<BF16, KVF8>(p, slot >> 4, (int)(slot & 15), kvh, g * 8, val, put_vs);
              }
              if constexpr (KVF8 != 0) val = to_f16x8_scaled<BF16>(val, inv_out_scale);
            }
            const uint16_t* e = reinterpret_cast<const uint16_t*>(&val);
#pragma unroll
            for (int x = 0; x < 8; ++x) *reinterpret_cast<uint16_t*>(base + g * 256 + x * 16) = e[x];
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bar_v_ready[st]);
      }
    }
  } else if (warp == kWarpMma) {
    // =============================== MMA issue ===============================
    regs_lower<kRegsIssue>();
    // In a pair only the first CTA issues: each MMA covers the 128 rows of a row tile in both
    // CTAs (M = 256), reading Q and P from each CTA and half of K / V from each CTA.
    if (ntiles > 0 && cta_rank == 0) {
      const bool issuer = lane == 0;
      constexpr int kM = PAIR ? 256 : 128;
      constexpr uint32_t idesc_qk = idesc_f16(MB ? 1 : 0, kM, kTileN);
      constexpr uint32_t idesc_pv = idesc_f16(MB ? 1 : 0, kM, D);
      auto wait_in = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        return mbar_wait(bar, parity, p.status, code);
      };
      auto commit = [&](uint64_t* bar) {
        if constexpr (PAIR) mma_commit_pair(bar); else mma_commit(bar);
      };
      bool ok = wait_in(&bar_q_ready, 0, 301);
      uint32_t v_ready_bits = 0;
      auto issue_qk = [&](int t, int st) {
        if (!issuer) return;
        const uint32_t qa = smem_u32(sQ) + t * (128 * D * 2);
        const uint32_t ka = smem_u32(sK) + st * Cfg::kKStageBytes;
        // descriptors of the first k-step; a k-step of 16 elements is 256 bytes further on
        // (the start-address field counts 16-byte units)
        const uint64_t da0 = smem_desc_nosw(qa, 128, Cfg::kRowGroupBytes);
        const uint64_t db0 = smem_desc_nosw(ka, 128, Cfg::kRowGroupBytes);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          if constexpr (PAIR) mma_ss_pair(tmem + t * 128, da0 + ks * 16, db0 + ks * 16, idesc_qk, ks > 0);
          else mma_ss(tmem + t * 128, da0 + ks * 16, db0 + ks * 16, idesc_qk, ks > 0);
        }
        commit(&bar_s_full[t]);
      };
      auto issue_pv = [&](int t, int st, int npages, bool first) {
        if (!issuer) return;
        const uint32_t va = smem_u32(sV) + st * Cfg::kVStageBytes;
        const uint64_t db0 = smem_desc_nosw(va, 128, 256);
        for (int pg = 0; pg < npages; ++pg) {
          const uint64_t db = db0 + (uint64_t)(pg * (Cfg::kVPageBytes >> 4));
          const uint32_t pa = tmem + t * 128 + (pg < 4 ? pg * 8 : 96 + (pg - 4) * 8);  // see p_col
          if constexpr (PAIR) mma_ts_pair(tmem + 256 + t * 128, pa, db, idesc_pv, !(first && pg == 0));
          else mma_ts(tmem + 256 + t * 128, pa, db, idesc_pv, !(first && pg == 0));
        }
      };
      if (ok) {
        ok = wait_in(&bar_k_ready[0], 0, 302);
        tc_fence_after_sync();
        if (ok) {
          issue_qk(0, 0);
          issue_qk(1, 0);
          if (issuer) commit(&bar_k_empty[0]);
          __syncwarp();
        }
      }
      for (int j = j0; j < j1 && ok; ++j) {
        const int st = (j - j0) % KS, u = (j - j0) / KS;
        const bool self = j >= n_ctx;
        const int npages = self ? kPagesPerTile : min(kPagesPerTile, ctx_pages - j * kPagesPerTile);
        const bool has_next = j + 1 < j1;
        const int st_n = (j + 1 - j0) % KS, u_n = (j + 1 - j0) / KS;
        // V of this tile (staged by the staging warps for new tokens and for fp8 caches)
        if (self || KVF8 != 0) {
          ok = wait_in(&bar_v_ready[st], (v_ready_bits >> st) & 1u, 303);
          v_ready_bits ^= 1u << st;
        } else {
          ok = mbar_wait(&bar_v_tma[st], (uint32_t)u & 1u, p.status, 304);
        }
        if (!ok) break;
        ok = wait_in(&bar_p_full[0], (uint32_t)(j - j0) & 1u, 305);
        if (!ok) break;
        tc_fence_after_sync();
        LA_STAMP(16, j - j0);
        issue_pv(0, st, npages, j == j0);
        if (has_next) {
          ok = wait_in(&bar_k_ready[st_n], (uint32_t)u_n & 1u, 306);
          if (!ok) break;
          tc_fence_after_sync();
          issue_qk(0, st_n);
        }
        LA_STAMP(17, j - j0);
        ok = wait_in(&bar_p_full[1], (uint32_t)(j - j0) & 1u, 307);
        if (!ok) break;
        tc_fence_after_sync();
        LA_STAMP(18, j - j0);
        issue_pv(1, st, npages, j == j0);
        if (issuer) commit(&bar_v_empty[st]);
        if (has_next) {
          issue_qk(1, st_n);
          if (issuer) commit(&bar_k_empty[st_n]);
        }
        LA_STAMP(19, j - j0);
        __syncwarp();
      }
      if (ok && issuer) commit(&bar_o_done);
      __syncwarp();
      }
  } else if (warp > kWarpMma + 1) {
    regs_lower<kRegsIssue>();  // padding warps of the last warpgroup
  } else {
    // =============================== TMA issue ===============================
    regs_lower<kRegsIssue>();
    bool ok = true;
    const int j_end = KVF8 != 0 ? j0 : min(j1, n_ctx);  // fp8 caches are staged with plain loads
    for (int j = j0; j < j_end && ok; ++j) {
      const int st = (j - j0) % KS, u = (j - j0) / KS;
      const int npages = min(kPagesPerTile, ctx_pages - j * kPagesPerTile);
      int coord = 0;
      if (lane < npages) coord = page_block(j * kPagesPerTile + lane) * p.page_ratio + kvh;
      if (u > 0) ok = mbar_wait(&bar_k_empty[st], (uint32_t)(u - 1) & 1u, p.status, 401);
      if (!ok) break;
      if constexpr (PAIR) {
        // K: this CTA's four pages of the tile, counted on its own barrier (its staging warps
        // rotate them before the pair's MMA thread hears of them).
        const int mine = max(0, min(4, npages - 4 * (int)cta_rank));
        const int kcoord = __shfl_sync(0xffffffffu, coord, (lane + 4 * (int)cta_rank) & 31);
        if (lane == 0) mbar_arrive_expect_tx(&bar_k_tma[st], (uint32_t)mine * Cfg::kPageBytes);
        __syncwarp();
        if (lane < mine)
          tma_load_5d(sK + st * Cfg::kKStageBytes + lane * Cfg::kPageBytes, &mapK, &bar_k_tma[st], 0, 0, 0, 0, kcoord);
        if (u > 0) ok = mbar_wait(&bar_v_empty[st], (uint32_t)(u - 1) & 1u, p.status, 402);
        if (!ok) break;
        // V: this CTA's half of the head dimension of every page; both CTAs' copies are
        // counted on the first CTA's barrier, which expects the bytes of both halves.
        if (lane == 0 && cta_rank == 0) mbar_arrive_expect_tx(&bar_v_tma[st], (uint32_t)npages * Cfg::kPageBytes);
        __syncwarp();
        if (lane < npages)
          tma_load_5d_pair(sV + st * Cfg::kVStageBytes + lane * Cfg::kVPageBytes, &mapV,
                           map_to_cta(smem_u32(&bar_v_tma[st]), 0), 0, 0, 0, (int)cta_rank * (D / 16), coord);
        continue;
      }
      if (lane == 0) mbar_arrive_expect_tx(&bar_k_tma[st], (uint32_t)npages * Cfg::kPageBytes);
      __syncwarp();
      if (lane < npages)
        tma_load_5d(sK + st * Cfg::kTileBytes + lane * Cfg::kPageBytes, &mapK, &bar_k_tma[st], 0, 0, 0, 0, coord);
      if (u > 0) ok = mbar_wait(&bar_v_empty[st], (uint32_t)(u - 1) & 1u, p.status, 402);
      if (!ok) break;
      if (lane == 0) mbar_arrive_expect_tx(&bar_v_tma[st], (uint32_t)npages * Cfg::kPageBytes);
      __syncwarp();
      if (lane < npages)
        tma_load_5d(sV + st * Cfg::kTileBytes + lane * Cfg::kPageBytes, &mapV, &bar_v_tma[st], 0, 0, 0, 0, coord);
    }
  }

  // ---- teardown: every role is done (or has given up); release tensor memory
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (PAIR) {
    // neither CTA may leave (its shared memory holds barriers the partner signals and
    // operands the pair's MMAs read) before both are done
    cluster_sync_all();
    if (warp == kWarpMma) tmem_dealloc_pair(tmem, 512);
  } else {
    if (warp == kWarpMma) tmem_dealloc(tmem, 512);
  }
}

template <int D, bool BF16, int KVF8>
__global__ void __launch_bounds__(kThreadsTc, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, TcParams p) {
  prefill_tc_body<D, BF16, KVF8, false>(mapK, mapV, p);
}

// The same kernel run by clusters of two CTAs (consecutive row blocks of one request and KV
// head).  mapV copies half of the head dimension of a page (16-bit caches; fp8 pages are copied by the staging warps).
template <int D, bool BF16, int KVF8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsTc, 1)
prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, TcParams p) {
  prefill_tc_body<D, BF16, KVF8, true>(mapK, mapV, p);
}

// Merge the per-split partial results: out = sum_s 2^(m_s - m*) O_s / sum_s 2^(m_s - m*) l_s.
template <int D, bool BF16>
__global__ void prefill_combine_kernel(TcParams p) {
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int s0 = p.qsl[b];
  const int qlen = p.qsl[b + 1] - s0;
  if (qlen <= 0 || (p.skip_decode && qlen == 1)) return;
  const int nrows = qlen * p.G;
  constexpr int kRowsPerBlock = 256 / (D / 4);
  const int R = blockIdx.x * kRowsPerBlock + threadIdx.x / (D / 4);
  const int d0 = (threadIdx.x % (D / 4)) * 4;
  if (R >= nrows) return;
  const int64_t slot0 = (((int64_t)b * p.Hkv + kvh) * p.rows_cap + R) * p.n_splits;
  float m_star = -INFINITY;
  for (int s = 0; s < p.n_splits; ++s) m_star = fmaxf(m_star, p.part_ml[(slot0 + s) * 2]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
  for (int s = 0; s < p.n_splits; ++s) {
    const float m = p.part_ml[(slot0 + s) * 2];
    if (m == -INFINITY) continue;
    const float w = exp2f(m - m_star);
    l += w * p.part_ml[(slot0 + s) * 2 + 1];
    const float4 o = *reinterpret_cast<const float4*>(p.part_o + (slot0 + s) * D + d0);
    acc[0] += w * o.x; acc[1] += w * o.y; acc[2] += w * o.z; acc[3] += w * o.w;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const int tq = R >> p.g_shift, head = kvh * p.G + (R & (p.G - 1));
  uint2 w2;
  w2.x = pack2<BF16>(acc[0] * inv, acc[1] * inv);
  w2.y = pack2<BF16>(acc[2] * inv, acc[3] * inv);
  if (p.peer.num_peers == 0) {
    uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + ((int64_t)(s0 + tq) * p.o_st + (int64_t)head * p.o_sh) * 2;
    *reinterpret_cast<uint2*>(orow + d0 * 2) = w2;
  } else {
    const int64_t prow = p.peer.rows ? p.peer.rows[s0 + tq] : (s0 + tq);
    const int64_t off = (prow * p.peer.stride_t + (int64_t)(p.peer.head_offset + head) * p.peer.stride_h + d0) * 2;
    for (int q = 0; q < p.peer.num_peers; ++q)
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(p.peer.out[q]) + off) = w2;
  }
}

// ---- host side ---------------------------------------------------------------------------
struct MapKey {
  const void* kc;
  const void* vc;
  int64_t nb, ksb, ksh, vsb, vsh;
  int D, dt, half_v;
  bool operator==(const MapKey& o) const {
    return kc == o.kc && vc == o.vc && nb == o.nb && ksb == o.ksb && ksh == o.ksh && vsb == o.vsb &&
           vsh == o.vsh && D == o.D && dt == o.dt && half_v == o.half_v;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.kc) ^ (std::hash<const void*>()(k.vc) << 1);
    h ^= std::hash<int64_t>()(k.nb * 131 + k.ksb * 17 + k.ksh + k.D * 7 + k.dt + k.half_v * 3);
    return h;
  }
};
struct MapPair {
  CUtensorMap k, v;
};
std::mutex g_map_mu;
std::unordered_map<MapKey, MapPair, MapKeyHash> g_maps;

// The two tensor maps of a 16-bit cache: one page of one head per box, laid out
// for the no-swizzle operand layout (see the head of this file).  half_v: the V box covers
// half of the head dimension (the kernel run by CTA pairs, where each CTA keeps one half).
int encode_maps(const LaPrefillArgs& a, bool half_v, MapPair* mp) {
  EncodeTiledFn enc = get_encode_tiled();
  LA_REQUIRE(enc != nullptr, LA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int D = a.head_dim;
  const cuuint64_t n_idx = (cuuint64_t)a.num_blocks * (cuuint64_t)(a.kc_stride_block / a.kc_stride_head);
  const CUtensorMapDataType dt =
      a.q_dtype == LA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint32_t es[5] = {1, 1, 1, 1, 1};
  {
    // K page of one head: [D/8][16 tokens][8 elements]; dims innermost first:
    // 8 elements, 8 tokens, D/8 groups, 2 token halves, (page, head)
    cuuint64_t dim[5] = {8, 8, (cuuint64_t)D / 8, 2, n_idx};
    cuuint64_t str[4] = {16, 256, 128, (cuuint64_t)a.kc_stride_head * 2};
    cuuint32_t box[5] = {8, 8, (cuuint32_t)D / 8, 2, 1};
    CUresult r = enc(&mp->k, dt, 5, const_cast<void*>(a.k_cache), dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LA_REQUIRE(r == CUDA_SUCCESS, LA_ERR_CUDA, "cuTensorMapEncodeTiled(K cache) failed with %d", (int)r);
  }
  {
    // V page of one head: [D][16 tokens]; dims innermost first:
    // 8 tokens, 8 dims, 2 token halves, D/8 dim groups, (page, head)
    cuuint64_t dim[5] = {8, 8, 2, (cuuint64_t)D / 8, n_idx};
    cuuint64_t str[4] = {32, 16, 256, (cuuint64_t)a.vc_stride_head * 2};
    cuuint32_t box[5] = {8, 8, 2, (cuuint32_t)D / (half_v ? 16 : 8), 1};
    CUresult r = enc(&mp->v, dt, 5, const_cast<void*>(a.v_cache), dim, str, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LA_REQUIRE(r == CUDA_SUCCESS, LA_ERR_CUDA, "cuTensorMapEncodeTiled(V cache) failed with %d", (int)r);
  }
  return LA_OK;
}

// Tensor maps of a cache, remembered per (pointers, shape).  A layer is called again and
// again with the same caches: the calling thread's last pair is checked first, without
// taking the lock of the shared table.
int cached_maps(const LaPrefillArgs& a, bool half_v, MapPair* out) {
  MapKey key{a.k_cache, a.v_cache, a.num_blocks, a.kc_stride_block, a.kc_stride_head,
             a.vc_stride_block, a.vc_stride_head, a.head_dim, a.q_dtype, half_v ? 1 : 0};
  thread_local MapKey last_key{};
  thread_local MapPair last_pair;
  thread_local bool have_last = false;
  if (have_last && last_key == key) {
    *out = last_pair;
    return LA_OK;
  }
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
      MapPair mp;
      int rc = encode_maps(a, half_v, &mp);
      if (rc != LA_OK) return rc;
      if (g_maps.size() > 4096) g_maps.clear();
      it = g_maps.emplace(key, mp).first;
    }
    *out = it->second;
  }
  last_key = key;
  last_pair = *out;
  have_last = true;
  return LA_OK;
}

int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

struct TcPlan {
  int mblocks, n_splits;
  bool pair;             // run by clusters of two CTAs (consecutive row blocks)
  int64_t rows_cap;
  size_t scratch_bytes;  // split-KV partials (0 when the KV range is not split)
};

TcPlan make_plan(const LaPrefillArgs& a) {
  const int G = a.num_q_heads / a.num_kv_heads;
  TcPlan pl;
  pl.mblocks = (int)(((int64_t)a.max_query_len * G + kRowsPerCta - 1) / kRowsPerCta);
  // CTA pairs: at least two row blocks per (request, KV head), so that a pair is not half
  // empty by construction.
  pl.pair = pl.mblocks >= 2;
  if (const char* e = getenv("LAZY_ATTN_B200_PREFILL_PAIR")) {  // experiments only
    if (e[0] == '0') pl.pair = false;
    if (e[0] == '1') pl.pair = true;
  }
  if (pl.pair) pl.mblocks = (pl.mblocks + 1) & ~1;
  pl.rows_cap = (int64_t)pl.mblocks * kRowsPerCta;
  // Split the KV range when the row blocks alone cannot fill the GPU.  The sequence
  // lengths live on the device, so the plan uses the caller's maxima.  Cost of a split
  // count s, in units of one tile step of a CTA: the grid runs in waves over the SMs (one
  // CTA, or half a pair, per SM); a CTA costs its tiles plus a fixed part (staging Q, the
  // first tile's latency, reading the accumulator out: about six tile steps); the merge
  // kernel streams s partial rows per output row.  The constants come from sweeps of the
  // split count on the 8B configuration at 1/1, 1/2, 1/4 and 1/8 of its heads, whose
  // measured order this model reproduces.
  const int64_t ctas = (int64_t)pl.mblocks * a.num_kv_heads * a.batch;
  int64_t max_seq = a.max_seq_len > 0 ? a.max_seq_len : 0;
  const int64_t tiles = (max_seq + kTileN - 1) / kTileN + 1;
  const int64_t units = pl.pair ? ctas / 2 : ctas;
  const int64_t slots = pl.pair ? 74 : 148;
  const double merge_per_split = 2.8 * (double)(pl.rows_cap * a.num_kv_heads * a.batch) / 16384.0;
  int best = 1;
  double best_cost = 0.0;
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && tiles / s < 4) break;
    const int64_t waves = (units * s + slots - 1) / slots;
    const double cost = (double)waves * (double)((tiles + s - 1) / s + 6) + (s > 1 ? merge_per_split * s : 0.0);
    if (s == 1 || cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  pl.n_splits = best;
  if (const char* e = getenv("LAZY_ATTN_B200_PREFILL_SPLITS")) {  // experiments only
    const int v = atoi(e);
    if (v >= 1 && v <= 16) pl.n_splits = v;
  }
  pl.scratch_bytes = 0;
  if (pl.n_splits > 1) {
    const size_t slots = (size_t)a.batch * a.num_kv_heads * pl.rows_cap * pl.n_splits;
    pl.scratch_bytes = slots * (a.head_dim + 2) * sizeof(float) + 256;
  }
  return pl;
}

}  // namespace

bool tc_prefill_supported(const LaPrefillArgs& a, const char** why) {
  const int G = a.num_kv_heads > 0 ? a.num_q_heads / a.num_kv_heads : 0;
  if (a.q_dtype != LA_DTYPE_BF16 && a.q_dtype != LA_DTYPE_F16) { *why = "activations must be bf16 or fp16"; return false; }
  if (a.kv_dtype != a.q_dtype && a.kv_dtype != LA_DTYPE_FP8_E4M3 && a.kv_dtype != LA_DTYPE_FP8_E5M2) { *why = "cache dtype must be the activation dtype or fp8"; return false; }
  if (a.head_dim != 64 && a.head_dim != 128) { *why = "head_dim must be 64 or 128"; return false; }
  if (a.block_size != 16) { *why = "block_size must be 16"; return false; }
  if (G < 1 || G > 128 || (G & (G - 1)) != 0) { *why = "query heads per KV head must be a power of two"; return false; }
  if (a.sliding_window > 0) { *why = "sliding window"; return false; }
  if (a.cos_sin_cache != nullptr && a.cos_sin_dtype != a.q_dtype) { *why = "cos/sin table dtype must equal the activation dtype"; return false; }
  if (a.kc_stride_head != (int64_t)a.head_dim * 16 || a.vc_stride_head != (int64_t)a.head_dim * 16) { *why = "cache heads must be densely packed"; return false; }
  if (a.kc_stride_block % a.kc_stride_head != 0 || a.kc_stride_block != a.vc_stride_block) { *why = "cache block stride"; return false; }
  if (a.q_stride_t % 8 || a.q_stride_h % 8 || a.k_stride_t % 8 || a.k_stride_h % 8 || a.v_stride_t % 8 ||
      a.v_stride_h % 8 || a.o_stride_t % 8 || a.o_stride_h % 8) { *why = "activation strides must be multiples of 8 elements"; return false; }
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
       reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.k_cache) |
       reinterpret_cast<uintptr_t>(a.v_cache) | reinterpret_cast<uintptr_t>(a.cos_sin_cache)) & 15) { *why = "pointers must be 16-byte aligned"; return false; }
  if (a.num_blocks <= 0) { *why = "num_blocks not given"; return false; }
  if (a.q_positions != nullptr && a.cos_sin_cache == nullptr) { *why = "the fused rotary op needs the cos/sin table"; return false; }
  if (a.peer.num_peers < 0 || a.peer.num_peers > LA_MAX_PEERS) { *why = "peer count out of range"; return false; }
  for (int q = 0; q < a.peer.num_peers; ++q)
    if (a.peer.out[q] == nullptr || (reinterpret_cast<uintptr_t>(a.peer.out[q]) & 15)) { *why = "peer output pointers must be non-null and 16-byte aligned"; return false; }
  if (a.peer.num_peers > 0 && (a.peer.stride_t % 8 || a.peer.stride_h % 8 || a.peer.head_offset < 0)) { *why = "peer output strides must be multiples of 8 elements"; return false; }
  return true;
}

size_t tc_prefill_workspace_bytes(const LaPrefillArgs& a) { return make_plan(a).scratch_bytes; }

namespace {

// The per-role register budgets assume the registers per thread the kernel is launched with; a build
// that came out with fewer would leave the softmax warps waiting for registers nobody can release.
int check_launch_registers(const void* kern) {
  cudaFuncAttributes attr;
  LA_CHECK_CUDA(cudaFuncGetAttributes(&attr, kern));
  LA_REQUIRE(attr.numRegs == kLaunchRegs, LA_ERR_UNSUPPORTED,
             "prefill kernel was built with %d registers per thread, its register budgets need %d", attr.numRegs,
             kLaunchRegs);
  return LA_OK;
}

template <int D, bool BF16, int KVF8>
int launch_tc_kv(const LaPrefillArgs& a, const TcParams& p, const MapPair& mp, const TcPlan& pl,
                  cudaStream_t stream) {
  using Cfg = TcCfg<D>;
  auto kern = prefill_tc_kernel<D, BF16, KVF8>;
  // the attribute is per device: remember on which devices this kernel has been prepared
  static std::atomic<uint64_t> prepared{0};
  int dev = 0;
  LA_CHECK_CUDA(cudaGetDevice(&dev));
  if (((prepared.load(std::memory_order_acquire) >> (dev & 63)) & 1ull) == 0) {
    LA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (const int rc = check_launch_registers(reinterpret_cast<const void*>(kern)); rc != LA_OK) return rc;
    prepared.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  dim3 grid(pl.mblocks, a.num_kv_heads, a.batch * pl.n_splits);
  kern<<<grid, kThreadsTc, Cfg::kSmemBytes, stream>>>(mp.k, mp.v, p);
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  if (pl.n_splits > 1) {
    constexpr int kRowsPerBlock = 256 / (D / 4);
    dim3 cgrid((unsigned)((pl.rows_cap + kRowsPerBlock - 1) / kRowsPerBlock), a.num_kv_heads, a.batch);
    prefill_combine_kernel<D, BF16><<<cgrid, 256, 0, stream>>>(p);
    count_launch();
    LA_CHECK_CUDA(cudaGetLastError());
  }
  return LA_OK;
}

template <int D, bool BF16, int KVF8>
int launch_tc_pair(const LaPrefillArgs& a, const TcParams& p, const MapPair& mp, const TcPlan& pl,
                   cudaStream_t stream) {
  using Cfg = TcCfg<D, true>;
  auto kern = prefill_tc_pair_kernel<D, BF16, KVF8>;
  static std::atomic<uint64_t> prepared{0};
  int dev = 0;
  LA_CHECK_CUDA(cudaGetDevice(&dev));
  if (((prepared.load(std::memory_order_acquire) >> (dev & 63)) & 1ull) == 0) {
    LA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (const int rc = check_launch_registers(reinterpret_cast<const void*>(kern)); rc != LA_OK) return rc;
    prepared.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  dim3 grid(pl.mblocks, a.num_kv_heads, a.batch * pl.n_splits);  // x is even: clusters of (2, 1, 1)
  kern<<<grid, kThreadsTc, Cfg::kSmemBytes, stream>>>(mp.k, mp.v, p);
  count_launch();
  LA_CHECK_CUDA(cudaGetLastError());
  if (pl.n_splits > 1) {
    constexpr int kRowsPerBlock = 256 / (D / 4);
    dim3 cgrid((unsigned)((pl.rows_cap + kRowsPerBlock - 1) / kRowsPerBlock), a.num_kv_heads, a.batch);
    prefill_combine_kernel<D, BF16><<<cgrid, 256, 0, stream>>>(p);
    count_launch();
    LA_CHECK_CUDA(cudaGetLastError());
  }
  return LA_OK;
}

template <int D, bool BF16>
int launch_tc(const LaPrefillArgs& a, const TcParams& p, const MapPair& mp, const TcPlan& pl, cudaStream_t stream) {
  if (pl.pair) {
    if (a.kv_dtype == LA_DTYPE_FP8_E4M3) return launch_tc_pair<D, BF16, 1>(a, p, mp, pl, stream);
    if (a.kv_dtype == LA_DTYPE_FP8_E5M2) return launch_tc_pair<D, BF16, 2>(a, p, mp, pl, stream);
    return launch_tc_pair<D, BF16, 0>(a, p, mp, pl, stream);
  }
  if (a.kv_dtype == LA_DTYPE_FP8_E4M3) return launch_tc_kv<D, BF16, 1>(a, p, mp, pl, stream);
  if (a.kv_dtype == LA_DTYPE_FP8_E5M2) return launch_tc_kv<D, BF16, 2>(a, p, mp, pl, stream);
  return launch_tc_kv<D, BF16, 0>(a, p, mp, pl, stream);
}

// The one launch path of the tensor-core kernel.  `scratch` holds the split-KV partials
// (the caller's workspace, or the library's built-in array for the allocation-free entry
// point); `keep_maps` says whether the tensor maps may be remembered between calls.
int launch_tc_with_scratch(const LaPrefillArgs& a, cudaStream_t stream, void* scratch, size_t scratch_bytes,
                           bool keep_maps, const char* who) {
  const TcPlan pl = make_plan(a);
  LA_REQUIRE((int64_t)a.batch * pl.n_splits <= 65535 && a.num_kv_heads <= 65535, LA_ERR_UNSUPPORTED,
             "%s: %d requests x %d splits (at most 65535) or %d KV heads (at most 65535) exceed the launch grid",
             who, a.batch, pl.n_splits, a.num_kv_heads);
  // The scratch is checked before anything touches the device, so that a caller who
  // forgot the workspace learns the size from the error text.
  LA_REQUIRE(pl.scratch_bytes == 0 || (scratch != nullptr && scratch_bytes >= pl.scratch_bytes), LA_ERR_WORKSPACE,
             "%s: this call splits the KV range %d ways and needs %zu bytes of scratch, %zu were given", who,
             pl.n_splits, pl.scratch_bytes, scratch ? scratch_bytes : (size_t)0);
  MapPair mp;
  TcParams p{};
  std::memset(&mp, 0, sizeof(mp));
  if (a.kv_dtype == a.q_dtype) {
    // 16-bit caches are read through tensor maps
    int rc = keep_maps ? cached_maps(a, pl.pair, &mp) : encode_maps(a, pl.pair, &mp);
    if (rc != LA_OK) return rc;
  } else {
    // fp8 caches are read with plain loads by the staging warps
    p.kc = reinterpret_cast<const uint8_t*>(a.k_cache);
    p.vc = reinterpret_cast<const uint8_t*>(a.v_cache);
    p.kc_sb = a.kc_stride_block; p.kc_sh = a.kc_stride_head;
    p.vc_sb = a.vc_stride_block; p.vc_sh = a.vc_stride_head;
    p.num_blocks = a.num_blocks;
    p.k_scale = a.k_scale; p.v_scale = a.v_scale;
  }
  p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out;
  p.q_st = a.q_stride_t; p.q_sh = a.q_stride_h;
  p.k_st = a.k_stride_t; p.k_sh = a.k_stride_h;
  p.v_st = a.v_stride_t; p.v_sh = a.v_stride_h;
  p.o_st = a.o_stride_t; p.o_sh = a.o_stride_h;
  p.block_table = a.block_table; p.q_offset = a.q_offset; p.q_mask = a.q_mask;
  p.table_stride = a.table_stride;
  p.packed = a.packed_block_table; p.packed_stride = a.packed_stride;
  p.slots = a.slot_mapping;
  p.q_pos = a.q_positions;
  {
    const int64_t e = a.kv_dtype == a.q_dtype ? 2 : 1;  // bytes per cache element
    p.kcw = reinterpret_cast<uint8_t*>(const_cast<void*>(a.k_cache));
    p.vcw = reinterpret_cast<uint8_t*>(const_cast<void*>(a.v_cache));
    p.kcw_sb = a.kc_stride_block * e; p.kcw_sh = a.kc_stride_head * e;
    p.vcw_sb = a.vc_stride_block * e; p.vcw_sh = a.vc_stride_head * e;
    if (a.slot_mapping != nullptr) { p.k_scale = a.k_scale; p.v_scale = a.v_scale; }
  }
  p.qsl = a.query_start_loc; p.seq_lens = a.seq_lens; p.is_lazy = a.is_lazy;
  p.cs = a.cos_sin_cache; p.cs_rows = a.cos_sin_rows;
  p.Hq = a.num_q_heads; p.Hkv = a.num_kv_heads; p.G = a.num_q_heads / a.num_kv_heads;
  p.g_shift = ilog2(p.G);
  p.rot_mode = a.rot_mode; p.is_mepic = a.is_mepic; p.skip_decode = a.skip_decode;
  p.n_splits = pl.n_splits;
  p.page_ratio = (int)(a.kc_stride_block / a.kc_stride_head);
  p.scale_log2 = a.sm_scale * 1.4426950408889634f;
  p.peer = a.peer;
  p.rows_cap = pl.rows_cap;
  if (pl.n_splits > 1) {
    // Every slot the merge kernel reads is written by the attention kernel of the same
    // call (empty splits write a neutral entry): the scratch never needs clearing.
    const size_t slots = (size_t)a.batch * a.num_kv_heads * pl.rows_cap * pl.n_splits;
    uintptr_t base = (reinterpret_cast<uintptr_t>(scratch) + 255) & ~uintptr_t(255);
    p.part_o = reinterpret_cast<float*>(base);
    p.part_ml = p.part_o + slots * a.head_dim;
  }
  p.status = device_status_ptr();
  LA_REQUIRE(p.status != nullptr, LA_ERR_CUDA, "%s: device status word unavailable", who);
  const bool bf16 = a.q_dtype == LA_DTYPE_BF16;
  if (a.head_dim == 128) return bf16 ? launch_tc<128, true>(a, p, mp, pl, stream) : launch_tc<128, false>(a, p, mp, pl, stream);
  return bf16 ? launch_tc<64, true>(a, p, mp, pl, stream) : launch_tc<64, false>(a, p, mp, pl, stream);
}

}  // namespace

int launch_tc_prefill(const LaPrefillArgs& a, cudaStream_t stream) {
  return launch_tc_with_scratch(a, stream, a.workspace, a.workspace_bytes, true, "la_prefill_fwd");
}

}  // namespace la

// ---- allocation-free entry point ---------------------------------------------------------
namespace la {
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(32) << 20;  // 32 MiB per GPU that loads the library
constexpr int kMaxDevices = 64;

// Split-KV scratch that lives in the library image instead of in memory the
// caller (or the Python layer) allocates.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_noalloc_mu;
void* g_noalloc_addr[kMaxDevices] = {nullptr};

// Device address of the scratch on the current device.  In host code the array's
// name is only a handle: the address a kernel can use comes from the runtime.
int noalloc_scratch(void** out) {
  int dev = -1;
  LA_CHECK_CUDA(cudaGetDevice(&dev));
  LA_REQUIRE(dev >= 0 && dev < kMaxDevices, LA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_addr[dev] == nullptr) {
    void* ptr = nullptr;
    LA_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    LA_REQUIRE(ptr != nullptr, LA_ERR_CUDA, "built-in scratch has no device address");
    g_noalloc_addr[dev] = ptr;
  }
  *out = g_noalloc_addr[dev];
  return LA_OK;
}

}  // namespace
}  // namespace la

extern "C" int la_prefill_fwd_noalloc(const LaPrefillArgs* args, void* stream) {
  using namespace la;
  int rc = validate_prefill_args(args);
  if (rc != LA_OK) return rc;
  if (args->batch == 0 || args->max_query_len <= 0) return LA_OK;
  const char* why = "";
  LA_REQUIRE(tc_prefill_supported(*args, &why), LA_ERR_UNSUPPORTED,
             "la_prefill_fwd_noalloc: arguments outside the tensor-core kernel: %s", why);
  const size_t need = tc_prefill_workspace_bytes(*args);
  LA_REQUIRE(need <= kNoAllocScratchBytes, LA_ERR_WORKSPACE,
             "la_prefill_fwd_noalloc: this call needs %zu bytes of split-KV scratch, the built-in scratch holds "
             "%zu; use la_prefill_fwd with a caller-provided workspace",
             need, kNoAllocScratchBytes);
  void* scratch = nullptr;
  rc = noalloc_scratch(&scratch);
  if (rc != LA_OK) return rc;
  // the tensor maps are encoded into this call's own storage (the shared table of
  // remembered maps may grow, i.e. allocate host memory)
  return launch_tc_with_scratch(*args, (cudaStream_t)stream, scratch, kNoAllocScratchBytes, false,
                                "la_prefill_fwd_noalloc");
}

#ifdef LA_TRACE
// Copies the timeline of the last traced launch to the host (tuning builds only).
extern "C" int la_trace_read(long long* out) {
  LA_CHECK_CUDA(cudaDeviceSynchronize());
  LA_CHECK_CUDA(cudaMemcpyFromSymbol(out, la::g_trace, sizeof(long long) * la::kTraceRows * la::kTraceCols));
  return LA_OK;
}
#endif
