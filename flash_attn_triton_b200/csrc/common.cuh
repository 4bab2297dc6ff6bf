// Shared device/host helpers for the sm_100a attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fa_b200.h"

#define FA_LOG2E 1.4426950408889634f
#define FA_LN2 0.6931471805599453f

namespace fa {

// ---------------------------------------------------------------------------------------
// error plumbing (host)
// ---------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int check_launch(const char* what);
int ensure_device(int device);
int sm_count(int device);
// Counter pair for one launch of a persistent kernel (work queue: [0] next candidate, [1] CTAs
// finished; both zero between launches).  Pairs come from a fixed array inside the library and
// are handed out in rotation, so launches that overlap on the GPU use different pairs as long as
// fewer than kWorkQueues of them are in flight on one device.  Null (with the error set) on failure.
// Time-outs of bounded device-side waits.  host_wait_word(): the word (in mapped host memory, as
// a device-visible pointer; null when the mapping is unavailable) that a kernel of `device` sets
// when one of its waits runs out.  host_wait_status(): its current value, read without touching
// the GPU; the tcgen05 launchers refuse to launch while it is non-zero.
int* host_wait_word(int device);
int host_wait_status(int device);
constexpr int kWorkQueues = 64;
unsigned int* work_queue(int device);  // streaming multiprocessors of `device` (the persistent kernels launch one CTA each)

#define FA_REQUIRE(cond, ...)      \
  do {                             \
    if (!(cond)) {                 \
      fa::set_error(__VA_ARGS__);  \
      return FA_ERR_INVALID;       \
    }                              \
  } while (0)

// ---------------------------------------------------------------------------------------
// Score pipeline shared by every kernel.  All fields are per launch except `slope`,
// which kernels fetch per (batch, head).
// ---------------------------------------------------------------------------------------
struct ScoreCfg {
  float scale;        // softmax_scale
  float scale_log2;   // softmax_scale * log2(e)
  float softcap;      // 0 = off
  float inv_softcap;  // 1/softcap
  int causal;
  int wl, wr;         // window; -1 = open
  int has_alibi;
  // taken by the mma.sync kernels only
  const float* bias;        // additive fp32 bias or null; element (b, h, row, col) through bias_stride
  int64_t bias_stride[4];
  float dropout_p;          // 0 = off
  float dropout_scale;      // 1 / (1 - p)
  uint32_t seed_lo, seed_hi;
  uint32_t drop_stride;     // counter of element (row, col) = (row0 + row) * drop_stride + col
};

__host__ __device__ inline ScoreCfg make_score_cfg(float scale, float softcap, int causal, int wl,
                                                   int wr, bool alibi) {
  ScoreCfg c;
  c.scale = scale;
  c.scale_log2 = scale * FA_LOG2E;
  c.softcap = softcap;
  c.inv_softcap = softcap > 0.f ? 1.f / softcap : 0.f;
  c.causal = causal;
  c.wl = wl;
  c.wr = wr;
  c.has_alibi = alibi ? 1 : 0;
  c.bias = nullptr;
  c.bias_stride[0] = c.bias_stride[1] = c.bias_stride[2] = c.bias_stride[3] = 0;
  c.dropout_p = 0.f;
  c.dropout_scale = 1.f;
  c.seed_lo = c.seed_hi = c.drop_stride = 0u;
  return c;
}

// Philox4x32-10 (Salmon et al.) with key (k0, k1) and counter (c0, 0, 0, 0); first output word.
// This is the generator behind the reference's tl.rand(seed, offset): key = the 64-bit seed,
// c0 = the element's offset.
__host__ __device__ inline uint32_t philox_first(uint32_t c0, uint32_t k0, uint32_t k1) {
  uint32_t c1 = 0u, c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t pa = (uint64_t)0xD2511F53u * c0, pb = (uint64_t)0xCD9E8D57u * c2;
    c0 = (uint32_t)(pb >> 32) ^ c1 ^ k0;
    c2 = (uint32_t)(pa >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)pb;
    c3 = (uint32_t)pa;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}
// The 32 random bits as a float in [0, 1): the signed value folded to non-negative, times 2^-31.
__host__ __device__ inline float uniform_from_bits(uint32_t bits) {
  int32_t x = (int32_t)bits;
  if (x < 0) x = -x - 1;
  return (float)x * 4.6566127342e-10f;
}
// Dropout keep test of element (row, col) of a sequence whose first packed row is row0.
__device__ __forceinline__ bool dropout_keep(const ScoreCfg& c, uint32_t row0, int row, int col) {
  const uint32_t offset = (row0 + (uint32_t)row) * c.drop_stride + (uint32_t)col;
  return uniform_from_bits(philox_first(offset, c.seed_lo, c.seed_hi)) > c.dropout_p;
}
__device__ __forceinline__ float bias_at(const ScoreCfg& c, int b, int h, int row, int col) {
  return c.bias[(int64_t)b * c.bias_stride[0] + (int64_t)h * c.bias_stride[1] + (int64_t)row * c.bias_stride[2] +
                (int64_t)col * c.bias_stride[3]];
}

// ex2.approx without the denormal handling exp2f() adds
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32 pairs (one issue slot for two results) and the three-input maximum of sm_100.
// The element-wise warps of the tcgen05 kernels are short of issue slots, not of FP32 lanes.
__device__ __forceinline__ uint64_t f2_pack(float x, float y) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ float2 f2_unpack(uint64_t r) {
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(r));
  return d;
}
__device__ __forceinline__ float2 f2fma(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(f2_pack(a.x, a.y)), "l"(f2_pack(b.x, b.y)), "l"(f2_pack(c.x, c.y)));
  return f2_unpack(d);
}
__device__ __forceinline__ float2 f2add(float2 a, float2 b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(f2_pack(a.x, a.y)), "l"(f2_pack(b.x, b.y)));
  return f2_unpack(d);
}
__device__ __forceinline__ float2 f2mul(float2 a, float2 b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(f2_pack(a.x, a.y)), "l"(f2_pack(b.x, b.y)));
  return f2_unpack(d);
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x of a pair on the FMA pipe instead of the special-function unit (16 results per clock per
// SM, as scarce as the tensor cores in these kernels): round-to-nearest split x = n + f with
// f in [-0.5, 0.5], a degree-3 minimax polynomial for 2^f (relative error 1.0e-4, below the
// rounding of the 16-bit probabilities it feeds), n added into the exponent field; packed fp32,
// about 5.5 issue slots per result.  Arguments below -125 return 2^-125 rather than 0, so masked
// (-inf) scores must not come here.  Measured: a loss wherever the caller keeps a whole row of
// scores in registers (the polynomial wants ~10 more per pair in flight); a gain of 3-8 % in the
// persistent forward on long items once the exp2 pass re-reads its scores from tensor memory in
// chunks (fwd_persist_sm100.cu, kPoly).  The backward kernels keep kEvery = 0.
__device__ __forceinline__ float2 ex2_fma2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 magic = make_float2(12582912.f, 12582912.f), nmagic = make_float2(-12582912.f, -12582912.f);
  const float2 t = f2add(x, magic);
  const float2 n = f2add(t, nmagic);
  const float2 f = f2fma(n, make_float2(-1.f, -1.f), x);
  float2 p = f2fma(make_float2(0.05500862f, 0.05500862f), f, make_float2(0.24221021f, 0.24221021f));
  p = f2fma(p, f, make_float2(0.6932829f, 0.6932829f));
  p = f2fma(p, f, make_float2(1.f, 1.f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}
// Every kEvery-th PAIR (index pair) of an unrolled loop goes to ex2_fma2 (0 = none).
template <int kEvery> __device__ __forceinline__ float2 ex2_pair(float2 a, int pair) {
  if (kEvery > 0 && (pair % (kEvery > 0 ? kEvery : 1)) == (kEvery > 0 ? kEvery : 1) - 1) return ex2_fma2(a);
  return make_float2(ex2(a.x), ex2(a.y));
}

// tanh through one exp2 and one reciprocal: 1 - 2/(exp(2x)+1); saturates cleanly to +-1.
__device__ __forceinline__ float fast_tanh(float x) {
  const float e = ex2(x * (2.f * FA_LOG2E));
  return 1.f - __fdividef(2.f, e + 1.f);
}

// Raw dot product -> score in the log2 domain (unmasked).  `dist` = q position - key position
// as a float (exact: positions are far below 2^24; the tcgen05 kernels derive it from one
// conversion per tile instead of one per element).  `th` returns tanh(s/softcap) when softcap
// is on (needed by the backward), else 0.
__device__ __forceinline__ float score_log2_dist(const ScoreCfg& c, float slope, float dot, float dist,
                                                 float& th, float bias = 0.f) {
  th = 0.f;
  if (!c.has_alibi && c.softcap == 0.f && c.bias == nullptr) return dot * c.scale_log2;
  float s = dot * c.scale;
  if (c.has_alibi) s = fmaf(-slope, fabsf(dist), s);
  s += bias;                                   // after ALiBi, before the soft cap
  if (c.softcap > 0.f) {
    th = fast_tanh(s * c.inv_softcap);
    s = c.softcap * th;
  }
  return s * FA_LOG2E;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The same for the kernels that are compiled per feature set: ALiBi always applied (a zero slope
// leaves the score unchanged, exactly), the soft cap selected at compile time.  Written so that
// everything that does not depend on the element is a loop-invariant product the compiler hoists:
//   no cap:  dot * scale_log2 - (slope log2e) |dist|                               2 instructions
//   cap:     tanh = tanh.approx((dot * scale - slope |dist|) / cap)                1 + 1 MUFU,
//            score = cap log2e * tanh, which the caller folds into the FMA that forms the exp2
//            argument (soft_cap_factor()).
// tanh.approx.f32 has a relative error of 2^-11, the rounding of the 16-bit probabilities the
// score ends up in; against an fp32 computation the outputs and gradients of the packed feature tests
// moved by less than their last digit when it replaced 1 - 2 / (2^u + 1) (two MUFU results and
// three more instructions per score: the element-wise warps of these variants are MUFU-bound).
template <bool kCap>
__device__ __forceinline__ float score_unit_feat(const ScoreCfg& c, float slope, float dot, float dist, float& th) {
  if (!kCap) {
    th = 0.f;
    return fmaf(-(slope * FA_LOG2E), fabsf(dist), dot * c.scale_log2);
  }
  th = tanh_approx(fmaf(-(slope * c.inv_softcap), fabsf(dist), dot * (c.scale * c.inv_softcap)));
  return th;
}
// The same for a pair of scores with packed arithmetic (half the instructions: the unrolled score
// loops of the feature variants are what the instruction cache has to hold).  d2 = the pair's
// (query position - key position); kAbs = false where every visible element has d >= 0 (causal).
struct FeatK {
  float2 ka, kb;
};
template <bool kCap> __device__ __forceinline__ FeatK feat_k(const ScoreCfg& c, float slope) {
  const float ka = kCap ? -(slope * c.inv_softcap) : -(slope * FA_LOG2E);
  const float kb = kCap ? c.scale * c.inv_softcap : c.scale_log2;
  FeatK k;
  k.ka = make_float2(ka, ka);
  k.kb = make_float2(kb, kb);
  return k;
}
template <bool kCap, bool kAbs>
__device__ __forceinline__ float2 score_unit_feat2(const FeatK& k, float2 dot2, float2 d2) {
  if (kAbs) {
    d2.x = fabsf(d2.x);
    d2.y = fabsf(d2.y);
  }
  const float2 y = f2fma(k.ka, d2, f2mul(dot2, k.kb));
  if (!kCap) return y;
  return make_float2(tanh_approx(y.x), tanh_approx(y.y));
}
// score in the log2 domain = score_unit_feat() * soft_cap_factor()
template <bool kCap> __device__ __forceinline__ float soft_cap_factor(const ScoreCfg& c) {
  return kCap ? c.softcap * FA_LOG2E : 1.f;
}
// score in the log2 domain + addend (the negated row maximum or LSE), one FMA after the unit score
template <bool kCap>
__device__ __forceinline__ float score_log2_feat_add(const ScoreCfg& c, float slope, float dot, float dist,
                                                     float addend, float& th) {
  if (!kCap) {
    th = 0.f;
    return fmaf(-(slope * FA_LOG2E), fabsf(dist), fmaf(dot, c.scale_log2, addend));
  }
  return fmaf(score_unit_feat<true>(c, slope, dot, dist, th), c.softcap * FA_LOG2E, addend);
}
__device__ __forceinline__ float score_log2(const ScoreCfg& c, float slope, float dot, int qpos,
                                            int kpos, float& th, float bias = 0.f) {
  return score_log2_dist(c, slope, dot, (float)(qpos - kpos), th, bias);
}

__device__ __forceinline__ bool visible(const ScoreCfg& c, int qpos, int kpos, int k_len) {
  bool ok = kpos < k_len;
  if (c.causal) ok = ok && (kpos <= qpos);
  if (c.wl >= 0) ok = ok && (kpos >= qpos - c.wl);
  if (c.wr >= 0) ok = ok && (kpos <= qpos + c.wr);
  return ok;
}

// The mask as intervals.  For one key the query positions that see it, and for one query the
// key positions it sees, are contiguous: a per-element test inside an unrolled loop is then two
// integer instructions and a select instead of a chain of short-circuit branches (which the
// compiler turns into divergent control flow: measured at more than 200 cycles per element).
__device__ __forceinline__ void visible_q_interval(const ScoreCfg& c, int kpos, int& lo, int& hi) {
  lo = -(1 << 30);
  hi = 1 << 30;
  if (c.causal) lo = kpos;                       // kpos <= qpos
  if (c.wr >= 0) lo = max(lo, kpos - c.wr);      // kpos <= qpos + wr
  if (c.wl >= 0) hi = kpos + c.wl;               // kpos >= qpos - wl
}
__device__ __forceinline__ void visible_k_interval(const ScoreCfg& c, int qpos, int k_len, int& lo, int& hi) {
  lo = 0;
  hi = k_len - 1;
  if (c.causal) hi = min(hi, qpos);
  if (c.wr >= 0) hi = min(hi, qpos + c.wr);
  if (c.wl >= 0) lo = max(lo, qpos - c.wl);
}
// Columns [first, last] of a tile (relative to its first column; any integers, possibly empty):
// column j is inside iff (unsigned)(j - lo) <= span.
struct ColMask {
  int lo;
  unsigned int span;
};
__device__ __forceinline__ ColMask make_col_mask(int first, int last) {
  first = max(first, -(1 << 20));
  last = min(last, 1 << 20);
  ColMask m;
  if (last < first) {
    m.lo = 1 << 28;
    m.span = 0u;
  } else {
    m.lo = first;
    m.span = (unsigned int)(last - first);
  }
  return m;
}
__device__ __forceinline__ bool col_visible(const ColMask& m, int j) { return (unsigned int)(j - m.lo) <= m.span; }

// Key range [lo, hi) any query position in [qpos_min, qpos_max] can see.
__device__ __forceinline__ void visible_key_range(const ScoreCfg& c, int qpos_min, int qpos_max,
                                                  int k_len, int& lo, int& hi) {
  int right = c.wr;                      // -1 open
  if (c.causal) right = (right >= 0) ? min(right, 0) : 0;
  hi = k_len;
  if (right >= 0) hi = min(k_len, qpos_max + right + 1);
  lo = 0;
  if (c.wl >= 0) lo = max(0, qpos_min - c.wl);
  if (hi < 0) hi = 0;
  if (lo > hi) lo = hi;
}

// Query-position range [lo, hi) that can see any key in [k_min, k_max].
__host__ __device__ __forceinline__ void visible_query_range(const ScoreCfg& c, int k_min, int k_max,
                                                    int qpos_begin, int qpos_end, int& lo,
                                                    int& hi) {
  int right = c.wr;
  if (c.causal) right = (right >= 0) ? min(right, 0) : 0;
  lo = qpos_begin;
  hi = qpos_end;
  if (right >= 0) lo = max(lo, k_min - right);  // kpos <= qpos + right
  if (c.wl >= 0) hi = min(hi, k_max + c.wl + 1);  // kpos >= qpos - wl
  if (lo > hi) lo = hi;
}

// ---------------------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};

// ---------------------------------------------------------------------------------------
// warp-level MMA toolkit (mma.sync m16n8k16, ldmatrix, cp.async)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4],
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16-byte async copy; bytes = 0 zero-fills the destination.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Tile of ROWS x D elements in shared memory with a 16-byte pad per row (row pitch D+8):
// ldmatrix over 8 consecutive rows then touches 8 different bank groups.
template <int D> struct TilePitch { static constexpr int value = D + 8; };

// Async-load `ROWS` rows of D elements (2-byte type) starting at global row `row0`;
// rows >= rows_valid are zero-filled.  `NT` threads cooperate.
template <int ROWS, int D, int NT, typename T>
__device__ __forceinline__ void load_tile_async(T* smem, const T* gbase, int64_t row_stride,
                                                int row0, int rows_valid, int tid) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  constexpr int P = TilePitch<D>::value;
  for (int i = tid; i < ROWS * CPR; i += NT) {
    int r = i / CPR, c = i % CPR;
    int gr = row0 + r;
    bool ok = gr < rows_valid;
    const T* src = gbase + (int64_t)(ok ? gr : 0) * row_stride + c * 8;
    cp_async16(smem_u32(smem + r * P + c * 8), src, ok ? 16 : 0);
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

// ---------------------------------------------------------------------------------------
// per-sequence geometry (dense or packed)
// ---------------------------------------------------------------------------------------
struct SeqInfo {
  int q_len, k_len;
  int64_t q_row0, k_row0;  // first row of this sequence in the row dimension
  int64_t q_boff, k_boff;  // 1 for dense (multiply stride[0] by batch), 0 for packed
};

__device__ __forceinline__ SeqInfo seq_info(const fa_attn_args& p, int b) {
  SeqInfo s;
  if (p.cu_seqlens_q) {
    int q0 = p.cu_seqlens_q[b], q1 = p.cu_seqlens_q[b + 1];
    int k0 = p.cu_seqlens_k[b], k1 = p.cu_seqlens_k[b + 1];
    s.q_len = q1 - q0;
    s.k_len = k1 - k0;
    s.q_row0 = q0;
    s.k_row0 = k0;
    s.q_boff = 0;
    s.k_boff = 0;
  } else {
    s.q_len = p.seqlen_q;
    s.k_len = p.seqlen_k;
    s.q_row0 = 0;
    s.k_row0 = 0;
    s.q_boff = b;
    s.k_boff = b;
  }
  if (p.seqused_q) s.q_len = max(0, min(s.q_len, p.seqused_q[b]));
  if (p.seqused_k) s.k_len = max(0, min(s.k_len, p.seqused_k[b]));
  return s;
}

}  // namespace fa
