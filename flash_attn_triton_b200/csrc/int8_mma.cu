// INT8 path: the per-token K quantiser (bit-exact with the reference formula) and the
// INT8-QK^T forward on warp-level integer MMA (mma.sync m16n8k32 s8 -> s32).
#include "common.cuh"

namespace fa {

// round-half-away computed as floor(x+0.5) / ceil(x-0.5) in IEEE fp32; NOT roundf
// (differs at x = 0.49999997).  Explicit _rn intrinsics keep the compiler from fusing.
__device__ __forceinline__ int round_i8(float x) {
  return (int)(x >= 0.f ? floorf(__fadd_rn(x, 0.5f)) : ceilf(__fsub_rn(x, 0.5f)));
}

// The same function for |x| < 2^22 without the round-to-integer and float-to-int conversions,
// which run on the quarter-rate conversion pipe and bound a streaming kernel: ceil(x - 0.5) is
// -floor(|x| + 0.5) (fp32 rounding is symmetric), and floor(t) of a non-negative t < 2^23 is
// what the mantissa holds after t + 2^23 rounded DOWN (the sum's unit in the last place is 1).
__device__ __forceinline__ int round_i8_fast(float x) {
  const float t = __fadd_rn(fabsf(x), 0.5f);
  const int m = __float_as_int(__fadd_rd(t, 8388608.0f)) & 0x3ff;
  return x < 0.f ? -m : m;
}

// ---------------------------------------------------------------------------------------
// K quantiser: rows x D fp16 -> int8 codes + fp32 scale per row.  HBM-bound: 2 B read and
// 1 B written per element.  D/8 lanes share a row, 16 bytes each; every thread keeps kRows
// independent rows in flight per step (all loads are issued before the first is used) and the grid
// strides over the rows, a few resident blocks per SM, so that enough bytes are outstanding to
// cover the memory latency.  Loads and stores bypass L1 and are marked streaming: nothing is reused.
// ---------------------------------------------------------------------------------------
// kDivide: codes = round(x / s) (the reference's query form) instead of round(x * (1/s))
#ifndef FA_QUANT_ROWS
#define FA_QUANT_ROWS 6
#endif
#ifndef FA_QUANT_BLOCKS
#define FA_QUANT_BLOCKS 8
#endif
constexpr int kQuantRows = FA_QUANT_ROWS;
template <int D, bool kDivide = false>
__global__ void __launch_bounds__(256) quantize_k_kernel(const __half* __restrict__ k,
                                                         int8_t* __restrict__ k8,
                                                         float* __restrict__ s_k, int64_t rows) {
  constexpr int LPR = D / 8;
  constexpr int RPB = 256 / LPR;                     // rows per block and sub-step
  const int tid = threadIdx.x;
  const int c = tid % LPR;
  const int64_t step = (int64_t)gridDim.x * RPB * kQuantRows;
  for (int64_t blk = (int64_t)blockIdx.x * RPB * kQuantRows; blk < rows; blk += step) {   // block-uniform bound
    const int64_t base = blk + tid / LPR;
    uint4 raw[kQuantRows];
#pragma unroll
    for (int j = 0; j < kQuantRows; ++j) {
      const int64_t row = base + (int64_t)j * RPB;
      raw[j] = make_uint4(0, 0, 0, 0);
      if (row < rows) raw[j] = __ldcs(reinterpret_cast<const uint4*>(k + row * D + c * 8));
    }
#pragma unroll
    for (int j = 0; j < kQuantRows; ++j) {
      const int64_t row = base + (int64_t)j * RPB;
      const __half2* h2 = reinterpret_cast<const __half2*>(&raw[j]);
      float x[8];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h2[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
      // every lane of the warp takes part in the shuffles (the loop bound is warp-uniform)
#pragma unroll
      for (int s = LPR / 2; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
      const float sc = __fdiv_rn(fmaxf(amax, 1.0f), 127.0f);
      const float inv = __fdiv_rn(1.0f, sc);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = kDivide ? __fdiv_rn(x[i], sc) : __fmul_rn(x[i], inv);
        const float c2 = kDivide ? __fdiv_rn(x[4 + i], sc) : __fmul_rn(x[4 + i], inv);
        lo |= (uint32_t)(uint8_t)(int8_t)round_i8_fast(a) << (8 * i);
        hi |= (uint32_t)(uint8_t)(int8_t)round_i8_fast(c2) << (8 * i);
      }
      if (row < rows) {
        __stcs(reinterpret_cast<uint2*>(k8 + row * D + c * 8), make_uint2(lo, hi));
        if (c == 0) __stcs(s_k + row, sc);
      }
    }
  }
}

template <int D, bool kDivide>
static int launch_quantiser(const void* x, int8_t* x8, float* s, int64_t rows, cudaStream_t st, const char* what) {
  constexpr int RPB = 256 / (D / 8);
  const int64_t need = (rows + RPB * kQuantRows - 1) / (RPB * kQuantRows);
  int device = 0;
  cudaGetDevice(&device);
  const int64_t cap = (int64_t)sm_count(device) * FA_QUANT_BLOCKS;  // 8 blocks of 256 threads fill an SM
  quantize_k_kernel<D, kDivide><<<(unsigned)(need < cap ? need : cap), 256, 0, st>>>(
      reinterpret_cast<const __half*>(x), x8, s, rows);
  return check_launch(what);
}

int quantize_k(const void* k, int8_t* k8, float* s_k, int64_t rows, int head_dim, cudaStream_t st) {
  if (rows == 0) return FA_OK;
  switch (head_dim) {
    case 32: return launch_quantiser<32, false>(k, k8, s_k, rows, st, "quantize_k");
    case 64: return launch_quantiser<64, false>(k, k8, s_k, rows, st, "quantize_k");
    case 128: return launch_quantiser<128, false>(k, k8, s_k, rows, st, "quantize_k");
    case 256: return launch_quantiser<256, false>(k, k8, s_k, rows, st, "quantize_k");
  }
  set_error("INT8 path needs head_dim in {32,64,128,256}, got %d", head_dim);
  return FA_ERR_UNSUPPORTED;
}

// Per-query-row codes in the division form q / s_q (attention_kernel_int8.py:33-39, :100);
// used by the tcgen05 INT8 forward, which stages the codes with TMA.
int quantize_q(const void* q, int8_t* q8, float* s_q, int64_t rows, int head_dim, cudaStream_t st) {
  if (rows == 0) return FA_OK;
  if (head_dim != 128) {
    set_error("quantize_q: head_dim 128 only");
    return FA_ERR_UNSUPPORTED;
  }
  return launch_quantiser<128, true>(q, q8, s_q, rows, st, "quantize_q");
}

// ---------------------------------------------------------------------------------------
// INT8 forward, mma.sync version
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mma16832_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int D>
__global__ void __launch_bounds__(128) fwd_int8_mma_kernel(const fa_int8_args p) {
  using T = __half;
  constexpr int BM = 64, BN = 64, P = TilePitch<D>::value, P8 = D + 16, NT = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);                      // BM x P   (fp16 q, later O)
  T* sV = sQ + BM * P;                                         // 2 x BN x P
  int8_t* sQ8 = reinterpret_cast<int8_t*>(sV + 2 * BN * P);    // BM x P8
  int8_t* sK8 = sQ8 + BM * P8;                                 // 2 x BN x P8
  float* sSk = reinterpret_cast<float*>(sK8 + 2 * BN * P8);    // 2 x BN

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int mblk = blockIdx.x, bh = blockIdx.y;
  const int S = p.seqlen;
  const int m0 = mblk * BM;
  const T* qg = reinterpret_cast<const T*>(p.q) + (int64_t)bh * S * D;
  const T* vg = reinterpret_cast<const T*>(p.v) + (int64_t)bh * S * D;
  const int8_t* k8g = p.k8 + (int64_t)bh * S * D;
  const float* skg = p.s_k + (int64_t)bh * S;
  const int klen = p.seqlen_k_valid > 0 ? p.seqlen_k_valid : S;   // keys past it are padding
  const int off = p.q_pos_offset;                                 // query row i sits at position i + off
  const int n_all = (klen + BN - 1) / BN;
  const int n_hi = p.causal ? max(0, min(n_all, (min(m0 + BM, S) - 1 + off) / BN + 1)) : n_all;

  auto load_kv = [&](int n, int st) {
    load_tile_async<BN, D, NT>(sV + st * BN * P, vg, D, n * BN, S, tid);
    constexpr int CPR = D / 16;
    for (int i = tid; i < BN * CPR; i += NT) {
      int r = i / CPR, c = i % CPR;
      int gr = n * BN + r;
      bool ok = gr < S;
      cp_async16(smem_u32(sK8 + (st * BN + r) * P8 + c * 16), k8g + (int64_t)(ok ? gr : 0) * D + c * 16, ok ? 16 : 0);
    }
    if (tid < BN) {
      int gr = n * BN + tid;
      sSk[st * BN + tid] = gr < S ? skg[gr] : 1.0f;
    }
  };

  load_tile_async<BM, D, NT>(sQ, qg, D, m0, S, tid);
  cp_async_commit();
  load_kv(0, 0);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  // per-row quantisation of q (division form q / s_q), 2 lanes... one warp owns 16 rows;
  // lane pair (2 lanes per row) splits the row.
  float sq_row[2];  // scales of this thread's MMA rows g, g+8
  {
    const int r = warp * 16 + (lane >> 1);
    const int half = lane & 1;
    const T* src = sQ + r * P + half * (D / 2);
    float amax = 0.f;
    for (int d = 0; d < D / 2; ++d) amax = fmaxf(amax, fabsf(__half2float(src[d])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float sc = __fdiv_rn(fmaxf(amax, 1.0f), 127.0f);
    int8_t* dst = sQ8 + r * P8 + half * (D / 2);
    for (int d = 0; d < D / 2; ++d) dst[d] = (int8_t)round_i8(__fdiv_rn(__half2float(src[d]), sc));
    // hand the scale of row (warp*16 + g) and (+8) to the lanes that need it
    sq_row[0] = __shfl_sync(0xffffffffu, sc, 2 * g);
    sq_row[1] = __shfl_sync(0xffffffffu, sc, 2 * (g + 8));
  }
  __syncwarp();

  const float qk_scale = p.softmax_scale * 1.44269504f;
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int r0 = m0 + warp * 16 + g;

  for (int n = 0; n < n_hi; ++n) {
    const int st = n & 1;
    if (n + 1 < n_hi) {
      load_kv(n + 1, st ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int8_t* cK = sK8 + st * BN * P8;
    const T* cV = sV + st * BN * P;
    const float* cS = sSk + st * BN;

    int acc[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0;
#pragma unroll
    for (int kk = 0; kk < D / 32; ++kk) {
      uint32_t a[4];
      ldsm_x4(smem_u32(sQ8 + (warp * 16 + (lane & 15)) * P8 + kk * 32 + (lane >> 4) * 16), a[0], a[1], a[2], a[3]);
#pragma unroll
      for (int nb2 = 0; nb2 < BN / 16; ++nb2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(cK + (nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * P8 + kk * 32 + ((lane >> 3) & 1) * 16),
                b0, b1, b2, b3);
        mma16832_s8(acc[2 * nb2], a, b0, b1);
        mma16832_s8(acc[2 * nb2 + 1], a, b2, b3);
      }
    }
    float s[BN / 8][4];
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int cl = nb * 8 + 2 * t + (e & 1);
        const int col = n * BN + cl;
        const int row = r0 + i * 8;
        // (float(acc) * (s_q * s_k)) * qk_scale, then the additive -1e6 mask of the reference
        float v = __fmul_rn(__fmul_rn((float)acc[nb][e], __fmul_rn(sq_row[i], cS[cl])), qk_scale);
        const bool keep = col < klen && (!p.causal || col <= row + off);
        if (!keep) v += -1.0e6f;
        s[nb][e] = v;
        tmax[i] = fmaxf(tmax[i], v);
      }
    }
    float alpha[2], muse[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      muse[i] = fmaxf(mrow[i], quad_max(tmax[i]));
      alpha[i] = exp2f(mrow[i] - muse[i]);
      mrow[i] = muse[i];
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float pv = exp2f(s[nb][e] - muse[e >> 1]);
        s[nb][e] = pv;
        psum[e >> 1] += pv;
      }
    }
    lrow[0] = lrow[0] * alpha[0] + psum[0];
    lrow[1] = lrow[1] * alpha[1] + psum[1];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk2 = 0; kk2 < BN / 16; ++kk2) {
      uint32_t a[4];
      a[0] = Elem<T>::pack(s[2 * kk2][0], s[2 * kk2][1]);
      a[1] = Elem<T>::pack(s[2 * kk2][2], s[2 * kk2][3]);
      a[2] = Elem<T>::pack(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]);
      a[3] = Elem<T>::pack(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
#pragma unroll
      for (int db2 = 0; db2 < D / 16; ++db2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(cV + (kk2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P + db2 * 16 + (lane >> 4) * 8),
                  b0, b1, b2, b3);
        mma16816<T>(o[2 * db2], a, b0, b1);
        mma16816<T>(o[2 * db2 + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  float inv[2], lse[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float l = quad_sum(lrow[i]);
    inv[i] = l > 0.f ? 1.f / l : 0.f;
    lse[i] = l > 0.f ? mrow[i] + log2f(l) : -INFINITY;
  }
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) {
    *reinterpret_cast<uint32_t*>(sQ + (warp * 16 + g) * P + nb * 8 + 2 * t) =
        Elem<T>::pack(o[nb][0] * inv[0], o[nb][1] * inv[0]);
    *reinterpret_cast<uint32_t*>(sQ + (warp * 16 + g + 8) * P + nb * 8 + 2 * t) =
        Elem<T>::pack(o[nb][2] * inv[1], o[nb][3] * inv[1]);
  }
  if (p.lse2 != nullptr && t == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (r0 + i * 8 < S) p.lse2[(int64_t)bh * S + r0 + i * 8] = lse[i];
  }
  __syncthreads();
  T* og = reinterpret_cast<T*>(p.o) + (int64_t)bh * S * D;
  constexpr int CPR = D / 8;
  for (int i = tid; i < BM * CPR; i += NT) {
    int r = i / CPR, c = i % CPR;
    if (m0 + r < S)
      *reinterpret_cast<uint4*>(og + (int64_t)(m0 + r) * D + c * 8) =
          *reinterpret_cast<const uint4*>(sQ + r * P + c * 8);
  }
}

template <int D> static int launch_int8(const fa_int8_args& a, cudaStream_t st) {
  constexpr int P = TilePitch<D>::value, P8 = D + 16;
  constexpr size_t smem = (size_t)(64 + 2 * 64) * P * 2 + (size_t)(64 + 2 * 64) * P8 + 2 * 64 * sizeof(float);
  auto kern = fwd_int8_mma_kernel<D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("fwd_int8_mma: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return FA_ERR_LAUNCH;
    }
  }
  dim3 grid((a.seqlen + 63) / 64, a.batch * a.heads);
  kern<<<grid, 128, smem, st>>>(a);
  return check_launch("fwd_int8_mma");
}

int fwd_int8_mma(const fa_int8_args& a, cudaStream_t st) {
  if (a.batch * a.heads == 0 || a.seqlen == 0) return FA_OK;
  switch (a.head_dim) {
    case 32: return launch_int8<32>(a, st);
    case 64: return launch_int8<64>(a, st);
    case 128: return launch_int8<128>(a, st);
    case 256: return launch_int8<256>(a, st);
  }
  set_error("INT8 path needs head_dim in {32,64,128,256}, got %d", a.head_dim);
  return FA_ERR_UNSUPPORTED;
}

}  // namespace fa
