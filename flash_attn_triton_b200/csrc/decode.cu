// KV-cache decode: split-KV attention over a paged (or contiguous) cache with the in-place append
// and the rotary embedding fused in, then a small combine.  HBM-bound: the job of the main
// kernel is to stream every cached K/V byte exactly once at full bandwidth.
//
//   decode_kernel    : CTA = (split, kv head x row group, sequence).  The query rows of one
//                      GQA group (seqlen_q x group <= 16 per row group) form the M=16 side
//                      of mma.sync m16n8k16, so one K/V byte serves the whole group.  K/V
//                      tiles of 64 keys arrive through a 3-stage cp.async ring of 16-byte
//                      page-row gathers; 4 warps take 16 keys each and merge at the end.
//                      The new tokens (k_new rotated, v_new) never come from the cache: the CTAs
//                      whose split holds their positions put them into the staged tile
//                      themselves, and the CTA of row group 0 also writes them to their cache
//                      slots -- one writer per (sequence, kv head, token), no separate launch.
//   combine_kernel   : merges the per-split partial outputs with their base-2 LSEs.
#include <mutex>

#include "common.cuh"

namespace fa {

struct DecodeGeom {
  int chunk;       // keys per split (multiple of 64)
  int num_splits;  // grid.x
  int row_groups;  // ceil(seqlen_q * group / 16)
  int page_shift;  // log2(page_size) or -1
};

template <typename T> __device__ __forceinline__ T hmul_rn(T a, T b);
template <> __device__ __forceinline__ __half hmul_rn(__half a, __half b) { return __hmul_rn(a, b); }
template <> __device__ __forceinline__ __nv_bfloat16 hmul_rn(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmul_rn(a, b); }
template <typename T> __device__ __forceinline__ T hadd_rn(T a, T b);
template <> __device__ __forceinline__ __half hadd_rn(__half a, __half b) { return __hadd_rn(a, b); }
template <> __device__ __forceinline__ __nv_bfloat16 hadd_rn(__nv_bfloat16 a, __nv_bfloat16 b) { return __hadd_rn(a, b); }
template <typename T> __device__ __forceinline__ T hsub_rn(T a, T b);
template <> __device__ __forceinline__ __half hsub_rn(__half a, __half b) { return __hsub_rn(a, b); }
template <> __device__ __forceinline__ __nv_bfloat16 hsub_rn(__nv_bfloat16 a, __nv_bfloat16 b) { return __hsub_rn(a, b); }

// Rotary on element d of a head vector x (read through `get`), every product and sum
// rounded to T like the reference's eager arithmetic (flash_attn_interface.py:57-66).
// A position outside the table [0, rotary_seqlen) leaves the element unrotated (the host checks
// the lengths when validation is on; this keeps the read in bounds when it is off).
template <typename T, typename F>
__device__ __forceinline__ T rotary_elem(F get, int d, const T* cos, const T* sin, int pos,
                                         int rotary_dim, int interleaved, int rotary_seqlen) {
  if (d >= rotary_dim || pos < 0 || pos >= rotary_seqlen) return get(d);
  const int half = rotary_dim >> 1;
  int i, partner;
  bool first;
  if (interleaved) {
    i = d >> 1;
    first = (d & 1) == 0;
    partner = d ^ 1;
  } else {
    first = d < half;
    i = first ? d : d - half;
    partner = first ? d + half : d - half;
  }
  const T c = cos[(int64_t)pos * half + i], s = sin[(int64_t)pos * half + i];
  const T x = get(d), y = get(partner);
  // first: x*c - y*s ; second: y*s + x*c  (y = first element of the pair)
  return first ? hsub_rn(hmul_rn(x, c), hmul_rn(y, s)) : hadd_rn(hmul_rn(y, s), hmul_rn(x, c));
}

__device__ __forceinline__ int64_t cache_row_offset(const fa_decode_args& p, int b, int pos,
                                                    int page_shift, const int64_t* stride) {
  int page, row;
  if (p.block_table) {
    int pi;
    if (page_shift >= 0) {
      pi = pos >> page_shift;
      row = pos & (p.page_size - 1);
    } else {
      pi = pos / p.page_size;
      row = pos - pi * p.page_size;
    }
    page = p.block_table[(int64_t)b * p.block_table_stride + pi];
  } else {
    page = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
    row = pos;
  }
  return (int64_t)page * stride[0] + (int64_t)row * stride[1];
}

// ---------------------------------------------------------------------------------------
// split-KV attention
// ---------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(128) decode_kernel(const fa_decode_args p, const ScoreCfg cfg,
                                                     const DecodeGeom geo) {
  constexpr int BN = 64, P = TilePitch<D>::value, NT = 128, NS = 3;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);  // 16 x P
  T* sK = sQ + 16 * P;                     // NS x BN x P
  T* sV = sK + NS * BN * P;                // NS x BN x P
  // after the key loop the K/V ring is reused as the cross-warp merge buffer

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, b = blockIdx.z;
  const int hk = blockIdx.y / geo.row_groups, rg = blockIdx.y % geo.row_groups;
  const int G = p.heads_q / p.heads_kv;
  const int R = p.seqlen_q * G;  // query rows of this kv head: r = sq * G + gi
  const int len_old = p.cache_seqlens[b];
  const int n_new = p.k_new ? p.seqlen_new : 0;
  const int len = len_old + n_new;
  const int pad = p.cache_leftpad ? p.cache_leftpad[b] : 0;
  const int k_begin = split * geo.chunk;
  if (k_begin >= len && split > 0) return;
  const int k_end = min(len, k_begin + geo.chunk);
  const int ntiles = max(0, (k_end - k_begin + BN - 1) / BN);
  const T* kbase = reinterpret_cast<const T*>(p.k_cache) + (int64_t)hk * p.kc_stride[2];
  const T* vbase = reinterpret_cast<const T*>(p.v_cache) + (int64_t)hk * p.vc_stride[2];

  auto load_tile = [&](int ti, int st) {
    constexpr int CPR = D / 8;
    T* dK = sK + st * BN * P;
    T* dV = sV + st * BN * P;
    const int key0 = k_begin + ti * BN;
    if (geo.page_shift >= 6 && pad == 0) {
      // the 64-key tile lies inside one page (pages are a power of two >= 64 rows and tiles
      // start on multiples of 64): one table lookup per thread and tile
      const int64_t kt = cache_row_offset(p, b, key0, geo.page_shift, p.kc_stride);
      const int64_t vt = cache_row_offset(p, b, key0, geo.page_shift, p.vc_stride);
#pragma unroll
      for (int i = tid; i < BN * CPR; i += NT) {
        const int r = i / CPR, c = i % CPR;
        const bool ok = key0 + r < min(k_end, len_old);     // new tokens are staged from k_new / v_new below
        const int rr = ok ? r : 0;
        cp_async16(smem_u32(dK + r * P + c * 8), kbase + kt + rr * p.kc_stride[1] + c * 8, ok ? 16 : 0);
        cp_async16(smem_u32(dV + r * P + c * 8), vbase + vt + rr * p.vc_stride[1] + c * 8, ok ? 16 : 0);
      }
      return;
    }
    for (int i = tid; i < BN * CPR; i += NT) {
      const int r = i / CPR, c = i % CPR;
      const int key = key0 + r;
      const bool ok = key < min(k_end, len_old);
      const int pos = (ok ? key : k_begin) + pad;
      const int64_t ko = cache_row_offset(p, b, pos, geo.page_shift, p.kc_stride);
      const int64_t vo = cache_row_offset(p, b, pos, geo.page_shift, p.vc_stride);
      cp_async16(smem_u32(dK + r * P + c * 8), kbase + ko + c * 8, ok ? 16 : 0);
      cp_async16(smem_u32(dV + r * P + c * 8), vbase + vo + c * 8, ok ? 16 : 0);
    }
  };

#pragma unroll
  for (int i = 0; i < NS - 1; ++i) {
    if (i < ntiles) load_tile(i, i);
    cp_async_commit();
  }

  // ---- Q rows (rotary fused) -> shared memory -> A fragments held in registers ---------
  {
    const T* cos = reinterpret_cast<const T*>(p.rotary_cos);
    const T* sin = reinterpret_cast<const T*>(p.rotary_sin);
    for (int i = tid; i < 16 * D; i += NT) {
      const int r = i / D, d = i % D;
      const int gr = rg * 16 + r;
      T val = Elem<T>::from_f(0.f);
      if (gr < R) {
        const int sq = gr / G, gi = gr % G;
        const T* qrow = reinterpret_cast<const T*>(p.q) + b * p.q_stride[0] + sq * p.q_stride[1] +
                        (int64_t)(hk * G + gi) * p.q_stride[2];
        if (cos) {
          const int pos = len - p.seqlen_q + sq + pad;
          val = rotary_elem<T>([&](int j) { return qrow[j]; }, d, cos, sin, pos, p.rotary_dim,
                               p.rotary_interleaved, p.rotary_seqlen);
        } else {
          val = qrow[d];
        }
      }
      sQ[r * P + d] = val;
    }
  }
  __syncthreads();
  uint32_t aq[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
    ldsm_x4(smem_u32(sQ + (lane & 15) * P + kk * 16 + (lane >> 4) * 8), aq[kk][0], aq[kk][1],
            aq[kk][2], aq[kk][3]);

  // per-thread rows g and g+8 of the row group
  int qpos[2];
  float slope[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int gr = min(rg * 16 + g + i * 8, R - 1);
    const int sq = gr / G, gi = gr % G;
    qpos[i] = len - p.seqlen_q + sq;
    slope[i] = cfg.has_alibi ? p.alibi_slopes[b * p.heads_q + hk * G + gi] : 0.f;
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  for (int ti = 0; ti < ntiles; ++ti) {
    cp_async_wait<NS - 2>();
    __syncthreads();
    {
      const int nx = ti + NS - 1;
      if (nx < ntiles) load_tile(nx, nx % NS);
      cp_async_commit();
    }
    // ---- append: the new tokens of this tile, rotated, into the staged tile and the cache ----
    {
      const int key0 = k_begin + ti * BN;
      const int first = max(key0, len_old), last = min(key0 + BN, k_end);   // new keys [first, last)
      if (n_new > 0 && last > first) {
        const T* cos = reinterpret_cast<const T*>(p.rotary_cos);
        const T* sin = reinterpret_cast<const T*>(p.rotary_sin);
        T* dK = sK + (ti % NS) * BN * P;
        T* dV = sV + (ti % NS) * BN * P;
        for (int i = tid; i < (last - first) * D; i += NT) {
          const int key = first + i / D, d = i % D;
          const int tok = key - len_old, pos = key + pad;
          const T* kn = reinterpret_cast<const T*>(p.k_new) + b * p.kn_stride[0] + tok * p.kn_stride[1] +
                        hk * p.kn_stride[2];
          const T* vn = reinterpret_cast<const T*>(p.v_new) + b * p.vn_stride[0] + tok * p.vn_stride[1] +
                        hk * p.vn_stride[2];
          T kv = kn[d];
          if (cos) kv = rotary_elem<T>([&](int j) { return kn[j]; }, d, cos, sin, pos, p.rotary_dim,
                                         p.rotary_interleaved, p.rotary_seqlen);
          const T vv = vn[d];
          dK[(key - key0) * P + d] = kv;
          dV[(key - key0) * P + d] = vv;
          if (rg == 0) {
            reinterpret_cast<T*>(p.k_cache)[cache_row_offset(p, b, pos, geo.page_shift, p.kc_stride) +
                                            (int64_t)hk * p.kc_stride[2] + d] = kv;
            reinterpret_cast<T*>(p.v_cache)[cache_row_offset(p, b, pos, geo.page_shift, p.vc_stride) +
                                            (int64_t)hk * p.vc_stride[2] + d] = vv;
          }
        }
        __syncthreads();
      }
    }
    const T* cK = sK + (ti % NS) * BN * P + warp * 16 * P;
    const T* cV = sV + (ti % NS) * BN * P + warp * 16 * P;

    float s[2][4];
    s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
    s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(smem_u32(cK + ((lane & 7) + ((lane >> 4) << 3)) * P + kk * 16 + ((lane >> 3) & 1) * 8),
              b0, b1, b2, b3);
      mma16816<T>(s[0], aq[kk], b0, b1);
      mma16816<T>(s[1], aq[kk], b2, b3);
    }
    float tmax[2] = {-INFINITY, -INFINITY};
    const int keyw = k_begin + ti * BN + warp * 16;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int col = keyw + nb * 8 + 2 * t + (e & 1);
        float th;
        float v = score_log2(cfg, slope[i], s[nb][e], qpos[i], col, th);
        if (!visible(cfg, qpos[i], col, k_end)) v = -INFINITY;
        s[nb][e] = v;
        tmax[i] = fmaxf(tmax[i], v);
      }
    }
    float alpha[2], muse[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mnew = fmaxf(mrow[i], quad_max(tmax[i]));
      muse[i] = (mnew == -INFINITY) ? 0.f : mnew;
      alpha[i] = exp2f(mrow[i] - muse[i]);
      mrow[i] = mnew;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float pv = exp2f(s[nb][e] - muse[e >> 1]);
        s[nb][e] = pv;
        psum[e >> 1] += pv;
      }
    }
    lrow[0] = lrow[0] * alpha[0] + psum[0];
    lrow[1] = lrow[1] * alpha[1] + psum[1];
    uint32_t a[4];
    a[0] = Elem<T>::pack(s[0][0], s[0][1]);
    a[1] = Elem<T>::pack(s[0][2], s[0][3]);
    a[2] = Elem<T>::pack(s[1][0], s[1][1]);
    a[3] = Elem<T>::pack(s[1][2], s[1][3]);
#pragma unroll
    for (int db2 = 0; db2 < D / 16; ++db2) {
      o[2 * db2][0] *= alpha[0]; o[2 * db2][1] *= alpha[0];
      o[2 * db2][2] *= alpha[1]; o[2 * db2][3] *= alpha[1];
      o[2 * db2 + 1][0] *= alpha[0]; o[2 * db2 + 1][1] *= alpha[0];
      o[2 * db2 + 1][2] *= alpha[1]; o[2 * db2 + 1][3] *= alpha[1];
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(smem_u32(cV + ((lane & 7) + ((lane >> 3) & 1) * 8) * P + db2 * 16 + (lane >> 4) * 8),
                b0, b1, b2, b3);
      mma16816<T>(o[2 * db2], a, b0, b1);
      mma16816<T>(o[2 * db2 + 1], a, b2, b3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the 4 warps (each saw a quarter of every tile) ------------------------------
  constexpr int OP = D + 4;  // fp32 pitch
  float* sO = reinterpret_cast<float*>(sK);   // 4 x 16 x OP
  float* sM = sO + 4 * 16 * OP;               // 4 x 16
  float* sL = sM + 4 * 16;                    // 4 x 16
  {
    float l0 = quad_sum(lrow[0]), l1 = quad_sum(lrow[1]);
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
      *reinterpret_cast<float2*>(sO + (warp * 16 + g) * OP + nb * 8 + 2 * t) = make_float2(o[nb][0], o[nb][1]);
      *reinterpret_cast<float2*>(sO + (warp * 16 + g + 8) * OP + nb * 8 + 2 * t) = make_float2(o[nb][2], o[nb][3]);
    }
    if (t == 0) {
      sM[warp * 16 + g] = mrow[0];
      sM[warp * 16 + g + 8] = mrow[1];
      sL[warp * 16 + g] = l0;
      sL[warp * 16 + g + 8] = l1;
    }
  }
  __syncthreads();
  const bool direct = geo.num_splits == 1;
  float* ws_o = reinterpret_cast<float*>(p.workspace);
  float* ws_l = ws_o + (int64_t)p.batch * p.seqlen_q * p.heads_q * geo.num_splits * D;
  for (int i = tid; i < 16 * (D / 4); i += NT) {
    const int r = i / (D / 4), c4 = (i % (D / 4)) * 4;
    const int gr = rg * 16 + r;
    if (gr >= R) continue;
    float mstar = fmaxf(fmaxf(sM[r], sM[16 + r]), fmaxf(sM[32 + r], sM[48 + r]));
    float w[4], lsum = 0.f;
#pragma unroll
    for (int wv = 0; wv < 4; ++wv) {
      w[wv] = (mstar == -INFINITY) ? 0.f : exp2f(sM[wv * 16 + r] - mstar);
      lsum += w[wv] * sL[wv * 16 + r];
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int wv = 0; wv < 4; ++wv) {
      float4 x = *reinterpret_cast<const float4*>(sO + (wv * 16 + r) * OP + c4);
      acc.x += w[wv] * x.x; acc.y += w[wv] * x.y; acc.z += w[wv] * x.z; acc.w += w[wv] * x.w;
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    const int sq = gr / G, h = hk * G + gr % G;
    if (direct) {
      T* og = reinterpret_cast<T*>(p.o) + b * p.o_stride[0] + sq * p.o_stride[1] + (int64_t)h * p.o_stride[2] + c4;
      uint2 pk;
      pk.x = Elem<T>::pack(acc.x, acc.y);
      pk.y = Elem<T>::pack(acc.z, acc.w);
      *reinterpret_cast<uint2*>(og) = pk;
    } else {
      const int64_t row = (((int64_t)b * p.seqlen_q + sq) * p.heads_q + h) * geo.num_splits + split;
      *reinterpret_cast<float4*>(ws_o + row * D + c4) = acc;
      if (c4 == 0) ws_l[row] = lsum > 0.f ? mstar + log2f(lsum) : -INFINITY;
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(128) decode_combine_kernel(const fa_decode_args p, const DecodeGeom geo) {
  // one warp per output row (b, sq, h)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  const int64_t nrows = (int64_t)p.batch * p.seqlen_q * p.heads_q;
  if (row >= nrows) return;
  const int h = row % p.heads_q;
  const int sq = (row / p.heads_q) % p.seqlen_q;
  const int b = row / ((int64_t)p.heads_q * p.seqlen_q);
  const int len = p.cache_seqlens[b] + (p.k_new ? p.seqlen_new : 0);
  const int nact = max(1, min(geo.num_splits, (len + geo.chunk - 1) / geo.chunk));
  const float* ws_o = reinterpret_cast<const float*>(p.workspace);
  const float* ws_l = ws_o + nrows * geo.num_splits * D;
  const float* lrow = ws_l + row * geo.num_splits;
  float mstar = -INFINITY;
  for (int s = 0; s < nact; ++s) mstar = fmaxf(mstar, lrow[s]);
  constexpr int EPL = (D + 31) / 32;  // elements per lane
  float acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
  float wsum = 0.f;
  for (int s = 0; s < nact; ++s) {
    const float w = (mstar == -INFINITY) ? 0.f : exp2f(lrow[s] - mstar);
    wsum += w;
    const float* orow = ws_o + (row * geo.num_splits + s) * D;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int d = e * 32 + lane;
      if (d < D) acc[e] += w * orow[d];
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  T* og = reinterpret_cast<T*>(p.o) + b * p.o_stride[0] + sq * p.o_stride[1] + (int64_t)h * p.o_stride[2];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int d = e * 32 + lane;
    if (d < D) og[d] = Elem<T>::from_f(acc[e] * inv);
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static DecodeGeom decode_geometry(const fa_decode_args& a) {
  DecodeGeom g;
  const int G = a.heads_q / a.heads_kv;
  g.row_groups = (a.seqlen_q * G + 15) / 16;
  const int64_t cap = a.block_table ? (int64_t)a.block_table_stride * a.page_size : a.page_size;
  const int64_t max_len = cap > 0 ? cap : 1;
  const int64_t base_ctas = (int64_t)a.batch * a.heads_kv * g.row_groups;
  int splits;
  if (a.num_splits > 0) {
    splits = a.num_splits;
  } else {
    const int64_t target = 148 * 2 * 8;
    splits = (int)((target + base_ctas - 1) / (base_ctas > 0 ? base_ctas : 1));
    const int64_t max_splits = (max_len + 511) / 512;
    if (splits > max_splits) splits = (int)max_splits;
    if (splits < 1) splits = 1;
  }
  int64_t chunk = (max_len + splits - 1) / splits;
  chunk = (chunk + 63) / 64 * 64;
  if (chunk >= 256) chunk = (chunk + 255) / 256 * 256;
  g.chunk = (int)chunk;
  g.num_splits = (int)((max_len + chunk - 1) / chunk);
  if (g.num_splits < 1) g.num_splits = 1;
  g.page_shift = -1;
  if (a.page_size > 0 && (a.page_size & (a.page_size - 1)) == 0) {
    int s = 0;
    while ((1 << s) < a.page_size) ++s;
    g.page_shift = s;
  }
  return g;
}

size_t decode_workspace_bytes(const fa_decode_args& a) {
  if (a.heads_kv <= 0 || a.heads_q <= 0) return 0;
  DecodeGeom g = decode_geometry(a);
  if (g.num_splits == 1) return 0;
  return (size_t)a.batch * a.seqlen_q * a.heads_q * g.num_splits * (a.head_dim + 1) * sizeof(float);
}

template <typename T, int D>
static int launch_decode(const fa_decode_args& a, const ScoreCfg& cfg, const DecodeGeom& g, cudaStream_t st) {
  constexpr int P = TilePitch<D>::value;
  constexpr size_t ring = (size_t)(16 + 2 * 3 * 64) * P * sizeof(T);
  constexpr size_t merge = (size_t)16 * P * sizeof(T) + (size_t)(4 * 16 * (D + 4) + 128) * sizeof(float);
  constexpr size_t smem = ring > merge ? ring : merge;
  auto kern = decode_kernel<T, D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return FA_ERR_LAUNCH;
    }
  }
  dim3 grid(g.num_splits, a.heads_kv * g.row_groups, a.batch);
  kern<<<grid, 128, smem, st>>>(a, cfg, g);
  if (int r = check_launch("decode")) return r;
  if (g.num_splits > 1) {
    const int64_t rows = (int64_t)a.batch * a.seqlen_q * a.heads_q;
    decode_combine_kernel<T, D><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(a, g);
    return check_launch("decode_combine");
  }
  return FA_OK;
}

template <typename T>
static int decode_t(const fa_decode_args& a, const ScoreCfg& cfg, const DecodeGeom& g, cudaStream_t st) {
  switch (a.head_dim) {
    case 16: return launch_decode<T, 16>(a, cfg, g, st);
    case 32: return launch_decode<T, 32>(a, cfg, g, st);
    case 64: return launch_decode<T, 64>(a, cfg, g, st);
    case 128: return launch_decode<T, 128>(a, cfg, g, st);
    case 256: return launch_decode<T, 256>(a, cfg, g, st);
  }
  set_error("head_dim %d not in {16,32,64,128,256}", a.head_dim);
  return FA_ERR_UNSUPPORTED;
}

int decode_paged(const fa_decode_args& a, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen_q == 0 || a.heads_q == 0) return FA_OK;
  DecodeGeom g = decode_geometry(a);
  size_t need = decode_workspace_bytes(a);
  if (need > 0 && (a.workspace == nullptr || a.workspace_bytes < need)) {
    set_error("decode workspace too small: need %zu bytes, got %zu", need, a.workspace_bytes);
    return FA_ERR_WORKSPACE;
  }
  // bottom-right alignment: the causal mask and window are relative to the query's
  // position at the end of the cached sequence
  ScoreCfg cfg = make_score_cfg(a.softmax_scale, 0.f, a.causal, a.window_left, a.window_right,
                                a.alibi_slopes != nullptr);
  return a.dtype == FA_BF16 ? decode_t<__nv_bfloat16>(a, cfg, g, st) : decode_t<__half>(a, cfg, g, st);
}

// ---------------------------------------------------------------------------------------
// Decode without any allocation by anyone: the split-KV partials live in a fixed array
// that is part of the library image.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle: the device address has to be asked for,
// once per device, while that device is current.
static void* static_scratch_ptr(int device) {
  constexpr int kMaxDevices = 64;
  static void* ptrs[kMaxDevices] = {nullptr};
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) {
    set_error("device ordinal %d out of range for the static decode scratch", device);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[device] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("cudaGetSymbolAddress(static decode scratch) on device %d: %s", device,
                cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[device] = p;
  }
  return ptrs[device];
}

size_t decode_static_scratch_bytes() { return kStaticScratchBytes; }

int decode_paged_static(const fa_decode_args& a, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen_q == 0 || a.heads_q == 0) return FA_OK;
  const size_t need = decode_workspace_bytes(a);
  if (need > kStaticScratchBytes) {
    set_error("fa_decode_paged_static: this problem needs %zu bytes of split-KV scratch but the "
              "built-in array holds %zu; pass a smaller num_splits or use fa_decode_paged with "
              "your own workspace", need, kStaticScratchBytes);
    return FA_ERR_WORKSPACE;
  }
  void* p = static_scratch_ptr(a.device);
  if (p == nullptr) return FA_ERR_LAUNCH;
  fa_decode_args b = a;
  b.workspace = p;
  b.workspace_bytes = kStaticScratchBytes;
  return decode_paged(b, st);
}

}  // namespace fa
