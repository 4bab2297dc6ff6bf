// Forward attention on warp-level tensor-core MMA (mma.sync m16n8k16).
//
// This is the all-shapes kernel: every head_dim in {16,32,64,128,256}, fp16/bf16, dense or
// packed variable-length batches, GQA, causal / sliding window / ALiBi / softcap, arbitrary
// row/head strides.  The tcgen05 kernel (fwd_sm100.cu) takes over the shapes it is built
// for; this one stays the correctness baseline it is compared against at full size.
//
// One CTA = 64 query rows of one (batch, head); 4 warps x 16 rows.  K/V tiles of 64 keys
// are double-buffered in shared memory with cp.async.  Scores never leave registers.
#include "common.cuh"

namespace fa {

template <typename T, int D>
__global__ void __launch_bounds__(128)
fwd_mma_kernel(const fa_attn_args p, const ScoreCfg cfg) {
  constexpr int BM = 64, BN = 64, P = TilePitch<D>::value, NT = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + BM * P;
  T* sV = sK + 2 * BN * P;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int mblk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p, b);
  const int m0 = mblk * BM;
  if (m0 >= si.q_len) return;
  const int hk = h / (p.heads_q / p.heads_kv);
  const T* qg = reinterpret_cast<const T*>(p.q) + si.q_boff * p.q_stride[0] +
                si.q_row0 * p.q_stride[1] + (int64_t)h * p.q_stride[2];
  const T* kg = reinterpret_cast<const T*>(p.k) + si.k_boff * p.k_stride[0] +
                si.k_row0 * p.k_stride[1] + (int64_t)hk * p.k_stride[2];
  const T* vg = reinterpret_cast<const T*>(p.v) + si.k_boff * p.v_stride[0] +
                si.k_row0 * p.v_stride[1] + (int64_t)hk * p.v_stride[2];
  const float slope = cfg.has_alibi ? p.alibi_slopes[b * p.heads_q + h] : 0.f;
  const int off = p.q_pos_offset;

  int klo, khi;
  visible_key_range(cfg, m0 + off, min(m0 + BM, si.q_len) - 1 + off, si.k_len, klo, khi);
  const int n_lo = klo / BN, n_hi = (khi + BN - 1) / BN;

  load_tile_async<BM, D, NT>(sQ, qg, p.q_stride[1], m0, si.q_len, tid);
  if (n_lo < n_hi) {
    load_tile_async<BN, D, NT>(sK, kg, p.k_stride[1], n_lo * BN, si.k_len, tid);
    load_tile_async<BN, D, NT>(sV, vg, p.v_stride[1], n_lo * BN, si.k_len, tid);
  }
  cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int r0 = m0 + warp * 16 + g;  // this thread's rows: r0 and r0+8

  for (int n = n_lo; n < n_hi; ++n) {
    const int st = (n - n_lo) & 1;
    if (n + 1 < n_hi) {
      load_tile_async<BN, D, NT>(sK + (st ^ 1) * BN * P, kg, p.k_stride[1], (n + 1) * BN, si.k_len, tid);
      load_tile_async<BN, D, NT>(sV + (st ^ 1) * BN * P, vg, p.v_stride[1], (n + 1) * BN, si.k_len, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const T* cK = sK + st * BN * P;
    const T* cV = sV + st * BN * P;

    // ---- S = Q K^T -------------------------------------------------------------------
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(smem_u32(sQ + (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8), a[0], a[1],
              a[2], a[3]);
#pragma unroll
      for (int nb2 = 0; nb2 < BN / 16; ++nb2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(cK + (nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * P + kk * 16 +
                         ((lane >> 3) & 1) * 8),
                b0, b1, b2, b3);
        mma16816<T>(s[2 * nb2], a, b0, b1);
        mma16816<T>(s[2 * nb2 + 1], a, b2, b3);
      }
    }

    // ---- score pipeline + mask ---------------------------------------------------------
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r0 + (e >> 1) * 8;
        const int col = n * BN + nb * 8 + 2 * t + (e & 1);
        const bool inside = row < si.q_len && col < si.k_len;
        const float bias = (cfg.bias != nullptr && inside) ? bias_at(cfg, b, h, row, col) : 0.f;
        float th;
        float v = score_log2(cfg, slope, s[nb][e], row + off, col, th, bias);
        if (!visible(cfg, row + off, col, si.k_len)) v = -INFINITY;
        s[nb][e] = v;
        tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
      }
    }
    // ---- online softmax ----------------------------------------------------------------
    float alpha[2], muse[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mnew = fmaxf(mrow[i], quad_max(tmax[i]));
      muse[i] = (mnew == -INFINITY) ? 0.f : mnew;
      alpha[i] = exp2f(mrow[i] - muse[i]);  // mrow = -inf -> 0
      mrow[i] = mnew;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float pv = exp2f(s[nb][e] - muse[e >> 1]);
        psum[e >> 1] += pv;                      // the normaliser sums the probabilities before dropout
        if (cfg.dropout_p > 0.f) {
          const int row = r0 + (e >> 1) * 8, col = n * BN + nb * 8 + 2 * t + (e & 1);
          pv = dropout_keep(cfg, (uint32_t)si.q_row0, row, col) ? pv * cfg.dropout_scale : 0.f;
        }
        s[nb][e] = pv;
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) lrow[i] = lrow[i] * alpha[i] + psum[i];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }

    // ---- O += P V ------------------------------------------------------------------------
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
        ldsm_x4_t(smem_u32(cV + (kk2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P + db2 * 16 +
                           (lane >> 4) * 8),
                  b0, b1, b2, b3);
        mma16816<T>(o[2 * db2], a, b0, b1);
        mma16816<T>(o[2 * db2 + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- epilogue ----------------------------------------------------------------------------
  float inv[2], lse[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float l = quad_sum(lrow[i]);
    inv[i] = l > 0.f ? 1.f / l : 0.f;
    lse[i] = l > 0.f ? mrow[i] + log2f(l) : -INFINITY;
  }
  // stage O through the (now idle) Q tile so global stores are 16-byte and coalesced
#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) {
    uint32_t v0 = Elem<T>::pack(o[nb][0] * inv[0], o[nb][1] * inv[0]);
    uint32_t v1 = Elem<T>::pack(o[nb][2] * inv[1], o[nb][3] * inv[1]);
    *reinterpret_cast<uint32_t*>(sQ + (warp * 16 + g) * P + nb * 8 + 2 * t) = v0;
    *reinterpret_cast<uint32_t*>(sQ + (warp * 16 + g + 8) * P + nb * 8 + 2 * t) = v1;
  }
  if (p.lse2 != nullptr && t == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int row = r0 + i * 8;
      if (row < si.q_len)
        p.lse2[si.q_boff * p.lse_stride[0] + (si.q_row0 + row) * p.lse_stride[1] +
               (int64_t)h * p.lse_stride[2]] = lse[i];
    }
  }
  __syncthreads();
  T* og = reinterpret_cast<T*>(p.o) + si.q_boff * p.o_stride[0] + si.q_row0 * p.o_stride[1] +
          (int64_t)h * p.o_stride[2];
  constexpr int CPR = D / 8;
  for (int i = tid; i < BM * CPR; i += NT) {
    int r = i / CPR, c = i % CPR;
    if (m0 + r < si.q_len) {
      uint4 val = *reinterpret_cast<const uint4*>(sQ + r * P + c * 8);
      *reinterpret_cast<uint4*>(og + (int64_t)(m0 + r) * p.o_stride[1] + c * 8) = val;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Probabilities as a matrix: P[b, h, i, j] = exp2(score(i, j) - lse2[i]) (after dropout), fp32.
// CTA = a 64 x 64 tile of one (batch, head); the score tile is recomputed like in the forward.
// ---------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(128)
attn_probs_kernel(const fa_attn_args p, const ScoreCfg cfg, float* __restrict__ probs, const int64_t ps0,
                  const int64_t ps1, const int64_t ps2, const int64_t ps3, float* __restrict__ lse_nat,
                  const int64_t lse_nat_stride, const int n_col_tiles) {
  constexpr int BM = 64, BN = 64, P = TilePitch<D>::value, NT = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + BM * P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int mblk = blockIdx.x / n_col_tiles, nblk = blockIdx.x % n_col_tiles, h = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p, b);
  const int m0 = mblk * BM, n0 = nblk * BN;
  if (m0 >= si.q_len || n0 >= si.k_len) return;
  const int hk = h / (p.heads_q / p.heads_kv);
  const T* qg = reinterpret_cast<const T*>(p.q) + si.q_boff * p.q_stride[0] + si.q_row0 * p.q_stride[1] +
                (int64_t)h * p.q_stride[2];
  const T* kg = reinterpret_cast<const T*>(p.k) + si.k_boff * p.k_stride[0] + si.k_row0 * p.k_stride[1] +
                (int64_t)hk * p.k_stride[2];
  const float slope = cfg.has_alibi ? p.alibi_slopes[b * p.heads_q + h] : 0.f;
  const int off = p.q_pos_offset;
  load_tile_async<BM, D, NT>(sQ, qg, p.q_stride[1], m0, si.q_len, tid);
  load_tile_async<BN, D, NT>(sK, kg, p.k_stride[1], n0, si.k_len, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  float s[BN / 8][4];
#pragma unroll
  for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldsm_x4(smem_u32(sQ + (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
    for (int nb2 = 0; nb2 < BN / 16; ++nb2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(smem_u32(sK + (nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * P + kk * 16 + ((lane >> 3) & 1) * 8),
              b0, b1, b2, b3);
      mma16816<T>(s[2 * nb2], a, b0, b1);
      mma16816<T>(s[2 * nb2 + 1], a, b2, b3);
    }
  }
  const int r0 = m0 + warp * 16 + g;
  float l2[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + i * 8;
    l2[i] = -INFINITY;
    if (row < si.q_len)
      l2[i] = p.lse2[si.q_boff * p.lse_stride[0] + (si.q_row0 + row) * p.lse_stride[1] + (int64_t)h * p.lse_stride[2]];
    if (lse_nat != nullptr && nblk == 0 && t == 0 && row < si.q_len)
      lse_nat[((int64_t)b * p.heads_q + h) * lse_nat_stride + row] = l2[i] * FA_LN2;   // -inf stays -inf
  }
  float* pg = probs + (int64_t)b * ps0 + (int64_t)h * ps1;
#pragma unroll
  for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const int row = r0 + i * 8, col = n0 + nb * 8 + 2 * t + (e & 1);
      if (row >= si.q_len || col >= si.k_len) continue;
      const float bias = cfg.bias != nullptr ? bias_at(cfg, b, h, row, col) : 0.f;
      float th;
      const float sc = score_log2(cfg, slope, s[nb][e], row + off, col, th, bias);
      float pv = 0.f;
      if (l2[i] != -INFINITY && visible(cfg, row + off, col, si.k_len)) pv = exp2f(sc - l2[i]);
      if (cfg.dropout_p > 0.f) pv = dropout_keep(cfg, (uint32_t)si.q_row0, row, col) ? pv * cfg.dropout_scale : 0.f;
      pg[(int64_t)row * ps2 + (int64_t)col * ps3] = pv;
    }
  }
}

template <typename T, int D>
static int launch_probs(const fa_attn_args& a, const ScoreCfg& cfg, float* probs, const int64_t* ps, float* lse_nat,
                        int64_t lse_nat_stride, cudaStream_t st) {
  constexpr int P = TilePitch<D>::value;
  constexpr size_t smem = (size_t)(64 + 64) * P * sizeof(T);
  auto kern = attn_probs_kernel<T, D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("attn_probs: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return FA_ERR_LAUNCH;
    }
  }
  const int nct = (a.seqlen_k + 63) / 64;
  dim3 grid(((a.seqlen_q + 63) / 64) * nct, a.heads_q, a.batch);
  kern<<<grid, 128, smem, st>>>(a, cfg, probs, ps[0], ps[1], ps[2], ps[3], lse_nat, lse_nat_stride, nct);
  return check_launch("attn_probs");
}

int attn_probs(const fa_attn_args& a, const ScoreCfg& cfg, float* probs, const int64_t* ps, float* lse_nat,
               int64_t lse_nat_stride, cudaStream_t st) {
#define FA_P(TT, DD) return launch_probs<TT, DD>(a, cfg, probs, ps, lse_nat, lse_nat_stride, st)
  if (a.dtype == FA_BF16) {
    switch (a.head_dim) { case 16: FA_P(__nv_bfloat16, 16); case 32: FA_P(__nv_bfloat16, 32); case 64: FA_P(__nv_bfloat16, 64);
                          case 128: FA_P(__nv_bfloat16, 128); case 256: FA_P(__nv_bfloat16, 256); }
  } else {
    switch (a.head_dim) { case 16: FA_P(__half, 16); case 32: FA_P(__half, 32); case 64: FA_P(__half, 64);
                          case 128: FA_P(__half, 128); case 256: FA_P(__half, 256); }
  }
#undef FA_P
  set_error("head_dim %d not in {16,32,64,128,256}", a.head_dim);
  return FA_ERR_UNSUPPORTED;
}

template <typename T, int D>
static int launch_fwd(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  constexpr int P = TilePitch<D>::value;
  constexpr size_t smem = (size_t)(64 + 4 * 64) * P * sizeof(T);
  auto kern = fwd_mma_kernel<T, D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("fwd_mma: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return FA_ERR_LAUNCH;
    }
  }
  dim3 grid((a.seqlen_q + 63) / 64, a.heads_q, a.batch);
  kern<<<grid, 128, smem, st>>>(a, cfg);
  return check_launch("fwd_mma");
}

template <typename T>
static int dispatch_d(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  switch (a.head_dim) {
    case 16: return launch_fwd<T, 16>(a, cfg, st);
    case 32: return launch_fwd<T, 32>(a, cfg, st);
    case 64: return launch_fwd<T, 64>(a, cfg, st);
    case 128: return launch_fwd<T, 128>(a, cfg, st);
    case 256: return launch_fwd<T, 256>(a, cfg, st);
  }
  set_error("head_dim %d not in {16,32,64,128,256}", a.head_dim);
  return FA_ERR_UNSUPPORTED;
}

int fwd_mma(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen_q == 0 || a.heads_q == 0) return FA_OK;
  return a.dtype == FA_BF16 ? dispatch_d<__nv_bfloat16>(a, cfg, st) : dispatch_d<__half>(a, cfg, st);
}

}  // namespace fa
