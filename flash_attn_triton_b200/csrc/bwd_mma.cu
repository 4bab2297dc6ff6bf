// Backward attention on warp-level tensor-core MMA (mma.sync m16n8k16): the all-shapes
// kernels.  Three launches, no atomics, one writer per output element:
//   preprocess : delta = rowsum(O * dO)
//   dq         : CTA = 64 query rows of one (batch, head); loops key tiles
//   dkdv       : CTA = 64 keys of one (batch, kv head); loops the query heads of the group
//                and their query tiles, working on the TRANSPOSED score tile
//                S^T = K Q^T so that P^T and dS^T feed the next MMA straight from registers.
#include "common.cuh"

namespace fa {

// ---------------------------------------------------------------------------------------
// delta
// ---------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(128) bwd_preprocess_kernel(const fa_attn_args p) {
  constexpr int LPR = D / 8;        // lanes per row (one 16-byte chunk each)
  constexpr int RPW = 32 / LPR;     // rows per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p, b);
  const int row = (blockIdx.x * 4 + warp) * RPW + lane / LPR;
  const int c = lane % LPR;
  float acc = 0.f;
  const bool ok = row < si.q_len;
  if (ok) {
    const T* og = reinterpret_cast<const T*>(p.o) + si.q_boff * p.o_stride[0] +
                  (si.q_row0 + row) * p.o_stride[1] + (int64_t)h * p.o_stride[2] + c * 8;
    const T* dg = reinterpret_cast<const T*>(p.dout) + si.q_boff * p.do_stride[0] +
                  (si.q_row0 + row) * p.do_stride[1] + (int64_t)h * p.do_stride[2] + c * 8;
    uint4 ov = *reinterpret_cast<const uint4*>(og);
    uint4 dv = *reinterpret_cast<const uint4*>(dg);
    const uint32_t* ou = reinterpret_cast<const uint32_t*>(&ov);
    const uint32_t* du = reinterpret_cast<const uint32_t*>(&dv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = Elem<T>::unpack(ou[i]), y = Elem<T>::unpack(du[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int s = LPR / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (ok && c == 0)
    p.delta[si.q_boff * p.lse_stride[0] + (si.q_row0 + row) * p.lse_stride[1] +
            (int64_t)h * p.lse_stride[2]] = acc;
}

// ---------------------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(128) bwd_dq_mma_kernel(const fa_attn_args p, const ScoreCfg cfg) {
  constexpr int BM = 64, BN = 64, P = TilePitch<D>::value, NT = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sdO = sQ + BM * P;
  T* sK = sdO + BM * P;
  T* sV = sK + 2 * BN * P;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int mblk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p, b);
  const int m0 = mblk * BM;
  if (m0 >= si.q_len) return;
  const int hk = h / (p.heads_q / p.heads_kv);
  const T* qg = reinterpret_cast<const T*>(p.q) + si.q_boff * p.q_stride[0] +
                si.q_row0 * p.q_stride[1] + (int64_t)h * p.q_stride[2];
  const T* dog = reinterpret_cast<const T*>(p.dout) + si.q_boff * p.do_stride[0] +
                 si.q_row0 * p.do_stride[1] + (int64_t)h * p.do_stride[2];
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
  load_tile_async<BM, D, NT>(sdO, dog, p.do_stride[1], m0, si.q_len, tid);
  if (n_lo < n_hi) {
    load_tile_async<BN, D, NT>(sK, kg, p.k_stride[1], n_lo * BN, si.k_len, tid);
    load_tile_async<BN, D, NT>(sV, vg, p.v_stride[1], n_lo * BN, si.k_len, tid);
  }
  cp_async_commit();

  const int r0 = m0 + warp * 16 + g;
  float lse[2], dl[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int row = r0 + i * 8;
    bool ok = row < si.q_len;
    int64_t idx = si.q_boff * p.lse_stride[0] + (si.q_row0 + (ok ? row : 0)) * p.lse_stride[1] +
                  (int64_t)h * p.lse_stride[2];
    lse[i] = ok ? p.lse2[idx] : 0.f;
    dl[i] = ok ? p.delta[idx] : 0.f;
  }

  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

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

    float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t aq[4], ad[4];
      const int aoff = (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8;
      ldsm_x4(smem_u32(sQ + aoff), aq[0], aq[1], aq[2], aq[3]);
      ldsm_x4(smem_u32(sdO + aoff), ad[0], ad[1], ad[2], ad[3]);
#pragma unroll
      for (int nb2 = 0; nb2 < BN / 16; ++nb2) {
        const int boff = (nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * P + kk * 16 + ((lane >> 3) & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(cK + boff), b0, b1, b2, b3);
        mma16816<T>(s[2 * nb2], aq, b0, b1);
        mma16816<T>(s[2 * nb2 + 1], aq, b2, b3);
        ldsm_x4(smem_u32(cV + boff), b0, b1, b2, b3);
        mma16816<T>(dp[2 * nb2], ad, b0, b1);
        mma16816<T>(dp[2 * nb2 + 1], ad, b2, b3);
      }
    }
    // dS = P * (dP - delta) * d(softcap)
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int row = r0 + i * 8;
        const int col = n * BN + nb * 8 + 2 * t + (e & 1);
        const bool inside = row < si.q_len && col < si.k_len;
        const float bias = (cfg.bias != nullptr && inside) ? bias_at(cfg, b, h, row, col) : 0.f;
        float th;
        float sc = score_log2(cfg, slope, s[nb][e], row + off, col, th, bias);
        float pv = 0.f;
        if (visible(cfg, row + off, col, si.k_len) && lse[i] != -INFINITY) pv = exp2f(sc - lse[i]);
        // dropout as the reference applies it in its backward (attention_kernel.py:750-762): the
        // dropped-and-rescaled P multiplies (dP - delta)
        if (cfg.dropout_p > 0.f)
          pv = dropout_keep(cfg, (uint32_t)si.q_row0, row, col) ? pv * cfg.dropout_scale : 0.f;
        float ds = pv * (dp[nb][e] - dl[i]);
        if (cfg.softcap > 0.f) ds *= (1.f - th * th);
        s[nb][e] = ds;
      }
    }
    // dQ += dS K
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
        ldsm_x4_t(smem_u32(cK + (kk2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P + db2 * 16 +
                           (lane >> 4) * 8),
                  b0, b1, b2, b3);
        mma16816<T>(dq[2 * db2], a, b0, b1);
        mma16816<T>(dq[2 * db2 + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

#pragma unroll
  for (int nb = 0; nb < D / 8; ++nb) {
    uint32_t v0 = Elem<T>::pack(dq[nb][0] * cfg.scale, dq[nb][1] * cfg.scale);
    uint32_t v1 = Elem<T>::pack(dq[nb][2] * cfg.scale, dq[nb][3] * cfg.scale);
    *reinterpret_cast<uint32_t*>(sQ + (warp * 16 + g) * P + nb * 8 + 2 * t) = v0;
    *reinterpret_cast<uint32_t*>(sQ + (warp * 16 + g + 8) * P + nb * 8 + 2 * t) = v1;
  }
  __syncthreads();
  T* dqg = reinterpret_cast<T*>(p.dq) + si.q_boff * p.dq_stride[0] + si.q_row0 * p.dq_stride[1] +
           (int64_t)h * p.dq_stride[2];
  constexpr int CPR = D / 8;
  for (int i = tid; i < BM * CPR; i += NT) {
    int r = i / CPR, c = i % CPR;
    if (m0 + r < si.q_len)
      *reinterpret_cast<uint4*>(dqg + (int64_t)(m0 + r) * p.dq_stride[1] + c * 8) =
          *reinterpret_cast<const uint4*>(sQ + r * P + c * 8);
  }
}

// ---------------------------------------------------------------------------------------
// dK, dV.  DA = width of the head_dim slice this CTA accumulates (head_dim 256 is done as
// two slices of 128 so the fp32 accumulators fit in registers).
// ---------------------------------------------------------------------------------------
template <typename T, int D, int DA>
__global__ void __launch_bounds__(128) bwd_dkdv_mma_kernel(const fa_attn_args p, const ScoreCfg cfg) {
  constexpr int BM = 64, BN = 64, P = TilePitch<D>::value, NT = 128;
  constexpr int NSLICE = D / DA;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sK = reinterpret_cast<T*>(smem_raw);
  T* sV = sK + BN * P;
  T* sQ = sV + BN * P;           // 2 stages
  T* sdO = sQ + 2 * BM * P;      // 2 stages
  float* sLse = reinterpret_cast<float*>(sdO + 2 * BM * P);  // 2 x BM
  float* sDl = sLse + 2 * BM;                                // 2 x BM

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nblk = blockIdx.x, b = blockIdx.z;
  const int hk = blockIdx.y / NSLICE, dz = blockIdx.y % NSLICE;
  const SeqInfo si = seq_info(p, b);
  const int n0 = nblk * BN;
  if (n0 >= si.k_len) return;
  const int G = p.heads_q / p.heads_kv;
  const int off = p.q_pos_offset;
  const T* kg = reinterpret_cast<const T*>(p.k) + si.k_boff * p.k_stride[0] +
                si.k_row0 * p.k_stride[1] + (int64_t)hk * p.k_stride[2];
  const T* vg = reinterpret_cast<const T*>(p.v) + si.k_boff * p.v_stride[0] +
                si.k_row0 * p.v_stride[1] + (int64_t)hk * p.v_stride[2];

  // query rows that can see this key block
  int qlo, qhi;
  visible_query_range(cfg, n0, min(n0 + BN, si.k_len) - 1, off, si.q_len + off, qlo, qhi);
  const int m_lo = max(qlo - off, 0) / BM;
  const int m_hi = (max(qhi - off, 0) + BM - 1) / BM;
  const int ntiles = max(m_hi - m_lo, 0);
  const int total = ntiles * G;

  auto issue = [&](int it, int st) {
    const int hq = hk * G + it / ntiles;
    const int m = m_lo + it % ntiles;
    const T* qg = reinterpret_cast<const T*>(p.q) + si.q_boff * p.q_stride[0] +
                  si.q_row0 * p.q_stride[1] + (int64_t)hq * p.q_stride[2];
    const T* dog = reinterpret_cast<const T*>(p.dout) + si.q_boff * p.do_stride[0] +
                   si.q_row0 * p.do_stride[1] + (int64_t)hq * p.do_stride[2];
    load_tile_async<BM, D, NT>(sQ + st * BM * P, qg, p.q_stride[1], m * BM, si.q_len, tid);
    load_tile_async<BM, D, NT>(sdO + st * BM * P, dog, p.do_stride[1], m * BM, si.q_len, tid);
    if (tid < BM) {
      int row = m * BM + tid;
      bool ok = row < si.q_len;
      int64_t idx = si.q_boff * p.lse_stride[0] + (si.q_row0 + (ok ? row : 0)) * p.lse_stride[1] +
                    (int64_t)hq * p.lse_stride[2];
      sLse[st * BM + tid] = ok ? p.lse2[idx] : -INFINITY;
      sDl[st * BM + tid] = ok ? p.delta[idx] : 0.f;
    }
  };

  load_tile_async<BN, D, NT>(sK, kg, p.k_stride[1], n0, si.k_len, tid);
  load_tile_async<BN, D, NT>(sV, vg, p.v_stride[1], n0, si.k_len, tid);
  if (total > 0) issue(0, 0);
  cp_async_commit();

  float dk[DA / 8][4], dv[DA / 8][4];
#pragma unroll
  for (int i = 0; i < DA / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  const int key0 = n0 + warp * 16 + g;  // this thread's keys: key0, key0+8

  for (int it = 0; it < total; ++it) {
    const int st = it & 1;
    if (it + 1 < total) {
      issue(it + 1, st ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int hq = hk * G + it / ntiles;
    const int m = m_lo + it % ntiles;
    const float slope = cfg.has_alibi ? p.alibi_slopes[b * p.heads_q + hq] : 0.f;
    const T* cQ = sQ + st * BM * P;
    const T* cdO = sdO + st * BM * P;

    // S^T = K Q^T and dP^T = V dO^T : rows = keys (this warp's 16), cols = 64 query rows
    float s[BM / 8][4], dp[BM / 8][4];
#pragma unroll
    for (int i = 0; i < BM / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t ak[4], av[4];
      const int aoff = (warp * 16 + (lane & 15)) * P + kk * 16 + (lane >> 4) * 8;
      ldsm_x4(smem_u32(sK + aoff), ak[0], ak[1], ak[2], ak[3]);
      ldsm_x4(smem_u32(sV + aoff), av[0], av[1], av[2], av[3]);
#pragma unroll
      for (int nb2 = 0; nb2 < BM / 16; ++nb2) {
        const int boff = (nb2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * P + kk * 16 + ((lane >> 3) & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(cQ + boff), b0, b1, b2, b3);
        mma16816<T>(s[2 * nb2], ak, b0, b1);
        mma16816<T>(s[2 * nb2 + 1], ak, b2, b3);
        ldsm_x4(smem_u32(cdO + boff), b0, b1, b2, b3);
        mma16816<T>(dp[2 * nb2], av, b0, b1);
        mma16816<T>(dp[2 * nb2 + 1], av, b2, b3);
      }
    }
    // P^T (kept in s) and dS^T (kept in dp)
#pragma unroll
    for (int nb = 0; nb < BM / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + (e >> 1) * 8;
        const int qc = nb * 8 + 2 * t + (e & 1);  // query row inside the tile
        const int qrow = m * BM + qc;
        const float l2 = sLse[st * BM + qc];
        const bool inside = qrow < si.q_len && key < si.k_len;
        const float bias = (cfg.bias != nullptr && inside) ? bias_at(cfg, b, hq, qrow, key) : 0.f;
        float th;
        float sc = score_log2(cfg, slope, s[nb][e], qrow + off, key, th, bias);
        float pv = 0.f;
        if (qrow < si.q_len && l2 != -INFINITY && visible(cfg, qrow + off, key, si.k_len))
          pv = exp2f(sc - l2);
        // the same keep mask as in the forward (attention_kernel.py:641-652)
        if (cfg.dropout_p > 0.f)
          pv = dropout_keep(cfg, (uint32_t)si.q_row0, qrow, key) ? pv * cfg.dropout_scale : 0.f;
        float ds = pv * (dp[nb][e] - sDl[st * BM + qc]);
        if (cfg.softcap > 0.f) ds *= (1.f - th * th);
        s[nb][e] = pv;
        dp[nb][e] = ds;
      }
    }
    // dV += P^T dO ; dK += dS^T Q   (k = the tile's 64 query rows)
#pragma unroll
    for (int kk2 = 0; kk2 < BM / 16; ++kk2) {
      uint32_t ap[4], as[4];
      ap[0] = Elem<T>::pack(s[2 * kk2][0], s[2 * kk2][1]);
      ap[1] = Elem<T>::pack(s[2 * kk2][2], s[2 * kk2][3]);
      ap[2] = Elem<T>::pack(s[2 * kk2 + 1][0], s[2 * kk2 + 1][1]);
      ap[3] = Elem<T>::pack(s[2 * kk2 + 1][2], s[2 * kk2 + 1][3]);
      as[0] = Elem<T>::pack(dp[2 * kk2][0], dp[2 * kk2][1]);
      as[1] = Elem<T>::pack(dp[2 * kk2][2], dp[2 * kk2][3]);
      as[2] = Elem<T>::pack(dp[2 * kk2 + 1][0], dp[2 * kk2 + 1][1]);
      as[3] = Elem<T>::pack(dp[2 * kk2 + 1][2], dp[2 * kk2 + 1][3]);
#pragma unroll
      for (int db2 = 0; db2 < DA / 16; ++db2) {
        const int boff = (kk2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P + dz * DA + db2 * 16 +
                         (lane >> 4) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(cdO + boff), b0, b1, b2, b3);
        mma16816<T>(dv[2 * db2], ap, b0, b1);
        mma16816<T>(dv[2 * db2 + 1], ap, b2, b3);
        ldsm_x4_t(smem_u32(cQ + boff), b0, b1, b2, b3);
        mma16816<T>(dk[2 * db2], as, b0, b1);
        mma16816<T>(dk[2 * db2 + 1], as, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // stage dK then dV through the Q stage buffers (pitch P, only DA columns used)
  T* stK = sQ;
  T* stV = sQ + BM * P;
#pragma unroll
  for (int nb = 0; nb < DA / 8; ++nb) {
    const int c = nb * 8 + 2 * t;
    *reinterpret_cast<uint32_t*>(stK + (warp * 16 + g) * P + c) =
        Elem<T>::pack(dk[nb][0] * cfg.scale, dk[nb][1] * cfg.scale);
    *reinterpret_cast<uint32_t*>(stK + (warp * 16 + g + 8) * P + c) =
        Elem<T>::pack(dk[nb][2] * cfg.scale, dk[nb][3] * cfg.scale);
    *reinterpret_cast<uint32_t*>(stV + (warp * 16 + g) * P + c) = Elem<T>::pack(dv[nb][0], dv[nb][1]);
    *reinterpret_cast<uint32_t*>(stV + (warp * 16 + g + 8) * P + c) = Elem<T>::pack(dv[nb][2], dv[nb][3]);
  }
  __syncthreads();
  T* dkg = reinterpret_cast<T*>(p.dk) + si.k_boff * p.dk_stride[0] + si.k_row0 * p.dk_stride[1] +
           (int64_t)hk * p.dk_stride[2] + dz * DA;
  T* dvg = reinterpret_cast<T*>(p.dv) + si.k_boff * p.dv_stride[0] + si.k_row0 * p.dv_stride[1] +
           (int64_t)hk * p.dv_stride[2] + dz * DA;
  constexpr int CPR = DA / 8;
  for (int i = tid; i < BN * CPR; i += NT) {
    int r = i / CPR, c = i % CPR;
    if (n0 + r < si.k_len) {
      *reinterpret_cast<uint4*>(dkg + (int64_t)(n0 + r) * p.dk_stride[1] + c * 8) =
          *reinterpret_cast<const uint4*>(stK + r * P + c * 8);
      *reinterpret_cast<uint4*>(dvg + (int64_t)(n0 + r) * p.dv_stride[1] + c * 8) =
          *reinterpret_cast<const uint4*>(stV + r * P + c * 8);
    }
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
template <typename K> static int set_smem(K kern, size_t smem, const char* what) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("%s: cudaFuncSetAttribute(%zu): %s", what, smem, cudaGetErrorString(e));
      return FA_ERR_LAUNCH;
    }
  }
  return FA_OK;
}

template <typename T, int D> static int launch_pre(const fa_attn_args& a, cudaStream_t st) {
  constexpr int RPB = 4 * (32 / (D / 8));
  dim3 grid((a.seqlen_q + RPB - 1) / RPB, a.heads_q, a.batch);
  bwd_preprocess_kernel<T, D><<<grid, 128, 0, st>>>(a);
  return check_launch("bwd_preprocess");
}
template <typename T, int D> static int launch_dq(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  constexpr size_t smem = (size_t)(2 * 64 + 4 * 64) * TilePitch<D>::value * sizeof(T);
  auto kern = bwd_dq_mma_kernel<T, D>;
  if (int r = set_smem(kern, smem, "bwd_dq_mma")) return r;
  dim3 grid((a.seqlen_q + 63) / 64, a.heads_q, a.batch);
  kern<<<grid, 128, smem, st>>>(a, cfg);
  return check_launch("bwd_dq_mma");
}
template <typename T, int D> static int launch_dkdv(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  constexpr int DA = D > 128 ? 128 : D;
  constexpr size_t smem = (size_t)(2 * 64 + 4 * 64) * TilePitch<D>::value * sizeof(T) + 4 * 64 * sizeof(float);
  auto kern = bwd_dkdv_mma_kernel<T, D, DA>;
  if (int r = set_smem(kern, smem, "bwd_dkdv_mma")) return r;
  dim3 grid((a.seqlen_k + 63) / 64, a.heads_kv * (D / DA), a.batch);
  kern<<<grid, 128, smem, st>>>(a, cfg);
  return check_launch("bwd_dkdv_mma");
}

#define FA_DISPATCH_D(FN, ...)                                        \
  switch (a.head_dim) {                                               \
    case 16: return FN<T, 16>(__VA_ARGS__);                           \
    case 32: return FN<T, 32>(__VA_ARGS__);                           \
    case 64: return FN<T, 64>(__VA_ARGS__);                           \
    case 128: return FN<T, 128>(__VA_ARGS__);                         \
    case 256: return FN<T, 256>(__VA_ARGS__);                         \
  }                                                                   \
  set_error("head_dim %d not in {16,32,64,128,256}", a.head_dim);     \
  return FA_ERR_UNSUPPORTED;

template <typename T> static int pre_t(const fa_attn_args& a, cudaStream_t st) { FA_DISPATCH_D(launch_pre, a, st) }
template <typename T> static int dq_t(const fa_attn_args& a, const ScoreCfg& c, cudaStream_t st) { FA_DISPATCH_D(launch_dq, a, c, st) }
template <typename T> static int dkdv_t(const fa_attn_args& a, const ScoreCfg& c, cudaStream_t st) { FA_DISPATCH_D(launch_dkdv, a, c, st) }

int bwd_preprocess(const fa_attn_args& a, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen_q == 0 || a.heads_q == 0) return FA_OK;
  return a.dtype == FA_BF16 ? pre_t<__nv_bfloat16>(a, st) : pre_t<__half>(a, st);
}
int bwd_dq_mma(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen_q == 0 || a.heads_q == 0) return FA_OK;
  return a.dtype == FA_BF16 ? dq_t<__nv_bfloat16>(a, cfg, st) : dq_t<__half>(a, cfg, st);
}
int bwd_dkdv_mma(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen_k == 0 || a.heads_kv == 0) return FA_OK;
  return a.dtype == FA_BF16 ? dkdv_t<__nv_bfloat16>(a, cfg, st) : dkdv_t<__half>(a, cfg, st);
}

}  // namespace fa
