// dK, dV with one CTA per block of 128 keys (grid = key blocks x kv heads x batch): the roles of
// the persistent kernel of bwd_sm100.cu without its work queue, and with K kept in shared memory so
// that P^T and dS^T each have tensor-memory columns of their own.  Measured on B200 it is the
// faster of the two on every plain dense shape (2-7 % without a mask, 10-15 % with the causal mask
// or GQA); the host side of bwd_sm100.cu sends those here and packed batches and the ALiBi /
// soft-cap variants to the persistent kernel.
//
//   CTA = 128 keys of one (batch, kv head); loops over the query tiles (and the query heads of the
//   GQA group) that can see them, on the TRANSPOSED tiles S^T = K Q^T, dP^T = V dO^T so that a TMEM
//   lane is a key; P^T and dS^T go back to TMEM and feed dV += P^T dO, dK += dS^T Q as the A operand.
//   Row statistics (-lse2, -delta) ride in the GEMMs through 16-column operand tiles.
//   TMEM: R (128 fp32 columns: S^T, then dP^T) | P^T (64) | dS^T (64) | dV (128) | dK (128); K and V
//   stay in shared memory.
#include <cstddef>
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace fa {

using namespace sm100;

__device__ int g_bwd_cta_status = 0;

namespace {

constexpr int kT = 128;        // tile edge: rows of Q / keys of K,V per tile
constexpr int kHalfT = 64;     // columns per element-wise group
constexpr int kBwdThreads = 384;
// Register re-balancing (setmaxnreg): the CTA starts with 168 registers per thread; the four
// service warps drop to kRegsService and the eight element-wise warps grow to kRegsEw.
// setmaxnreg.inc blocks until the registers exist, so the split has to satisfy
// (kRegsEw - 168) * 256 <= (168 - kRegsService) * 128.
constexpr int kRegsService = 88, kRegsEw = 208;
// Share of the exponentials of the unmasked fast path that run on the FMA pipe (every n-th).
#ifndef FA_POLY_BWD
#define FA_POLY_BWD 0
#endif
constexpr int kPolyEvery = FA_POLY_BWD;
static_assert((kRegsEw - 168) * 256 <= (168 - kRegsService) * 128, "register split");

template <int D> struct BCfg {
  static constexpr int kTileBytes = kT * D * 2;
  static constexpr int kBoxes = D / 64;
  // dK/dV kernel: V and K resident, a ring of Q tiles (Q(i) lives from S(i) to dK(i)) and a ring of
  // dO tiles (dO(i) from dP(i) to dV(i)).
  static constexpr int kStagesQ = (D == 128) ? 2 : 3;
  static constexpr int kStagesO = (D == 128) ? 2 : 4;
  static constexpr int kSmemTiles = (2 + kStagesQ + kStagesO) * kTileBytes;
  // dK/dV kernel: 128 x 16 operand tiles that carry the row statistics into the GEMMs
  // (two constant ones on the key side, one per ring stage on the query side)
  static constexpr int kAugBytes = kT * 16 * 2;
  static constexpr int kAugTotal = (2 + kStagesQ) * kAugBytes;
  static constexpr int kSmemBytes = kSmemTiles + kAugTotal + 1024 + 8192;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  // dQ kernel: the K ring is one stage deeper than the V ring.  K(k+1) is needed by S(k+1) at
  // the START of step k while K(k) is still read by dQ(k) at its end; with two stages the slot
  // of K(k+1) is only freed by dQ(k-1), and the load's latency landed on the critical path.
  // This kernel only touches the barriers of BShared (512 bytes), not its statistics arrays.
  static constexpr int kStagesK = (D == 128) ? 3 : 4;
  static constexpr int kStagesV = (D == 128) ? 2 : 4;
  static constexpr int kSmemTilesDq = (2 + kStagesK + kStagesV) * kTileBytes;
  static constexpr int kSmemBytesDq = kSmemTilesDq + 1024 + 512;
  static_assert(kSmemBytesDq <= 227 * 1024, "shared memory budget (dQ)");
};

struct BShared {
  uint64_t res_full;      // resident tiles (K,V or Q,dO) landed
  uint64_t full_a[4];     // streamed tile A (Q in dK/dV, K in dQ) landed
  uint64_t full_b[4];     // streamed tile B (dO in dK/dV, V in dQ) landed
  uint64_t empty_a[4];    // last MMA reading tile A (and its statistics) finished
  uint64_t empty_b[4];    // last MMA reading tile B finished
  uint64_t stat_full[4];  // statistics of the streamed query tile written (dK/dV kernel)
  uint64_t s_full[2];     // S computed ([buffer] in the dQ kernel, [0] in the dK/dV kernel)
  uint64_t dp_full;       // dP computed
  uint64_t p_ready;       // P written back (256 arrivals; dK/dV kernel)
  uint64_t ds_ready;      // dS written back (256 arrivals)
  uint64_t r_free;        // dK/dV kernel: scores, then dP, read out of their shared TMEM region (256 arrivals)
  uint64_t p_free;        // dK/dV kernel: dV MMA that read P finished
  uint64_t ds_free;       // dK/dV kernel: dK MMA that read dS finished
  uint64_t acc_done;      // every accumulation MMA finished
  uint32_t tmem_base;
  volatile int abort_flag;
  alignas(16) float lse[4][kT];  // [stage][row of the streamed query tile]: MINUS the base-2 LSE
  alignas(16) float delta[4][kT];  //                                       MINUS delta
};
static_assert(sizeof(BShared) <= 8192, "BShared must fit its reserve");
static_assert(offsetof(BShared, lse) <= 512, "the dQ kernel reserves 512 bytes for the barriers");

template <typename T> struct BFmt;
template <> struct BFmt<__half> { static constexpr int code = 0; };
template <> struct BFmt<__nv_bfloat16> { static constexpr int code = 1; };

__device__ __forceinline__ bool bwait(uint64_t* bar, uint32_t parity, BShared* sh, int code) {
  return bounded_wait(bar, parity, &sh->abort_flag, &g_bwd_cta_status, code);
}

// For roles that are far ahead of the critical path (producer, statistics loader): back off
// between polls so the spin does not take issue slots from the element-wise warps.
__device__ __forceinline__ bool bwait_relaxed(uint64_t* bar, uint32_t parity, BShared* sh, int code) {
  const uint32_t a = smem_u32(bar);
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait(a, parity)) return true;
    __nanosleep(100);
  }
  return bwait(bar, parity, sh, code);
}

// TMA loads of one 128 x D tile (D/64 boxes) at (row, head, batch)
template <int D>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int row,
                                          int head, int batch) {
#pragma unroll
  for (int x = 0; x < D / 64; ++x) tma_load_4d(dst + x * (kT * 128), tm, bar, x * 64, head, row, batch);
}

// 128 x 128 x D product of two K-major tiles (contraction over head_dim): D/16 MMAs.
// Whole warp, uniform control flow; the lane with leader != 0 issues.
template <int D>
__device__ __forceinline__ void mma_kmajor(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem,
                                           uint32_t idesc, uint32_t leader) {
  const uint64_t da = make_smem_desc(a_smem, 16, 1024), db = make_smem_desc(b_smem, 16, 1024);
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t o = ((kk / 4) * (kT * 128) + (kk % 4) * 32) >> 4;
    mma_f16_ss_lp(d_tmem, da + o, db + o, idesc, kk > 0, leader);
  }
}

// 128 x 128 x D product with A (128 rows x D, 16-bit pairs, D/2 columns) in TMEM and B a K-major tile.
template <int D>
__device__ __forceinline__ void mma_kmajor_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem,
                                              uint32_t idesc, uint32_t leader) {
  const uint64_t db = make_smem_desc(b_smem, 16, 1024);
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t o = ((kk / 4) * (kT * 128) + (kk % 4) * 32) >> 4;
    mma_f16_ts_lp(d_tmem, a_tmem + kk * 8, db + o, idesc, kk > 0, leader);
  }
}

// acc(128 x D) += A(128 x 128, fp16 pairs in TMEM) * B(128 rows x D, MN-major smem tile).
// A is stored as two 32-column blocks (written by the two element-wise groups) at
// a_tmem and a_tmem + kGroupStride.
template <int D, int kGroupStride = 64>
__device__ __forceinline__ void mma_from_tmem(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem,
                                              uint32_t idesc, bool accumulate, uint32_t leader) {
  const uint64_t db = make_smem_desc(b_smem, kT * 128, 1024);
#pragma unroll
  for (int kk = 0; kk < kT / 16; ++kk) {
    const uint32_t a = a_tmem + (kk / 4) * kGroupStride + (kk % 4) * 8;
    mma_f16_ts_lp(d_tmem, a, db + ((kk * 2048) >> 4), idesc, (accumulate || kk > 0) ? 1u : 0u, leader);
  }
}

}  // namespace

// =======================================================================================
// dK, dV
// =======================================================================================
template <typename T, int D, bool kExtras>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_cta_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                      const fa_attn_args p, const ScoreCfg cfg, int* const host_status) {
  using C = BCfg<D>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  BShared* sh = reinterpret_cast<BShared*>(tiles + C::kSmemTiles + C::kAugTotal);
  const uint32_t sV = smem_u32(tiles), sK = sV + C::kTileBytes;
  const uint32_t sRingQ = sK + C::kTileBytes, sRingO = sRingQ + C::kStagesQ * C::kTileBytes;
  // statistics operands: [0] key side of the score GEMM, [1] key side of the dP GEMM,
  // [2 + stage] query side (written per streamed query tile by the statistics warp)
  unsigned char* aug = tiles + C::kSmemTiles;
  const uint32_t sAug = sV + C::kSmemTiles;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const SeqInfo si = seq_info(p, b);
  const int n0 = nblk * kT;
  if (n0 >= si.k_len) return;
  const int G = p.heads_q / p.heads_kv;
  const int off = p.q_pos_offset;

  int qlo, qhi;
  visible_query_range(cfg, n0, min(n0 + kT, si.k_len) - 1, off, si.q_len + off, qlo, qhi);
  const int m_lo = max(qlo - off, 0) / kT;
  const int m_hi = (max(qhi - off, 0) + kT - 1) / kT;
  const int ntiles = max(m_hi - m_lo, 0);
  const int total = ntiles * G;

  if (tid == 0) {
    mbar_init(smem_u32(&sh->res_full), 1);
    mbar_init(smem_u32(&sh->s_full[0]), 1);
    mbar_init(smem_u32(&sh->s_full[1]), 1);
    mbar_init(smem_u32(&sh->dp_full), 1);
    mbar_init(smem_u32(&sh->p_ready), 256);
    mbar_init(smem_u32(&sh->ds_ready), 256);
    mbar_init(smem_u32(&sh->r_free), 256);
    mbar_init(smem_u32(&sh->p_free), 1);
    mbar_init(smem_u32(&sh->ds_free), 1);
    mbar_init(smem_u32(&sh->acc_done), 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&sh->full_a[i]), 2);   // the TMA load of Q and the statistics warp
      mbar_init(smem_u32(&sh->full_b[i]), 1);
      mbar_init(smem_u32(&sh->empty_a[i]), 2);  // one commit from each of the two issuer warps
      mbar_init(smem_u32(&sh->empty_b[i]), 2);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  {
    // Statistics operands, no-swizzle K-major layout: columns 0-7 of row r at
    // (r / 8) * 128 + (r % 8) * 16, columns 8-15 (always zero) 2048 bytes further.
    // Query side, per row:  [l_hi, l_hi, l_lo, l_lo, d_hi, d_lo, 0, 0]  with l = -lse2, d = -delta
    // key side, scores:     [w_hi, w_lo, w_hi, w_lo, 0, 0, 0, 0]        with w = 1 / scale_log2
    // key side, dP:         [0, 0, 0, 0, 1, 1, 0, 0]
    // so the score GEMM yields S - lse2 / scale_log2 and the dP GEMM dP - delta.
    const float w = 1.f / cfg.scale_log2;
    const T w_hi = Elem<T>::from_f(w), w_lo = Elem<T>::from_f(w - Elem<T>::to_f(w_hi));
    const uint32_t wp = (uint32_t)(*reinterpret_cast<const uint16_t*>(&w_hi)) |
                        ((uint32_t)(*reinterpret_cast<const uint16_t*>(&w_lo)) << 16);
    const uint32_t ones = Elem<T>::pack(1.f, 1.f);
    uint4* a4 = reinterpret_cast<uint4*>(aug);
    for (int i = tid; i < C::kAugTotal / 16; i += kBwdThreads) {
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (i < kT) val = make_uint4(wp, wp, 0u, 0u);
      else if (i >= C::kAugBytes / 16 && i < C::kAugBytes / 16 + kT) val = make_uint4(0u, 0u, ones, 0u);
      a4[i] = val;
    }
    fence_proxy_async();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  // TMEM: R (128 fp32 columns: S^T, then dP^T of a tile) | P^T (64) | dS^T (64) | dV | dK
  const uint32_t tR = tmem, tXp = tmem + 128, tXs = tmem + 192, tdV = tmem + 256, tdK = tmem + 384;

  if (warp == 8) {
    // ------------------------------- TMA producer ---------------------------------------
    reg_dealloc<kRegsService>();
    if (lane == 0 && total > 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      prefetch_tmap(&tmdO);
      {
        const uint32_t bar = smem_u32(&sh->res_full);
        mbar_expect_tx(bar, 2 * C::kTileBytes);
        load_tile<D>(sK, &tmK, bar, (int)si.k_row0 + n0, hk, (int)si.k_boff);
        load_tile<D>(sV, &tmV, bar, (int)si.k_row0 + n0, hk, (int)si.k_boff);
      }
      for (int it = 0; it < total; ++it) {
        const int hq = hk * G + it / ntiles, m = m_lo + it % ntiles;
        const int sq = it % C::kStagesQ, so = it % C::kStagesO;
        // Q's slot frees after dK of the tile that held it
        if (!bwait_relaxed(&sh->empty_a[sq], ((it / C::kStagesQ) & 1) ^ 1, sh, 41)) break;
        {
          const uint32_t bar = smem_u32(&sh->full_a[sq]);
          mbar_expect_tx(bar, C::kTileBytes);
          load_tile<D>(sRingQ + sq * C::kTileBytes, &tmQ, bar, (int)si.q_row0 + m * kT, hq, (int)si.q_boff);
        }
        if (!bwait_relaxed(&sh->empty_b[so], ((it / C::kStagesO) & 1) ^ 1, sh, 41)) break;
        {
          const uint32_t bar = smem_u32(&sh->full_b[so]);
          mbar_expect_tx(bar, C::kTileBytes);
          load_tile<D>(sRingO + so * C::kTileBytes, &tmdO, bar, (int)si.q_row0 + m * kT, hq, (int)si.q_boff);
        }
      }
    }
  } else if (warp == 10) {
    // ------------------------------- statistics loader ----------------------------------
    // The loads of tile it+1 are ISSUED right after tile it has been written and only consumed
    // after the wait for the next slot, so their latency hides behind that wait (nothing reads
    // the registers in between: a scoreboard stall before the poll would serialise the two).
    reg_dealloc<kRegsService>();
    int stage = 0;
    uint32_t phase = 0;
    float rl[kT / 32], rd[kT / 32];                  // statistics of rows lane, lane + 32, ... as loaded
    auto fetch = [&](int it) {
      const int hq = hk * G + it / ntiles, m = m_lo + it % ntiles;
#pragma unroll
      for (int k = 0; k < kT / 32; ++k) {
        const int row = m * kT + lane + 32 * k;
        rl[k] = INFINITY;
        rd[k] = 0.f;
        if (row < si.q_len) {
          const int64_t idx = si.q_boff * p.lse_stride[0] + (si.q_row0 + row) * p.lse_stride[1] +
                              (int64_t)hq * p.lse_stride[2];
          rl[k] = p.lse2[idx];
          rd[k] = p.delta[idx];
        }
      }
    };
    if (total > 0) fetch(0);
    for (int it = 0; it < total; ++it) {
      bool w = true;
      if (lane == 0) w = bwait_relaxed(&sh->empty_a[stage], phase ^ 1, sh, 42);
      if (!__all_sync(0xffffffffu, w)) break;
      uint4* q4 = reinterpret_cast<uint4*>(aug + (2 + stage) * C::kAugBytes);
#pragma unroll
      for (int k = 0; k < kT / 32; ++k) {
        const int i = lane + 32 * k;
        // NEGATED; rows that do not exist or see no key get a large finite value instead of
        // infinity (an infinity would meet the zeros of the other GEMM's key-side operand): P = 0
        float nl2 = -rl[k];
        const float ndl = fminf(fmaxf(-rd[k], -60000.f), 60000.f);   // kept inside the 16-bit range
        if (!(fabsf(nl2) < 60000.f)) nl2 = -60000.f;
        // the feature variant adds the LSE after the soft cap, in the element-wise warps
        if (kExtras) sh->lse[stage][i] = nl2 == -60000.f ? -INFINITY : nl2;
        const float lf = kExtras ? 0.f : nl2;
        const T l_hi = Elem<T>::from_f(lf), l_lo = Elem<T>::from_f(lf - Elem<T>::to_f(l_hi));
        const T d_hi = Elem<T>::from_f(ndl), d_lo = Elem<T>::from_f(ndl - Elem<T>::to_f(d_hi));
        const uint32_t lh = *reinterpret_cast<const uint16_t*>(&l_hi), ll = *reinterpret_cast<const uint16_t*>(&l_lo);
        const uint32_t dh = *reinterpret_cast<const uint16_t*>(&d_hi), dl = *reinterpret_cast<const uint16_t*>(&d_lo);
        q4[i] = make_uint4(lh | (lh << 16), ll | (ll << 16), dh | (dl << 16), 0u);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->full_a[stage]));
      if (++stage == C::kStagesQ) { stage = 0; phase ^= 1; }
      if (it + 1 < total) fetch(it + 1);
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -----------------------------------------
    reg_dealloc<kRegsService>();
    if (total > 0) {
      constexpr uint32_t idesc_s = make_idesc(1, BFmt<T>::code, 0, 0, kT, kT);
      constexpr uint32_t idesc_acc = make_idesc(1, BFmt<T>::code, 0, 1, kT, D);
      const uint32_t leader = elect_one() ? 1u : 0u;
      bool ok = true;
      // every lane polls (uniform control flow, no vote needed: a completed phase is seen by all)
      auto wq = [&](uint64_t* bar, uint32_t parity, int code) {
        if (ok) ok = bwait(bar, parity, sh, code);
        tc_fence_after();
      };
      auto slotQ = [&](int it) { return sRingQ + (it % C::kStagesQ) * C::kTileBytes; };
      auto slotO = [&](int it) { return sRingO + (it % C::kStagesO) * C::kTileBytes; };
      auto stat_desc = [&](int it) {
        return make_smem_desc_noswizzle(sAug + (2 + it % C::kStagesQ) * C::kAugBytes, 2048, 128);
      };
      const uint64_t dstat_s = make_smem_desc_noswizzle(sAug, 2048, 128);
      const uint64_t dstat_dp = make_smem_desc_noswizzle(sAug + C::kAugBytes, 2048, 128);
      // S^T(i) = K Q(i)^T - lse2 / scale_log2; waits for Q(i) and its statistics
      auto issue_s = [&](int i) {
        const int st = i % C::kStagesQ;
        const uint32_t ph = (i / C::kStagesQ) & 1;
        wq(&sh->full_a[st], ph, 44);
        if (i > 0) wq(&sh->r_free, 1, 49);                                     // dP(i-1) read out
        if (!ok) return;
        mma_kmajor<D>(tR, sK, slotQ(i), idesc_s, leader);
        if (!kExtras) mma_f16_ss_lp(tR, dstat_s, stat_desc(i), idesc_s, 1u, leader);
        mma_commit_lp(smem_u32(&sh->s_full[0]), leader);
      };
      // This warp issues the GEMMs into the fp32 region R: dP(i), then S(i+1) -- each once the
      // element-wise warps have read its predecessor out of R (r_free).  Warp 11 issues the
      // accumulating GEMMs dV(i), dK(i) that read P, dS from region X.  The exp2 phase of tile
      // i+1 runs under dK(i), dP(i+1); its dS phase under dV(i+1), S(i+2).
      wq(&sh->res_full, 0, 43);
      issue_s(0);
      for (int i = 0; i < total && ok; ++i) {
        const int st = i % C::kStagesQ, so = i % C::kStagesO;
        wq(&sh->full_b[so], (i / C::kStagesO) & 1, 44);
        wq(&sh->r_free, 0, 49);                                                // S(i) read out
        if (!ok) break;
        mma_kmajor<D>(tR, sV, slotO(i), idesc_s, leader);                      // dP^T(i) = V dO(i)^T
        mma_f16_ss_lp(tR, dstat_dp, stat_desc(i), idesc_s, 1u, leader);        //           - delta
        mma_commit_lp(smem_u32(&sh->dp_full), leader);
        mma_commit_lp(smem_u32(&sh->empty_b[so]), leader);   // this warp's last reads of dO(i) and of
        mma_commit_lp(smem_u32(&sh->empty_a[st]), leader);   // Q(i) and its statistics
        if (i + 1 < total) issue_s(i + 1);
      }
      __syncwarp();
    }
  } else if (warp == 11) {
    // ------------------------------- MMA issuer, accumulations --------------------------
    reg_dealloc<kRegsService>();
    if (total > 0) {
      constexpr uint32_t idesc_acc = make_idesc(1, BFmt<T>::code, 0, 1, kT, D);
      const uint32_t leader = elect_one() ? 1u : 0u;
      bool ok = true;
      auto wq = [&](uint64_t* bar, uint32_t parity, int code) {
        if (ok) ok = bwait(bar, parity, sh, code);
        tc_fence_after();
      };
      for (int i = 0; i < total && ok; ++i) {
        const int st = i % C::kStagesQ, so = i % C::kStagesO;
        // dO(i) may land after P(i) is ready; Q(i) has been read by S(i) long before dS(i) exists
        wq(&sh->full_b[so], (i / C::kStagesO) & 1, 44);
        wq(&sh->p_ready, i & 1, 45);
        // Both accumulations are issued once dS(i) is stored: S(i+1), which the other issuer queues as
        // soon as dP(i) has been read, then runs ahead of dV(i), and the element-wise warps find
        // their next scores ready (P and dS have regions of their own, so nothing waits for dV).
        wq(&sh->ds_ready, i & 1, 46);
        if (!ok) break;
        // dK first: it releases the Q slot, and the two-stage Q ring needs that slot back for Q(i+2)
        // well before S(i+2); dO(i)'s slot is not wanted before dP(i+2)
        mma_from_tmem<D, 32>(tdK, tXs, sRingQ + st * C::kTileBytes, idesc_acc, i > 0, leader); // dK += dS(i)^T Q(i)
        mma_commit_lp(smem_u32(&sh->empty_a[st]), leader);
        mma_commit_lp(smem_u32(&sh->ds_free), leader);
        mma_from_tmem<D, 32>(tdV, tXp, sRingO + so * C::kTileBytes, idesc_acc, i > 0, leader); // dV += P(i)^T dO(i)
        mma_commit_lp(smem_u32(&sh->empty_b[so]), leader);
        mma_commit_lp(smem_u32(&sh->p_free), leader);
      }
      mma_commit_lp(smem_u32(&sh->acc_done), leader);
      __syncwarp();
    }
  } else {
    // ------------------------------- element-wise groups --------------------------------
    reg_alloc<kRegsEw>();
    const int x = warp >> 2;                         // column half
    const int lrow = (warp & 3) * 32 + lane;         // TMEM lane = key inside the tile
    const int key = n0 + lrow;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tRx = tR + lane_addr + x * kHalfT;            // fp32 scores / dP: this group's 64 columns
    const uint32_t tXpx = tXp + lane_addr + x * (kHalfT / 2);    // P^T as 16-bit pairs: 32 columns
    const uint32_t tXsx = tXs + lane_addr + x * (kHalfT / 2);    // dS^T, a region of its own
    bool ok = true;
    for (int it = 0; it < total && ok; ++it) {
      const int stage = it % C::kStagesQ;
      const int hq = hk * G + it / ntiles, m = m_lo + it % ntiles;
      const int q0 = m * kT + x * kHalfT;            // first query row of this thread's columns
      const float slope = (kExtras && cfg.has_alibi) ? p.alibi_slopes[b * p.heads_q + hq] : 0.f;
      bool masked = false;
      if (cfg.causal) masked |= (n0 + kT - 1 > q0 + off);
      if (cfg.wl >= 0) masked |= (n0 < q0 + kHalfT - 1 + off - cfg.wl);
      if (cfg.wr >= 0) masked |= (n0 + kT - 1 > q0 + off + cfg.wr);

      // Only the feature path still needs the LSE per column (it is added after the soft cap);
      // it is fetched into registers BEFORE the wait for the scores: shared-memory loads issued
      // while the tensor pipe streams its operands take hundreds of cycles, and here that
      // latency hides behind the wait.  Otherwise the GEMMs deliver S - lse and dP - delta.
      float st[kHalfT];                              // -lse, later the soft cap's tanh factor
      if (kExtras) {
        ok = bwait(&sh->full_a[stage], (it / C::kStagesQ) & 1, sh, 47);
        if (!ok) break;
        const float4* L4 = reinterpret_cast<const float4*>(&sh->lse[stage][x * kHalfT]);
#pragma unroll
        for (int i4 = 0; i4 < kHalfT / 4; ++i4) {
          const float4 l4 = L4[i4];
          st[i4 * 4] = l4.x; st[i4 * 4 + 1] = l4.y; st[i4 * 4 + 2] = l4.z; st[i4 * 4 + 3] = l4.w;
        }
      }
      ok = bwait(&sh->s_full[0], it & 1, sh, 46);
      if (!ok) break;
      tc_fence_after();

      // ---- exp phase: P = exp2(score - lse), written back over S as T pairs -------------
      uint32_t r0[32], r1[32];
      tmem_ld32(tRx, r0);
      tmem_ld32(tRx + 32, r1);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->r_free));            // the scores are in registers: dP may take the region
      float pf[kHalfT];                              // P in fp32, kept for the dS phase
      const float dist0 = (float)(q0 + off - key);   // query position - key position of column 0
      int vq_lo, vq_hi;
      visible_q_interval(cfg, key, vq_lo, vq_hi);
      const ColMask cm = make_col_mask(vq_lo - (q0 + off), vq_hi - (q0 + off));
      auto exp_body = [&](auto slow_tag) {
        constexpr bool kSlow = decltype(slow_tag)::value;
        if (kSlow) {
#pragma unroll
          for (int i = 0; i < kHalfT; ++i) {
            const float sv = __uint_as_float(i < 32 ? r0[i & 31] : r1[i & 31]);
            float th = 0.f;
            float sc;
            if (kExtras) sc = score_log2_dist(cfg, slope, sv, dist0 + (float)i, th) + st[i];
            else sc = sv * cfg.scale_log2;
            float pe = ex2(sc);
            if (masked) pe = col_visible(cm, i) ? pe : 0.f;
            pf[i] = pe;
            // the tanh factor of the soft cap is folded into the copy kept for dS
            if (kExtras && cfg.softcap > 0.f) st[i] = 1.f - th * th;
          }
        } else {
          const float2 c2 = make_float2(cfg.scale_log2, cfg.scale_log2);
#pragma unroll
          for (int i = 0; i < kHalfT; i += 2) {
            const uint32_t* rr = i < 32 ? r0 : r1;
            const float2 a = f2mul(make_float2(__uint_as_float(rr[i & 31]), __uint_as_float(rr[(i & 31) + 1])), c2);
            const float2 pe = ex2_pair<kPolyEvery>(a, i >> 1);
            pf[i] = pe.x;
            pf[i + 1] = pe.y;
          }
        }
      };
      if (kExtras || masked) exp_body(std::true_type{});
      else exp_body(std::false_type{});
      // the P region holds P(it-1) until its dV MMA has finished (p_free): long ago by now
      if (it > 0) {
        ok = bwait(&sh->p_free, (it - 1) & 1, sh, 51);
        if (!ok) break;
        tc_fence_after();
      }
      {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = Elem<T>::pack(pf[c * 32 + 2 * i], pf[c * 32 + 2 * i + 1]);
          tmem_st16(tXpx + c * 16, pk);
        }
      }
      if (kExtras && cfg.softcap > 0.f) {
#pragma unroll
        for (int i = 0; i < kHalfT; ++i) pf[i] *= st[i];
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->p_ready));

      // ---- dS phase: dS = P (dP - delta), written back over dP ---------------------------
      ok = bwait(&sh->dp_full, it & 1, sh, 48);
      if (!ok) break;
      tc_fence_after();
      tmem_ld32(tRx, r0);
      tmem_ld32(tRx + 32, r1);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->r_free));            // dP is in registers: the next S may take the region
      uint32_t pk0[16], pk1[16];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int e = 2 * i;
        const uint32_t* rr = e < 32 ? r0 : r1;
        const float2 ds = f2mul(make_float2(pf[e], pf[e + 1]),
                                make_float2(__uint_as_float(rr[e & 31]), __uint_as_float(rr[(e & 31) + 1])));
        if (i < 16) pk0[i] = Elem<T>::pack(ds.x, ds.y);
        else pk1[i - 16] = Elem<T>::pack(ds.x, ds.y);
      }
      // the dS region holds dS(it-1) until its dK MMA has finished (ds_free): dS does not wait for
      // the dV MMA of this tile, which still reads P from the other region
      if (it > 0) {
        ok = bwait(&sh->ds_free, (it - 1) & 1, sh, 50);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st16(tXsx, pk0);
      tmem_st16(tXsx + 16, pk1);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->ds_ready));
    }

    // ---- epilogue: group A stores dV, group B stores dK * softmax_scale -------------------
    // Each group stages its tile in shared memory (dV over V, dK over a Q slot: every MMA is done) in
    // the swizzled box layout and lets the TMA unit write full rows; a packed tile that reaches
    // past the end of its sequence is stored row by row instead.
    if (ok && total > 0) ok = bwait(&sh->acc_done, 0, sh, 49);
    if (ok) {
      tc_fence_after();
      const uint32_t tsrc = (x == 0 ? tdV : tdK) + lane_addr;
      const float mul = (x == 0) ? 1.f : cfg.scale;
      const bool via_tma = (p.cu_seqlens_k == nullptr) || (n0 + kT <= si.k_len);
      const uint32_t stg = (x == 0) ? sV : sRingQ;   // dV over V, dK over the first Q slot
      T* base = (x == 0) ? reinterpret_cast<T*>(p.dv) + si.k_boff * p.dv_stride[0] +
                               (si.k_row0 + key) * p.dv_stride[1] + (int64_t)hk * p.dv_stride[2]
                         : reinterpret_cast<T*>(p.dk) + si.k_boff * p.dk_stride[0] +
                               (si.k_row0 + key) * p.dk_stride[1] + (int64_t)hk * p.dk_stride[2];
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r[32];
        if (total > 0) {
          tmem_ld32(tsrc + cc * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = Elem<T>::pack(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
          v.y = Elem<T>::pack(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
          v.z = Elem<T>::pack(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
          v.w = Elem<T>::pack(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
          if (via_tma) {
            const int col = cc * 32 + i;
            st_shared_v4(sw128_addr(stg + (col / 64) * (kT * 128), lrow, (col % 64) / 8), v);
          } else if (key < si.k_len) {
            *reinterpret_cast<uint4*>(base + cc * 32 + i) = v;
          }
        }
      }
      if (via_tma) {
        fence_proxy_async();
        if (x == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
        else asm volatile("bar.sync 2, 128;\n" ::: "memory");
        if ((tid & 127) == 0) {
          const CUtensorMap* tm = (x == 0) ? &tmdV : &tmdK;
#pragma unroll
          for (int bx = 0; bx < D / 64; ++bx)
            tma_store_4d(tm, stg + bx * (kT * 128), bx * 64, hk, (int)si.k_row0 + n0, (int)si.k_boff);
          tma_store_commit();
          tma_store_wait_read();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
  if (tid == 0) report_abort(sh->abort_flag, host_status);
}


// =======================================================================================
// host side
// =======================================================================================
namespace {

bool make_map4(CUtensorMap* m, const void* base, const int64_t* stride, int rows, int heads, int batch,
               int D, bool packed) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)rows, (uint64_t)(packed ? 1 : batch)};
  const uint64_t strides[3] = {(uint64_t)stride[2] * 2, (uint64_t)stride[1] * 2,
                               (uint64_t)(packed ? (int64_t)rows * stride[1] : stride[0]) * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap(m, base, 2, 4, dims, strides, box);
}

struct Maps { CUtensorMap q, k, v, dout, dq, dk, dv; };

bool make_maps(Maps& m, const fa_attn_args& a) {
  const bool packed = a.cu_seqlens_q != nullptr;
  const int qr = packed ? a.total_q : a.seqlen_q, kr = packed ? a.total_k : a.seqlen_k;
  const int D = a.head_dim;
  return make_map4(&m.q, a.q, a.q_stride, qr, a.heads_q, a.batch, D, packed) &&
         make_map4(&m.k, a.k, a.k_stride, kr, a.heads_kv, a.batch, D, packed) &&
         make_map4(&m.v, a.v, a.v_stride, kr, a.heads_kv, a.batch, D, packed) &&
         make_map4(&m.dout, a.dout, a.do_stride, qr, a.heads_q, a.batch, D, packed) &&
         (a.dq == nullptr || make_map4(&m.dq, a.dq, a.dq_stride, qr, a.heads_q, a.batch, D, packed)) &&
         (a.dk == nullptr || make_map4(&m.dk, a.dk, a.dk_stride, kr, a.heads_kv, a.batch, D, packed)) &&
         (a.dv == nullptr || make_map4(&m.dv, a.dv, a.dv_stride, kr, a.heads_kv, a.batch, D, packed));
}

template <typename K> int set_smem_attr(K kern, int bytes, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute(%d): %s", what, bytes, cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  return FA_OK;
}

template <typename T, int D>
int launch_dkdv(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  Maps m{};
  if (!make_maps(m, a)) {
    set_error("bwd_dkdv_cta_sm100: cuTensorMapEncodeTiled failed");
    return FA_ERR_LAUNCH;
  }
  auto kern = bwd_dkdv_cta_kernel<T, D, false>;   // the feature variants always take the persistent kernel
  if (int r = set_smem_attr(kern, BCfg<D>::kSmemBytes, "bwd_dkdv_cta_sm100")) return r;
  dim3 grid((a.seqlen_k + kT - 1) / kT, a.heads_kv, a.batch);
  kern<<<grid, kBwdThreads, BCfg<D>::kSmemBytes, st>>>(m.q, m.k, m.v, m.dout, m.dk, m.dv, a, cfg, host_wait_word(a.device));
  return check_launch("bwd_dkdv_cta_sm100");
}

}  // namespace

int bwd_dkdv_cta_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  if (a.head_dim == 128)
    return a.dtype == FA_BF16 ? launch_dkdv<__nv_bfloat16, 128>(a, cfg, st) : launch_dkdv<__half, 128>(a, cfg, st);
  return a.dtype == FA_BF16 ? launch_dkdv<__nv_bfloat16, 64>(a, cfg, st) : launch_dkdv<__half, 64>(a, cfg, st);
}


void bwd_dkdv_cta_clear_status() {
  const int z = 0;
  cudaMemcpyToSymbol(g_bwd_cta_status, &z, sizeof(int));
}

int bwd_dkdv_cta_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_bwd_cta_status, sizeof(int));
  return v;
}

}  // namespace fa
