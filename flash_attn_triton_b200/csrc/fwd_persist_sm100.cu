// Forward attention on the 5th-generation tensor cores, PERSISTENT: the pipeline of fwd_sm100.cu
// (two query tiles of 128 rows per work item, one softmax warpgroup, score buffer and output
// accumulator per tile = "stream"; TMA-staged K/V ring; tcgen05.mma into tensor memory; P over S in
// place; lazy rescale; P V in two key halves) with one CTA per SM that takes work items from a queue
// instead of one CTA per item:
//
//   * a counter in global memory hands out candidates (batch, head, pair of query tiles) in the
//     order of the non-persistent grid -- the CTAs that run together work on the same heads, whose
//     K/V stay in L2, and within a head the heavy items of a causal mask come first.  The producer
//     lane draws a candidate when the loads of the current item are all issued and publishes it
//     to the other roles through a small ring in shared memory;
//   * barriers, tensor memory and tensor maps are set up once; every barrier parity follows a
//     running count (ring position, tiles of a stream, items);
//   * the Q tiles of the next item are loaded as soon as the last Q K^T of the current one has
//     been issued (`q_empty`), its first K/V tiles as ring slots free up: the tensor pipe goes on
//     with the next item while the softmax groups still normalise and store the previous output;
//   * the output tiles are staged in two ring entries of their own at the end of the item's
//     K/V sequence (K0 V0 ... K(n-1) V(n-1) O_0 O_1) and written by the TMA unit; the storing thread
//     releases the entry when the unit has read it.
//
// Roles (384 threads): warps 0-3 / 4-7 softmax groups of streams 0 / 1, warp 8 TMA producer and
// queue, warp 9 MMA issuer, warps 10-11 idle (they complete the warpgroup that gives its registers
// to the softmax groups).  TMEM (512 columns): S[0] | S[1] | O_0 | O_1.
// Every mbarrier wait is bounded; on timeout the CTA records a status, frees its TMEM and returns.
#include <type_traits>

#include <cstdlib>
#include "common.cuh"
#include "sm100.cuh"

namespace fa {

using namespace sm100;

__device__ int g_fwdp_sm100_status = 0;

namespace {

constexpr int kBM = 128;          // query rows per tile (two tiles per work item)
constexpr int kBN = 128;          // keys per K/V tile
constexpr int kThreads = 384;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kMaxStages = 8;
constexpr int kSched = 4;         // depth of the in-CTA ring of work-queue entries
constexpr int kConsumers = 9;     // warps that read the queue: 8 softmax warps and the MMA issuer

template <int D> struct PCfg {
  static constexpr int kTileBytes = kBN * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 8;
  static constexpr int kBoxes = D / 64;
  static constexpr int kSmemTiles = (2 + kStages) * kTileBytes;
  static constexpr int kSmemBytes = kSmemTiles + 1024 /*align slack*/ + 1024 /*barriers*/;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct PShared {
  uint64_t q_full;               // both Q tiles of an item landed
  uint64_t q_empty;              // the last Q K^T of an item has finished reading them
  uint64_t kv_full[kMaxStages];
  uint64_t kv_empty[kMaxStages];
  uint64_t s_full[2];            // [stream]: its score tile computed
  uint64_t p_ready[2];           // [stream]: P written back (128 arrivals)
  uint64_t p_half[2];            // [stream]: the first 64 keys of P written back (128 arrivals)
  uint64_t o_ready[2];           // [stream]: its latest P V finished
  uint64_t sched_full[kSched];   // queue entry published by the producer lane
  uint64_t sched_empty[kSched];  // ... read by every consuming warp
  int sched_item[kSched];        // candidate index, -1 = no more work
  uint32_t tmem_base;
  volatile int abort_flag;
};
static_assert(sizeof(PShared) <= 1024, "PShared must fit its reserve");

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, PShared* sh, int code) {
  return bounded_wait(bar, parity, &sh->abort_flag, &g_fwdp_sm100_status, code);
}

template <typename T> struct PFmt;
template <> struct PFmt<__half> { static constexpr int code = 0; };
template <> struct PFmt<__nv_bfloat16> { static constexpr int code = 1; };

// Geometry of a work item, derived from its candidate index by every role on its own.
struct Geo {
  SeqInfo si;
  int b, h, hk, m00;
  int n_hi, nsteps;              // key tiles [n_hi - nsteps, n_hi); step j works on tile n_hi - 1 - j
  int jb0, je0, jb1, je1;        // stream x is active for the steps [jb_x, je_x)
  __device__ __forceinline__ int jb(int x) const { return x ? jb1 : jb0; }
  __device__ __forceinline__ int je(int x) const { return x ? je1 : je0; }
};

// false: the candidate lies outside its sequence (packed batches) and is skipped
__device__ __forceinline__ bool item_geo(const fa_attn_args& p, const ScoreCfg& cfg, int c, int npair, Geo& g) {
  const int pr = c % npair;
  g.h = (c / npair) % p.heads_q;
  g.b = c / (npair * p.heads_q);
  const int mblk = cfg.causal ? (npair - 1 - pr) : pr;      // heavy blocks first
  g.si = seq_info(p, g.b);
  g.m00 = mblk * 2 * kBM;
  if (g.m00 >= g.si.q_len) return false;
  g.hk = g.h / (p.heads_q / p.heads_kv);
  const int off = p.q_pos_offset;
  auto tile_range = [&](int m0, int& lo, int& hi) {
    lo = hi = 0;
    if (m0 < g.si.q_len) {
      int klo, khi;
      visible_key_range(cfg, m0 + off, min(m0 + kBM, g.si.q_len) - 1 + off, g.si.k_len, klo, khi);
      if (khi > klo) {
        lo = klo / kBN;
        hi = (khi + kBN - 1) / kBN;
      }
    }
  };
  int nlo0, nhi0, nlo1, nhi1;
  tile_range(g.m00, nlo0, nhi0);
  tile_range(g.m00 + kBM, nlo1, nhi1);
  const bool has0 = nhi0 > nlo0, has1 = nhi1 > nlo1;
  const int n_lo = has0 ? (has1 ? min(nlo0, nlo1) : nlo0) : nlo1;
  g.n_hi = has0 ? (has1 ? max(nhi0, nhi1) : nhi0) : nhi1;
  g.nsteps = (has0 || has1) ? g.n_hi - n_lo : 0;
  g.jb0 = has0 ? g.n_hi - nhi0 : 0;
  g.je0 = has0 ? g.n_hi - nlo0 : 0;
  g.jb1 = has1 ? g.n_hi - nhi1 : 0;
  g.je1 = has1 ? g.n_hi - nlo1 : 0;
  return true;
}

// Entry number idx of this CTA's queue ring, as seen by a consuming warp (all lanes together).
__device__ __forceinline__ int sched_get(PShared* sh, int idx, bool& ok) {
  const int slot = idx % kSched;
  if (!wait_bar(&sh->sched_full[slot], (idx / kSched) & 1, sh, 61)) {
    ok = false;
    return -1;
  }
  const int c = sh->sched_item[slot];
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&sh->sched_empty[slot]));
  return c;
}

}  // namespace

// kPoly > 0: on unmasked tiles of the plain variant every kPoly-th pair of exponentials runs on
// the FMA pipe (ex2_fma2) and the scores are read from tensor memory a second time for the exp2
// pass, 32 columns at a time and one chunk ahead, instead of staying in 128 registers (the
// polynomial needs the registers; without them it was a loss).  The host picks it for long items.
template <typename T, int D, bool kExtras, int kPoly>
__global__ void __launch_bounds__(kThreads, 1)
fwd_persist_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                         const fa_attn_args p, const ScoreCfg cfg, const int npair, const int ncand,
                         unsigned int* const queue, int* const host_status) {
  constexpr bool kPvSplit = !kExtras;     // P V in two key halves (measured: helps the plain variants only)
  using C = PCfg<D>;
  constexpr int S = C::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PShared* sh = reinterpret_cast<PShared*>(tiles + C::kSmemTiles);
  const uint32_t sQ = smem_u32(tiles);                 // + x * kTileBytes
  const uint32_t sKV = sQ + 2 * C::kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int off = p.q_pos_offset;

  if (tid == 0) {
    mbar_init(smem_u32(&sh->q_full), 1);
    mbar_init(smem_u32(&sh->q_empty), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sh->s_full[i]), 1);
      mbar_init(smem_u32(&sh->o_ready[i]), 1);
      mbar_init(smem_u32(&sh->p_ready[i]), 128);
      mbar_init(smem_u32(&sh->p_half[i]), 128);
    }
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&sh->kv_full[i]), 1);
      mbar_init(smem_u32(&sh->kv_empty[i]), 1);
    }
    for (int i = 0; i < kSched; ++i) {
      mbar_init(smem_u32(&sh->sched_full[i]), 1);
      mbar_init(smem_u32(&sh->sched_empty[i]), kConsumers);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&sh->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  // Ring bookkeeping shared by every role: an item with n steps takes the ring positions
  //   K_0 V_0 K_1 V_1 ... K_(n-1) V_(n-1) O_0 O_1        (2 n + 2 entries, none when n = 0)
  // and every role advances the same position counter; position `pos` lives in slot pos % S and
  // completes phase (pos / S) & 1 of that slot's barriers.  K/V entries are released by the MMA
  // that read them, the two output entries by the thread that stored them.

  if (warp >= 10) {
    reg_dealloc<72>();
  } else if (warp == 8) {
    // ------------------------------- TMA producer and work queue ------------------------
    reg_dealloc<72>();
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      prefetch_tmap(&tmO);
      int pos = 0, qi = 0, fidx = 0;
      bool ok = true;
      while (ok) {
        // draw the next item (as late as possible: all loads of the previous one are issued)
        Geo g;
        int c = -1;
        for (;;) {
          const unsigned int u = atomicAdd(&queue[0], 1u);
          if (u >= (unsigned int)ncand) break;
          if (item_geo(p, cfg, (int)u, npair, g)) {
            c = (int)u;
            break;
          }
        }
        {
          const int slot = fidx % kSched;
          ok = wait_bar(&sh->sched_empty[slot], ((fidx / kSched) & 1) ^ 1, sh, 60);
          if (!ok) break;
          sh->sched_item[slot] = c;
          mbar_arrive(smem_u32(&sh->sched_full[slot]));
          ++fidx;
        }
        if (c < 0) break;
        if (g.nsteps == 0) continue;
        const int krow0 = (int)g.si.k_row0, kb = (int)g.si.k_boff;
        auto load_kv = [&](const CUtensorMap* tm, int tile) {
          if (!ok) return;
          const int slot = pos % S;
          ok = wait_bar(&sh->kv_empty[slot], ((pos / S) & 1) ^ 1, sh, 11);
          if (!ok) return;
          const uint32_t bar = smem_u32(&sh->kv_full[slot]);
          mbar_expect_tx(bar, C::kTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sKV + slot * C::kTileBytes + bx * (kBN * 128), tm, bar, bx * 64, g.hk, krow0 + tile * kBN, kb);
          ++pos;
        };
        // K_0 first (its slot is usually free long before the Q tiles are)
        load_kv(&tmK, g.n_hi - 1);
        // both Q tiles, once the previous item's last Q K^T has finished with them
        if (ok) ok = wait_bar(&sh->q_empty, (qi & 1) ^ 1, sh, 12);
        if (!ok) break;
        {
          const uint32_t bar = smem_u32(&sh->q_full);
          const int ntile = (g.m00 + kBM < g.si.q_len) ? 2 : 1;
          mbar_expect_tx(bar, ntile * C::kTileBytes);
          for (int x = 0; x < ntile; ++x)
            for (int bx = 0; bx < C::kBoxes; ++bx)
              tma_load_4d(sQ + x * C::kTileBytes + bx * (kBM * 128), &tmQ, bar, bx * 64, g.h,
                          (int)g.si.q_row0 + g.m00 + x * kBM, (int)g.si.q_boff);
          ++qi;
        }
        for (int j = 0; j < g.nsteps && ok; ++j) {
          load_kv(&tmV, g.n_hi - 1 - j);
          if (j + 1 < g.nsteps) load_kv(&tmK, g.n_hi - 2 - j);
        }
        // the two output entries: nothing to load, but their slots must be free and their
        // "landed" phase has to complete like any other entry's
        for (int x = 0; x < 2 && ok; ++x) {
          const int slot = pos % S;
          ok = wait_bar(&sh->kv_empty[slot], ((pos / S) & 1) ^ 1, sh, 13);
          if (ok) mbar_arrive(smem_u32(&sh->kv_full[slot]));
          ++pos;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -----------------------------------------
    // The whole warp runs the control flow in lock step and every lane polls the barriers;
    // the lane chosen once by elect_one issues the MMAs and commits.
    reg_dealloc<72>();
    constexpr uint32_t idesc_qk = make_idesc(1, PFmt<T>::code, 0, 0, kBM, kBN);
    constexpr uint32_t idesc_pv = make_idesc(1, PFmt<T>::code, 0, 1, kBM, D);
    const uint32_t leader = elect_one() ? 1u : 0u;
    bool ok = true;
    auto wwait = [&](uint64_t* bar, uint32_t parity, int code) {
      if (ok) ok = wait_bar(bar, parity, sh, code);
      tc_fence_after();
    };
    // S[x] = Q_x K^T with the K tile at kbase
    auto issue_qk = [&](int x, uint32_t kbase) {
      const uint64_t dq = make_smem_desc(sQ + x * C::kTileBytes, 16, 1024);
      const uint64_t dk = make_smem_desc(kbase, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t o = ((kk / 4) * (kBM * 128) + (kk % 4) * 32) >> 4;
        mma_f16_ss_lp(tmem + x * kBN, dq + o, dk + o, idesc_qk, kk > 0, leader);
      }
      mma_commit_lp(smem_u32(&sh->s_full[x]), leader);
    };
    int pos = 0, qi = 0, sidx = 0;
    int pcnt[2] = {0, 0};                                // P tiles consumed so far, per stream
    for (;;) {
      const int c = sched_get(sh, sidx++, ok);
      if (!ok || c < 0) break;
      Geo g;
      item_geo(p, cfg, c, npair, g);
      if (g.nsteps == 0) continue;
      const int nsteps = g.nsteps;
      // the last step in which any stream still needs a new score tile, i.e. the last Q K^T
      wwait(&sh->kv_full[pos % S], (pos / S) & 1, 22);   // K_0
      wwait(&sh->q_full, qi & 1, 21);
      if (!ok) break;
      ++qi;
      {
        const uint32_t kbase = sKV + (pos % S) * C::kTileBytes;
        if (g.jb0 == 0 && g.je0 > 0) issue_qk(0, kbase);
        if (g.jb1 == 0 && g.je1 > 0) issue_qk(1, kbase);
        if (nsteps == 1) mma_commit_lp(smem_u32(&sh->q_empty), leader);
        mma_commit_lp(smem_u32(&sh->kv_empty[pos % S]), leader);
        ++pos;
      }
      for (int j = 0; j < nsteps && ok; ++j) {
        const int vpos = pos, kpos = pos + 1;
        wwait(&sh->kv_full[vpos % S], (vpos / S) & 1, 24);          // V_j
        if (!ok) break;
        const uint32_t vbase = sKV + (vpos % S) * C::kTileBytes;
        const bool more = j + 1 < nsteps;
        const uint32_t kbase = sKV + (kpos % S) * C::kTileBytes;
        bool k_waited = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (j >= g.jb(x) && j < g.je(x)) {
            const uint32_t a = tmem + x * kBN;
            const uint64_t dv = make_smem_desc(vbase, kBN * 128, 1024);
            const bool acc = j > g.jb(x);
            if (kPvSplit) {
              wwait(&sh->p_half[x], pcnt[x] & 1, 25 + x);
              if (!ok) break;
#pragma unroll
              for (int kk = 0; kk < kBN / 32; ++kk)
                mma_f16_ts_lp(tmem + 256 + x * 128, a + kk * 8, dv + ((kk * 2048) >> 4), idesc_pv,
                              (acc || kk > 0) ? 1u : 0u, leader);
            }
            wwait(&sh->p_ready[x], pcnt[x] & 1, 25 + x);
            if (!ok) break;
            ++pcnt[x];
#pragma unroll
            for (int kk = kPvSplit ? kBN / 32 : 0; kk < kBN / 16; ++kk)
              mma_f16_ts_lp(tmem + 256 + x * 128, a + kk * 8, dv + ((kk * 2048) >> 4), idesc_pv,
                            (acc || kk > 0) ? 1u : 0u, leader);
            mma_commit_lp(smem_u32(&sh->o_ready[x]), leader);
          }
          if (more && j + 1 >= g.jb(x) && j + 1 < g.je(x)) {
            if (!k_waited) {
              wwait(&sh->kv_full[kpos % S], (kpos / S) & 1, 22);   // K_{j+1}
              if (!ok) break;
              k_waited = true;
            }
            issue_qk(x, kbase);
          }
        }
        if (!ok) break;
        mma_commit_lp(smem_u32(&sh->kv_empty[vpos % S]), leader);
        ++pos;
        if (more) {
          // a K tile that no stream needs (cannot happen for contiguous visible ranges) would
          // still have to be consumed to keep the ring in step
          if (!k_waited) wwait(&sh->kv_full[kpos % S], (kpos / S) & 1, 22);
          if (j + 2 == nsteps) mma_commit_lp(smem_u32(&sh->q_empty), leader);   // that was the item's last Q K^T
          mma_commit_lp(smem_u32(&sh->kv_empty[kpos % S]), leader);
          ++pos;
        }
      }
      pos += 2;                                          // the two output entries
    }
  } else {
    // ------------------------------- softmax groups -------------------------------------
    reg_alloc<216>();
    const int x = warp >> 2;                         // stream = query tile of the item
    const int row_in_tile = (warp & 3) * 32 + lane;  // TMEM lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tSx = tmem + lane_addr + x * kBN;
    const uint32_t tOx = tmem + lane_addr + 256 + x * 128;
    bool ok = true;
    int pos = 0, sidx = 0, qi = 0;
    int tc = 0;                                      // tiles of this stream so far (all items)

    for (;;) {
      const int c = sched_get(sh, sidx++, ok);
      if (!ok || c < 0) break;
      Geo g;
      item_geo(p, cfg, c, npair, g);
      const SeqInfo& si = g.si;
      const int b = g.b, h = g.h;
      const int m0 = g.m00 + x * kBM;
      const int row = m0 + row_in_tile;                // query row inside the sequence
      const int qpos = row + off;
      const float slope = (kExtras && cfg.has_alibi) ? p.alibi_slopes[b * p.heads_q + h] : 0.f;
      float m_used = -INFINITY, l = 0.f;
      const int tq_min = m0 + off, tq_max = tq_min + kBM - 1;
      const int my_jb = g.jb(x), my_je = g.je(x);
      const int my_tiles = my_je - my_jb;

      for (int j = my_jb; j < my_je && ok; ++j, ++tc) {
        const int t = j - my_jb;                       // index of the tile inside this stream's item
        const int k0 = (g.n_hi - 1 - j) * kBN;
        bool masked = (k0 + kBN > si.k_len);
        if (cfg.causal) masked |= (k0 + kBN - 1 > tq_min);
        if (cfg.wl >= 0) masked |= (k0 < tq_max - cfg.wl);
        if (cfg.wr >= 0) masked |= (k0 + kBN - 1 > tq_min + cfg.wr);

        ok = wait_bar(&sh->s_full[x], tc & 1, sh, 31 + x);
        if (!ok) break;
        tc_fence_after();

        // ---- the 128 scores of this row into registers -------------------------------------
        uint32_t r[4][32];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld32(tSx + cc * 32, r[cc]);
        tmem_wait_ld();

        const bool prescaled = kExtras || masked;
        // columns (keys) of this tile that this thread's query row sees (used by masked tiles only)
        ColMask cm;
        if (masked) {
          int vk_lo, vk_hi;
          visible_k_interval(cfg, qpos, si.k_len, vk_lo, vk_hi);
          cm = make_col_mask(vk_lo - k0, vk_hi - k0);
        }
        if (prescaled) {
          // score pipeline and mask applied once, in place; values end up in the log2 domain.
          // One body, compiled per (masked tile, soft cap): no branch inside the unrolled loops.
          const float dist0 = (float)(qpos - k0);
          auto score_tile = [&](auto mask_tag, auto cap_tag, auto abs_tag) {
            constexpr bool kMask = decltype(mask_tag)::value;
            constexpr bool kCap = decltype(cap_tag)::value;
            constexpr bool kAbs = decltype(abs_tag)::value;
            if (kExtras) {
              // packed pairs; the distance of a pair's columns goes down by (2, 2)
              const FeatK fk = feat_k<kCap>(cfg, slope);
              const float2 step2 = make_float2(-2.f, -2.f);
              float2 d2 = make_float2(dist0, dist0 - 1.f);
#pragma unroll
              for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  float2 v = score_unit_feat2<kCap, kAbs>(
                      fk, make_float2(__uint_as_float(r[cc][i]), __uint_as_float(r[cc][i + 1])), d2);
                  if (kMask) {
                    v.x = col_visible(cm, cc * 32 + i) ? v.x : -INFINITY;
                    v.y = col_visible(cm, cc * 32 + i + 1) ? v.y : -INFINITY;
                  }
                  r[cc][i] = __float_as_uint(v.x);
                  r[cc][i + 1] = __float_as_uint(v.y);
                  d2 = f2add(d2, step2);
                }
              }
            } else {
#pragma unroll
              for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  float v = __uint_as_float(r[cc][i]) * cfg.scale_log2;
                  if (kMask) v = col_visible(cm, cc * 32 + i) ? v : -INFINITY;
                  r[cc][i] = __float_as_uint(v);
                }
              }
            }
          };
          const bool cap = kExtras && cfg.softcap > 0.f;
          const bool need_abs = kExtras && !cfg.causal;    // under the causal mask visible keys lie at distance >= 0
          auto run_score = [&](auto mask_tag) {
            if (cap) {
              if (need_abs) score_tile(mask_tag, std::true_type{}, std::true_type{});
              else score_tile(mask_tag, std::true_type{}, std::false_type{});
            } else {
              if (need_abs) score_tile(mask_tag, std::false_type{}, std::true_type{});
              else score_tile(mask_tag, std::false_type{}, std::false_type{});
            }
          };
          if (masked) run_score(std::true_type{});
          else run_score(std::false_type{});
        }

        // ---- packed batches: keep the next sequence's values out of P V ---------------------
        // The last key tile of a packed sequence also holds rows of the NEXT sequence.  Their
        // probabilities are exactly 0, but 0 * inf or 0 * NaN is NaN: zero those rows of the V tile
        // (ring position pos + 2 j + 1) before P is handed to the issuer.  One thread per row; a
        // row is D contiguous 16-bit values per 64-wide box, so the swizzle does not matter.
        // Both streams may do it for the same tile (zeros over zeros).
        if (p.cu_seqlens_k != nullptr && k0 + kBN > si.k_len) {
          const int vpos = pos + 2 * j + 1;
          ok = wait_bar(&sh->kv_full[vpos % S], (vpos / S) & 1, sh, 39);
          if (!ok) break;
          if (k0 + row_in_tile >= si.k_len) {
            unsigned char* vrow = tiles + C::kTileBytes * (2 + vpos % S) + row_in_tile * 128;
#pragma unroll
            for (int bx = 0; bx < C::kBoxes; ++bx) {
#pragma unroll
              for (int c16 = 0; c16 < 8; ++c16)
                reinterpret_cast<uint4*>(vrow + bx * (kBN * 128))[c16] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
          fence_proxy_async();
        }

        // ---- row maximum: eight chains of three-input maxima --------------------------------
        float mx;
        {
          float mt[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            mt[i] = fmax3(__uint_as_float(r[0][i]), __uint_as_float(r[0][8 + i]), __uint_as_float(r[0][16 + i]));
#pragma unroll
          for (int i = 0; i < 8; ++i) mt[i] = fmaxf(mt[i], __uint_as_float(r[0][24 + i]));
#pragma unroll
          for (int cc = 1; cc < 4; ++cc) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              mt[i] = fmax3(mt[i], __uint_as_float(r[cc][i]), __uint_as_float(r[cc][8 + i]));
              mt[i] = fmax3(mt[i], __uint_as_float(r[cc][16 + i]), __uint_as_float(r[cc][24 + i]));
            }
          }
          mx = fmaxf(fmax3(mt[0], mt[1], mt[2]), fmaxf(fmax3(mt[3], mt[4], mt[5]), fmaxf(mt[6], mt[7])));
        }
        // what the stored values are multiplied by to give log2-domain scores: softmax_scale log2e
        // on the plain path, cap log2e for capped scores (stored as tanh), else 1; all >= 0
        const float mul = !prescaled ? cfg.scale_log2 : ((kExtras && cfg.softcap > 0.f) ? cfg.softcap * FA_LOG2E : 1.f);
        mx *= mul;

        // ---- lazy rescale ----------------------------------------------------------------
        if (t == 0) {
          m_used = mx;
        } else {
          const bool need = mx > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            // The previous P V of this stream is its (tc-1)-th; the one of this tile cannot
            // complete before P is written below, so the barrier is at most one phase ahead
            // of the parity waited for here.
            ok = wait_bar(&sh->o_ready[x], (tc - 1) & 1, sh, 33 + x);
            if (!ok) break;
            tc_fence_after();
            const float alpha = need ? exp2f(m_used - mx) : 1.f;  // m_used = -inf -> 0
            if (need) {
              m_used = mx;
              l *= alpha;
            }
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t ro[32];
              tmem_ld32(tOx + cc * 32, ro);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
              tmem_st32(tOx + cc * 32, ro);
            }
            tmem_wait_st();
          }
        }
        const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;

        // ---- P = exp2(s - m), row sum, P -> TMEM in place over S ----------------------------
        // packed pairs: one FMA, two exponentials, one conversion and one add per two scores
        if (kPoly > 0 && !prescaled) {
          const float2 mul2 = make_float2(mul, mul), nm2 = make_float2(-m_safe, -m_safe);
          float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
          uint32_t ra[32], rb[32];
          tmem_ld32(tSx, ra);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t (&cur)[32] = (cc & 1) ? rb : ra;
            uint32_t (&nxt)[32] = (cc & 1) ? ra : rb;
            tmem_wait_ld();
            if (cc < 3) tmem_ld32(tSx + (cc + 1) * 32, nxt);
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 a = f2fma(make_float2(__uint_as_float(cur[i]), __uint_as_float(cur[i + 1])), mul2, nm2);
              const float2 pe = ex2_pair<kPoly>(a, i >> 1);
              pk[i >> 1] = Elem<T>::pack(pe.x, pe.y);
              acc2[(i >> 1) & 1] = f2add(acc2[(i >> 1) & 1], pe);
            }
            tmem_st16(tSx + cc * 16, pk);
            if (kPvSplit && cc == 1) {
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(smem_u32(&sh->p_half[x]));
            }
          }
          l += (acc2[0].x + acc2[0].y) + (acc2[1].x + acc2[1].y);
        } else {
          const float2 mul2 = make_float2(mul, mul), nm2 = make_float2(-m_safe, -m_safe);
          float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 a = f2fma(make_float2(__uint_as_float(r[cc][i]), __uint_as_float(r[cc][i + 1])), mul2, nm2);
              const float2 pe = make_float2(ex2(a.x), ex2(a.y));
              pk[i >> 1] = Elem<T>::pack(pe.x, pe.y);
              acc2[(i >> 1) & 1] = f2add(acc2[(i >> 1) & 1], pe);
            }
            tmem_st16(tSx + cc * 16, pk);
            if (kPvSplit && cc == 1) {
              // the first 64 keys of P are complete: the issuer starts P V on them while the
              // second half of the exponentials runs
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(smem_u32(&sh->p_half[x]));
            }
          }
          l += (acc2[0].x + acc2[0].y) + (acc2[1].x + acc2[1].y);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh->p_ready[x]));
      }
      if (!ok) break;

      // ---- epilogue: O / l -> global, base-2 LSE ------------------------------------------
      if (my_tiles > 0) ok = wait_bar(&sh->o_ready[x], (tc - 1) & 1, sh, 35 + x);
      if (!ok) break;
      tc_fence_after();
      // The tile is staged in this stream's output entry of the ring (swizzled box layout) and
      // written by the TMA unit as full rows; a packed tile that reaches past the end of its
      // sequence is stored row by row instead (the unit would write the neighbour's rows), and so
      // is the all-zero tile of a stream without visible keys.
      const bool uses_ring = g.nsteps > 0;
      const int opos = pos + 2 * g.nsteps + x;
      const bool in_seq = m0 < si.q_len;
      const bool via_tma = uses_ring && in_seq && my_tiles > 0 &&
                           ((p.cu_seqlens_q == nullptr) || (m0 + kBM <= si.q_len));
      if (uses_ring) {
        // The entry is ours once the producer has passed it (its previous occupant is released).
        // A parity wait must not run a whole phase ahead of its barrier, and a stream with few or
        // no tiles gets here long before the ring does: walk up the entries of that slot from the
        // last position this stream KNOWS to have landed -- its own last V tile, or, without
        // tiles, everything before this item once the item's Q tiles have landed (the producer
        // passes the previous item's output entries before it loads them).
        int known = pos + 2 * my_je - 1;
        if (my_tiles == 0) {
          ok = wait_bar(&sh->q_full, qi & 1, sh, 37);
          if (!ok) break;
          known = pos - 1;
        }
        ++qi;
        for (int q = opos - S * ((opos - known - 1) / S); q <= opos && ok; q += S)
          ok = wait_bar(&sh->kv_full[q % S], (q / S) & 1, sh, 36);
        if (!ok) break;
      }
      if (in_seq) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool row_ok = row < si.q_len;
        const uint32_t sOx = sKV + (opos % S) * C::kTileBytes;
        T* og = reinterpret_cast<T*>(p.o) + si.q_boff * p.o_stride[0] +
                (si.q_row0 + row) * p.o_stride[1] + (int64_t)h * p.o_stride[2];
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t ra[32];
          if (my_tiles > 0) {
            tmem_ld32(tOx + cc * 32, ra);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) ra[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = Elem<T>::pack(__uint_as_float(ra[i]) * inv, __uint_as_float(ra[i + 1]) * inv);
            v.y = Elem<T>::pack(__uint_as_float(ra[i + 2]) * inv, __uint_as_float(ra[i + 3]) * inv);
            v.z = Elem<T>::pack(__uint_as_float(ra[i + 4]) * inv, __uint_as_float(ra[i + 5]) * inv);
            v.w = Elem<T>::pack(__uint_as_float(ra[i + 6]) * inv, __uint_as_float(ra[i + 7]) * inv);
            if (via_tma) {
              const int col = cc * 32 + i;                   // first of 8 columns = one 16-byte chunk
              st_shared_v4(sw128_addr(sOx + (col / 64) * (kBM * 128), row_in_tile, (col % 64) / 8), v);
            } else if (row_ok) {
              *reinterpret_cast<uint4*>(og + cc * 32 + i) = v;
            }
          }
        }
        tc_fence_before();
        if (via_tma) {
          fence_proxy_async();
          if (x == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
          else asm volatile("bar.sync 2, 128;\n" ::: "memory");
          if ((tid & 127) == 0) {
#pragma unroll
            for (int bx = 0; bx < D / 64; ++bx)
              tma_store_4d(&tmO, sOx + bx * (kBM * 128), bx * 64, h, (int)si.q_row0 + m0, (int)si.q_boff);
            tma_store_commit();
            tma_store_wait_read();
          }
        }
        if (row_ok && p.lse2 != nullptr)
          p.lse2[si.q_boff * p.lse_stride[0] + (si.q_row0 + row) * p.lse_stride[1] +
                 (int64_t)h * p.lse_stride[2]] = l > 0.f ? m_used + log2f(l) : -INFINITY;
      }
      if (uses_ring) {
        // hand the entry back (after the unit has read it, if it was used)
        if ((tid & 127) == 0) mbar_arrive(smem_u32(&sh->kv_empty[opos % S]));
        pos += 2 * g.nsteps + 2;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
  if (tid == 0) {
    report_abort(sh->abort_flag, host_status);
    // the last CTA to finish puts the queue back to zero for the next launch that is given it
    __threadfence();
    const unsigned int done = atomicAdd(&queue[1], 1u);
    if (done == gridDim.x - 1) {
      queue[0] = 0u;
      queue[1] = 0u;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static bool make_map_p(CUtensorMap* m, const void* base, const int64_t* stride, int rows, int heads,
                       int batch, int D, bool packed) {
  // dims (innermost first): head_dim, heads, rows, batch
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)rows, (uint64_t)(packed ? 1 : batch)};
  const uint64_t strides[3] = {(uint64_t)stride[2] * 2, (uint64_t)stride[1] * 2,
                               (uint64_t)(packed ? (int64_t)rows * stride[1] : stride[0]) * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap(m, base, 2, 4, dims, strides, box);
}

template <typename T, int D>
static int launch_p(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st, int q_rows, int k_rows) {
  using C = PCfg<D>;
  CUtensorMap tq, tk, tv, to;
  const bool packed = a.cu_seqlens_q != nullptr;
  if (!make_map_p(&to, a.o, a.o_stride, q_rows, a.heads_q, a.batch, D, packed) ||
      !make_map_p(&tq, a.q, a.q_stride, q_rows, a.heads_q, a.batch, D, packed) ||
      !make_map_p(&tk, a.k, a.k_stride, k_rows, a.heads_kv, a.batch, D, packed) ||
      !make_map_p(&tv, a.v, a.v_stride, k_rows, a.heads_kv, a.batch, D, packed)) {
    set_error("fwd_persist_sm100: cuTensorMapEncodeTiled failed");
    return FA_ERR_LAUNCH;
  }
  const bool extras = cfg.has_alibi || cfg.softcap > 0.f;
  // A quarter of the exponentials on the FMA pipe pays when both streams of a CTA spend most of
  // their time in unmasked tiles: measured with launches interleaved, D = 128, -3 % at 16 key
  // tiles per item without a mask, -6 % at 24, -8 % at 32; with the causal mask +3 % at 32 key
  // tiles (16.5 per item on average), +-1 % at 48, -4 % at 64, -7.5 % at 128.  D = 64: -6 to -9 %
  // without a mask from 16 key tiles up; causal +9 % at 16, +5 % at 32, 0 at 64, -4 % at 128.
  const int nk = (a.seqlen_k + kBN - 1) / kBN;
  bool poly = !extras && !packed && cfg.wl < 0 && cfg.wr < 0 && nk >= (cfg.causal ? (D == 64 ? 128 : 64) : 16);
  if (const char* e = getenv("FA_B200_FWD_POLY")) poly = !extras && atoi(e) != 0;   // tests: 0 = never, 1 = always
  auto kern = extras ? fwd_persist_sm100_kernel<T, D, true, 0>
                     : (poly ? fwd_persist_sm100_kernel<T, D, false, 4> : fwd_persist_sm100_kernel<T, D, false, 0>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) {
    set_error("fwd_persist_sm100: cudaFuncSetAttribute(%d): %s", C::kSmemBytes, cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  unsigned int* queue = work_queue(a.device);
  if (queue == nullptr) return FA_ERR_LAUNCH;
  const int npair = (a.seqlen_q + 2 * kBM - 1) / (2 * kBM);
  const int64_t ncand64 = (int64_t)npair * a.heads_q * a.batch;
  if (ncand64 > (1 << 30)) {
    set_error("fwd_persist_sm100: too many work items");
    return FA_ERR_UNSUPPORTED;
  }
  const int ncand = (int)ncand64;
  const int grid = ncand < sm_count(a.device) ? ncand : sm_count(a.device);
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, to, a, cfg, npair, ncand, queue, host_wait_word(a.device));
  return check_launch("fwd_persist_sm100");
}

int fwd_persist_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  const bool packed = a.cu_seqlens_q != nullptr;
  const int q_rows = packed ? a.total_q : a.seqlen_q;
  const int k_rows = packed ? a.total_k : a.seqlen_k;
  if (a.head_dim == 128)
    return a.dtype == FA_BF16 ? launch_p<__nv_bfloat16, 128>(a, cfg, st, q_rows, k_rows)
                              : launch_p<__half, 128>(a, cfg, st, q_rows, k_rows);
  return a.dtype == FA_BF16 ? launch_p<__nv_bfloat16, 64>(a, cfg, st, q_rows, k_rows)
                            : launch_p<__half, 64>(a, cfg, st, q_rows, k_rows);
}

int fwd_persist_sm100_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_fwdp_sm100_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

int fwd_persist_sm100_clear_status() {
  const int z = 0;
  return cudaMemcpyToSymbol(g_fwdp_sm100_status, &z, sizeof(int)) == cudaSuccess ? 0 : -1;
}

}  // namespace fa
