// Forward attention on the 5th-generation tensor cores: TMA-staged tiles, tcgen05.mma with
// accumulators in tensor memory, warp-specialised online softmax.
//
// One CTA owns TWO tiles of 128 query rows of one (batch, head) -- 256 consecutive rows -- and
// every K/V tile it loads is used by both: that halves the TMA writes into shared memory per
// score tile (the tensor pipe reads its operands from there at the full shared-memory bandwidth,
// so every byte counts) and the fixed cost per CTA.  Each query tile is a "stream" with its own
// softmax warpgroup, score buffer and output accumulator; the two streams run out of phase, so
// that while one group is in its exp2 (MUFU) phase the tensor pipe runs the other stream's
// P V and Q K^T:
//
//   warps 0-3   softmax group 0 : query rows   0..127 of the CTA (S[0], accumulator O_0)
//   warps 4-7   softmax group 1 : query rows 128..255 of the CTA (S[1], accumulator O_1)
//   warp  8     TMA producer    : both Q tiles once, then K/V tiles through a ring
//   warp  9     MMA issuer      : S[x] = Q_x K_j^T (SS);  O_x += P_x V_j (A = P_x from TMEM)
//   warps 10-11 idle (warp 10 stages the key scales of the INT8 variant); they complete the
//               third warpgroup so that it can hand its registers to the softmax groups
//
// One thread owns one query row (TMEM lane = row) and all 128 scores of a tile.  P (fp16/bf16)
// overwrites the first 64 columns of its S buffer; Q_x K_{j+1}^T may overwrite it because
// P_x V_j precedes it in the in-order tensor pipe.  The running maximum is only raised when it
// grows by more than 2^8 ("lazy rescale"), so O is rarely touched by the softmax warps.
//
// Step j of a CTA works on key tile n_hi - 1 - j: the tiles that need masking (the causal
// diagonal, the ragged end of the keys) come first, where they overlap the start-up of the
// pipeline.  With a causal mask the lower query tile sees one key tile less, so a stream is
// active only for the steps whose tile it can see.
//
// TMEM (512 columns): S[0] | S[1] | O_0 | O_1, 128 fp32 columns each (O uses head_dim).
// Shared memory: two Q tiles (128 x D each) + a ring of K/V tiles (128 keys x D), written by
// TMA with the 128-byte swizzle the MMA descriptors expect, in order of use K0, V0, K1, V1, ...
// The epilogue stages each output tile over its Q tile and lets the TMA unit store it.
//
// Every mbarrier wait is bounded; on timeout the CTA raises a device-side status word,
// releases its TMEM and returns.
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.cuh"
#define PROF_TAG fwd
#include "prof.cuh"
#include "sm100.cuh"

namespace fa {

using namespace sm100;

__device__ int g_fwd_sm100_status = 0;

namespace {

constexpr int kBM = 128;          // query rows per tile (two tiles per CTA)
constexpr int kBN = 128;          // keys per K/V tile
constexpr int kThreads = 384;     // 8 softmax warps + a warpgroup holding producer and MMA warps
constexpr float kRescaleThreshold = 8.0f;
// Share of the exponentials of the unmasked fast path that run on the FMA pipe (every n-th;
// 0 = none: measured slower here, the softmax warps are short of issue slots, not of MUFU).
#ifndef FA_POLY_FWD
#define FA_POLY_FWD 0
#endif
constexpr int kPolyEvery = FA_POLY_FWD;
// P V of a tile issued in two halves of 64 keys, the first as soon as its probabilities are stored.
#ifndef FA_PV_SPLIT
#define FA_PV_SPLIT 1
#endif
constexpr bool kPvSplitOn = FA_PV_SPLIT != 0;
constexpr int kMaxStages = 8;
constexpr int kSkSlots = 4;       // INT8 variant: key-scale tiles staged ahead

template <int D> struct Cfg {
  static constexpr int kTileBytes = kBN * D * 2;                    // one Q/K/V tile
  static constexpr int kStages = (D == 128) ? 4 : 8;                // K/V ring depth
  static constexpr int kBoxes = D / 64;                             // TMA boxes per tile
  static constexpr int kSmemTiles = (2 + kStages) * kTileBytes;
  static constexpr int kSmemBytes = kSmemTiles + 1024 /*align slack*/ + 4096 /*barriers, merge*/;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct Shared {
  uint64_t q_full;
  uint64_t kv_full[kMaxStages];
  uint64_t kv_empty[kMaxStages];
  uint64_t s_full[2];      // [stream]: its score tile computed
  uint64_t p_ready[2];     // [stream]: P written back (128 arrivals)
  uint64_t p_half[2];      // [stream]: the first 64 keys of P written back (128 arrivals)
  uint64_t o_ready[2];     // [stream]: its latest P V finished
  uint32_t tmem_base;
  volatile int abort_flag;
  // INT8 variant: key scales of the current score tiles, staged by warp 10
  // (a ring of kSkSlots key tiles: with a causal mask one stream runs a whole step ahead of the
  // other, and a slot is only released when BOTH groups are done with it)
  uint64_t sk_full[kSkSlots];   // scales of the key tile of step j (slot j % kSkSlots) written
  uint64_t sk_empty[kSkSlots];  // scales consumed (256 arrivals: both groups, active or not)
  alignas(16) float skt[kSkSlots][kBN];
};

// Bounded wait on an mbarrier phase; the common "already complete" case costs one try_wait.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, Shared* sh, int code) {
  return bounded_wait(bar, parity, &sh->abort_flag, &g_fwd_sm100_status, code);
}

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr int code = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr int code = 1; };

static_assert(sizeof(Shared) <= 4096, "Shared must fit its reserve");

}  // namespace

// kInt8: Q and K are int8 codes (tensor maps over the code buffers, 1 byte per element), QK^T is
// tcgen05.mma.kind::i8 with an int32 accumulator, and the per-row / per-key scales sq, sk are
// folded into the score epilogue; P@V stays in T.
template <typename T, int D, bool kExtras, bool kInt8>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                 const fa_attn_args p, const ScoreCfg cfg, const float* __restrict__ sq,
                 const float* __restrict__ sk, int* const host_status) {
  static_assert(!kInt8 || D == 128, "the INT8 variant stages 128-byte code rows");
  // measured: 2-3 % faster on the plain variants, 2 % slower on the feature variant (whose
  // element-wise phase is three times as long, so the extra wait for the store costs more than
  // the early start gains)
  constexpr bool kPvSplit = kPvSplitOn && !kExtras;
  using C = Cfg<D>;
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Shared* sh = reinterpret_cast<Shared*>(tiles + C::kSmemTiles);
  const uint32_t sQ = smem_u32(tiles);                 // + x * kTileBytes
  const uint32_t sKV = sQ + 2 * C::kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int mblk = cfg.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;  // heavy blocks first
  const SeqInfo si = seq_info(p, b);
  const int m00 = mblk * 2 * kBM;
  if (m00 >= si.q_len) return;
  const int hk = h / (p.heads_q / p.heads_kv);
  const int off = p.q_pos_offset;

  // Key tiles [nlo[x], nhi[x]) that the rows of stream x can see, and their union [n_lo, n_hi).
  // Step j works on tile n_hi - 1 - j; stream x is active for the steps [jb[x], je[x]).
  auto tile_range = [&](int m0, int& lo, int& hi) {
    lo = hi = 0;
    if (m0 < si.q_len) {
      int klo, khi;
      visible_key_range(cfg, m0 + off, min(m0 + kBM, si.q_len) - 1 + off, si.k_len, klo, khi);
      if (khi > klo) {
        lo = klo / kBN;
        hi = (khi + kBN - 1) / kBN;
      }
    }
  };
  int nlo0, nhi0, nlo1, nhi1;
  tile_range(m00, nlo0, nhi0);
  tile_range(m00 + kBM, nlo1, nhi1);
  const bool has0 = nhi0 > nlo0, has1 = nhi1 > nlo1;
  const int n_lo = has0 ? (has1 ? min(nlo0, nlo1) : nlo0) : nlo1;
  const int n_hi = has0 ? (has1 ? max(nhi0, nhi1) : nhi0) : nhi1;
  const int nsteps = (has0 || has1) ? n_hi - n_lo : 0;
  const int jb0 = has0 ? n_hi - nhi0 : 0, je0 = has0 ? n_hi - nlo0 : 0;
  const int jb1 = has1 ? n_hi - nhi1 : 0, je1 = has1 ? n_hi - nlo1 : 0;
  const bool q1_loaded = m00 + kBM < si.q_len;         // the second query tile exists

  if (tid == 0) {
    mbar_init(smem_u32(&sh->q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sh->s_full[i]), 1);
      mbar_init(smem_u32(&sh->o_ready[i]), 1);
      mbar_init(smem_u32(&sh->p_ready[i]), 128);
      mbar_init(smem_u32(&sh->p_half[i]), 128);
    }
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(smem_u32(&sh->kv_full[i]), 1);
      mbar_init(smem_u32(&sh->kv_empty[i]), 1);
    }
    for (int i = 0; i < kSkSlots; ++i) {
      mbar_init(smem_u32(&sh->sk_full[i]), 1);
      mbar_init(smem_u32(&sh->sk_empty[i]), 256);
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

  if (warp >= 10) {
    // idle warps of the producer/MMA warpgroup; in the INT8 variant warp 10 stages the key
    // scales of the key tile of step j into shared memory (slot j & 1)
    reg_dealloc<72>();
    if (kInt8 && warp == 10) {
      const int64_t bh_rows = ((int64_t)b * p.heads_q + h) * p.total_k;   // rows of the scale arrays per (batch, head)
      for (int j = 0; j < nsteps; ++j) {
        const int buf = j % kSkSlots;
        bool w = true;
        if (lane == 0) w = wait_bar(&sh->sk_empty[buf], ((j / kSkSlots) & 1) ^ 1, sh, 12);
        if (!__all_sync(0xffffffffu, w)) break;
        // staged pre-multiplied by softmax_scale * log2(e), so the consumers need two products
        for (int i = lane; i < kBN; i += 32) {
          const int col = (n_hi - 1 - j) * kBN + i;
          sh->skt[buf][i] = (col < si.k_len ? sk[bh_rows + col] : 1.f) * (cfg.scale * 1.44269504f);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->sk_full[buf]));
      }
    }
  } else if (warp == 8) {
    // ------------------------------- TMA producer ---------------------------------------
    reg_dealloc<72>();
    if (lane == 0 && nsteps > 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      prefetch_tmap(&tmO);
      const int krow0 = (int)si.k_row0;
      const int kb = (int)si.k_boff;
      {
        const uint32_t bar = smem_u32(&sh->q_full);
        const int ntile = q1_loaded ? 2 : 1;
        if (kInt8) {
          mbar_expect_tx(bar, ntile * kBM * D);
          for (int x = 0; x < ntile; ++x)
            tma_load_4d(sQ + x * C::kTileBytes, &tmQ, bar, 0, h, (int)si.q_row0 + m00 + x * kBM, (int)si.q_boff);
        } else {
          mbar_expect_tx(bar, ntile * C::kTileBytes);
          for (int x = 0; x < ntile; ++x)
            for (int bx = 0; bx < C::kBoxes; ++bx)
              tma_load_4d(sQ + x * C::kTileBytes + bx * (kBM * 128), &tmQ, bar, bx * 64, h,
                          (int)si.q_row0 + m00 + x * kBM, (int)si.q_boff);
        }
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto load_kv = [&](const CUtensorMap* tm, int tile, bool codes) {
        if (!ok) return;
        ok = wait_bar(&sh->kv_empty[stage], phase ^ 1, sh, 11);
        if (!ok) return;
        const uint32_t bar = smem_u32(&sh->kv_full[stage]);
        if (codes) {  // int8 K tile: one box of 128-byte rows
          mbar_expect_tx(bar, kBN * D);
          tma_load_4d(sKV + stage * C::kTileBytes, tm, bar, 0, hk, krow0 + tile * kBN, kb);
        } else {
          mbar_expect_tx(bar, C::kTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sKV + stage * C::kTileBytes + bx * (kBN * 128), tm, bar, bx * 64, hk,
                        krow0 + tile * kBN, kb);
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      };
      // order of use: K_0, then V_j, K_{j+1}
      load_kv(&tmK, n_hi - 1, kInt8);
      for (int j = 0; j < nsteps; ++j) {
        load_kv(&tmV, n_hi - 1 - j, false);
        if (j + 1 < nsteps) load_kv(&tmK, n_hi - 2 - j, kInt8);
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -----------------------------------------
    // The whole warp runs the control flow in lock step and every lane polls the barriers;
    // the lane chosen once by elect_one issues the MMAs and commits.
    reg_dealloc<72>();
    if (nsteps > 0) {
      constexpr uint32_t idesc_qk = make_idesc(1, Fmt<T>::code, 0, 0, kBM, kBN);
      constexpr uint32_t idesc_pv = make_idesc(1, Fmt<T>::code, 0, 1, kBM, D);
      const uint32_t leader = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto wwait = [&](uint64_t* bar, uint32_t parity, int code) {
        if (ok) ok = wait_bar(bar, parity, sh, code);
        tc_fence_after();
      };
      auto advance = [&]() { if (++stage == C::kStages) { stage = 0; phase ^= 1; } };
      // S[x] = Q_x K^T with the K tile at kbase
      auto issue_qk = [&](int x, uint32_t kbase) {
        const uint64_t dq = make_smem_desc(sQ + x * C::kTileBytes, 16, 1024);
        const uint64_t dk = make_smem_desc(kbase, 16, 1024);
        if (kInt8) {
          constexpr uint32_t idesc_i8 = make_idesc(2, 1, 0, 0, kBM, kBN);  // s32 <- s8 x s8
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < D / 32; ++kk)
              mma_i8_ss(tmem + x * kBN, dq + ((kk * 32) >> 4), dk + ((kk * 32) >> 4), idesc_i8, kk > 0);
          }
          __syncwarp();
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t o = ((kk / 4) * (kBM * 128) + (kk % 4) * 32) >> 4;
            mma_f16_ss_lp(tmem + x * kBN, dq + o, dk + o, idesc_qk, kk > 0, leader);
          }
        }
        mma_commit_lp(smem_u32(&sh->s_full[x]), leader);
      };
      int pcnt0 = 0, pcnt1 = 0;   // P tiles consumed so far, per stream
      wwait(&sh->q_full, 0, 21);
      wwait(&sh->kv_full[stage], phase, 22);
      if (ok) {
        const uint32_t kbase = sKV + stage * C::kTileBytes;
        if (jb0 == 0 && je0 > 0) issue_qk(0, kbase);
        if (jb1 == 0 && je1 > 0) issue_qk(1, kbase);
        mma_commit_lp(smem_u32(&sh->kv_empty[stage]), leader);
        advance();
      }
      for (int j = 0; j < nsteps && ok; ++j) {
        wwait(&sh->kv_full[stage], phase, 24);          // V_j
        if (!ok) break;
        const int vstage = stage;
        const uint32_t vbase = sKV + stage * C::kTileBytes;
        advance();
        const bool more = j + 1 < nsteps;
        const int kstage = stage;
        const uint32_t kbase = sKV + stage * C::kTileBytes;
        bool k_waited = false;
        auto do_stream = [&](int x, int sjb, int sje, int& pcnt) {
          if (j >= sjb && j < sje) {
            const uint32_t a = tmem + x * kBN;
            const uint64_t dv = make_smem_desc(vbase, kBN * 128, 1024);
            if (kPvSplit) {
              wwait(&sh->p_half[x], pcnt & 1, 25 + x);
              if (!ok) return;
#pragma unroll
              for (int kk = 0; kk < kBN / 32; ++kk)
                mma_f16_ts_lp(tmem + 256 + x * 128, a + kk * 8, dv + ((kk * 2048) >> 4), idesc_pv,
                              (j > sjb || kk > 0) ? 1u : 0u, leader);
            }
            wwait(&sh->p_ready[x], pcnt & 1, 25 + x);
            if (!ok) return;
            ++pcnt;
#pragma unroll
            for (int kk = kPvSplit ? kBN / 32 : 0; kk < kBN / 16; ++kk)
              mma_f16_ts_lp(tmem + 256 + x * 128, a + kk * 8, dv + ((kk * 2048) >> 4), idesc_pv,
                            (j > sjb || kk > 0) ? 1u : 0u, leader);
            mma_commit_lp(smem_u32(&sh->o_ready[x]), leader);
          }
          if (more && j + 1 >= sjb && j + 1 < sje) {
            if (!k_waited) {
              wwait(&sh->kv_full[kstage], phase, 22);   // K_{j+1}
              if (!ok) return;
              k_waited = true;
            }
            issue_qk(x, kbase);
          }
        };
        do_stream(0, jb0, je0, pcnt0);
        if (ok) do_stream(1, jb1, je1, pcnt1);
        if (!ok) break;
        mma_commit_lp(smem_u32(&sh->kv_empty[vstage]), leader);
        if (more) {
          // a K tile that no stream needs (cannot happen for contiguous visible ranges) would
          // still have to be consumed to keep the ring in step
          if (!k_waited) wwait(&sh->kv_full[kstage], phase, 22);
          mma_commit_lp(smem_u32(&sh->kv_empty[kstage]), leader);
          advance();
        }
      }
    }
  } else {
    // ------------------------------- softmax groups -------------------------------------
    reg_alloc<216>();
    PROF_VARS(12);
#ifdef FA_PROF
    const long long prof_start = clock64();
    long long prof_t1 = 0;
#endif
    const int x = warp >> 2;                         // stream = query tile of the CTA
    const int m0 = m00 + x * kBM;
    const int row_in_tile = (warp & 3) * 32 + lane;  // TMEM lane
    const int row = m0 + row_in_tile;                // query row inside the sequence
    const int qpos = row + off;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tSx = tmem + lane_addr + x * kBN;
    const uint32_t tOx = tmem + lane_addr + 256 + x * 128;
    const float slope = (kExtras && cfg.has_alibi) ? p.alibi_slopes[b * p.heads_q + h] : 0.f;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    const int tq_min = m0 + off, tq_max = tq_min + kBM - 1;
    // INT8: scale of this query row and the row of key scales of this (batch, head)
    const int64_t bh_rows = ((int64_t)b * p.heads_q + h) * p.total_k;
    const float sq_row = (kInt8 && row < si.q_len) ? sq[bh_rows + row] : 1.f;
    const int my_jb = x ? jb1 : jb0, my_je = x ? je1 : je0;

    for (int j = kInt8 ? 0 : my_jb; j < (kInt8 ? nsteps : my_je) && ok; ++j) {
      if (kInt8 && (j < my_jb || j >= my_je)) {
        // not this stream's tile, but the slot of its key scales is released by both groups
        ok = wait_bar(&sh->sk_full[j % kSkSlots], (j / kSkSlots) & 1, sh, 37 + x);
        if (ok) mbar_arrive(smem_u32(&sh->sk_empty[j % kSkSlots]));
        continue;
      }
      const int t = j - my_jb;                       // index of the tile inside this stream
      const int k0 = (n_hi - 1 - j) * kBN;
      bool masked = (k0 + kBN > si.k_len);
      if (cfg.causal) masked |= (k0 + kBN - 1 > tq_min);
      if (cfg.wl >= 0) masked |= (k0 < tq_max - cfg.wl);
      if (cfg.wr >= 0) masked |= (k0 + kBN - 1 > tq_min + cfg.wr);

      PROF_T0();
      ok = wait_bar(&sh->s_full[x], t & 1, sh, 31 + x);
#ifdef FA_PROF
      if (t == 0) PROF_ADD(1); else PROF_ADD(0);
      prof_t1 = clock64();
      PROF_COUNT(masked ? 9 : 8, 1);
#endif
      if (!ok) break;
      tc_fence_after();

      // ---- the 128 scores of this row into registers -------------------------------------
      uint32_t r[4][32];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) tmem_ld32(tSx + cc * 32, r[cc]);
      tmem_wait_ld();

      const bool prescaled = kExtras || masked || kInt8;
      // columns (keys) of this tile that this thread's query row sees (used by masked tiles only)
      ColMask cm;
      if (masked) {
        int vk_lo, vk_hi;
        visible_k_interval(cfg, qpos, si.k_len, vk_lo, vk_hi);
        cm = make_col_mask(vk_lo - k0, vk_hi - k0);
      }
      if (kInt8) {
        // score = float(acc) * s_q * (s_k * softmax_scale * log2 e): the same product as the
        // reference's (acc * (s_q * s_k)) * (scale * log2 e) up to the last rounding.
        // |acc| <= 128*127*127 < 2^22, so int -> float is exact through the 1.5*2^23 bias
        // (an integer add and a float subtract instead of a quarter-rate I2F); packed pairs.
        ok = wait_bar(&sh->sk_full[j % kSkSlots], (j / kSkSlots) & 1, sh, 37 + x);
        if (!ok) break;
        const float4* S4 = reinterpret_cast<const float4*>(&sh->skt[j % kSkSlots][0]);
        const float2 nb2 = make_float2(-12582912.0f, -12582912.0f);
        // Two copies of the loop: without the per-element mask test there are no branches inside,
        // so the compiler can issue the shared-memory loads of the scales in batches (each one
        // takes hundreds of cycles while the tensor pipe streams its operands).
        auto scale_tile = [&](auto mask_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 s4 = S4[cc * 8 + i4];
              const int i = i4 * 4;
              const float2 a01 = f2add(make_float2(__uint_as_float(0x4B400000u + r[cc][i]),
                                                   __uint_as_float(0x4B400000u + r[cc][i + 1])), nb2);
              const float2 a23 = f2add(make_float2(__uint_as_float(0x4B400000u + r[cc][i + 2]),
                                                   __uint_as_float(0x4B400000u + r[cc][i + 3])), nb2);
              // the per-query scale (positive, one value per thread) is applied after the maximum,
              // inside the FMA that forms the exp2 argument
              const float2 v01 = f2mul(a01, make_float2(s4.x, s4.y));
              const float2 v23 = f2mul(a23, make_float2(s4.z, s4.w));
              float v[4] = {v01.x, v01.y, v23.x, v23.y};
              if (kMask) {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = col_visible(cm, cc * 32 + i + e) ? v[e] : -INFINITY;
              }
#pragma unroll
              for (int e = 0; e < 4; ++e) r[cc][i + e] = __float_as_uint(v[e]);
            }
          }
        };
        if (masked) scale_tile(std::true_type{});
        else scale_tile(std::false_type{});
        mbar_arrive(smem_u32(&sh->sk_empty[j % kSkSlots]));
      } else if (prescaled) {
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
      // (ring entry 2 j + 1 in order of use K0 V0 K1 V1 ...) before P is handed to the issuer.
      // One thread per row; a row is D contiguous 16-bit values per 64-wide box, so the swizzle
      // does not matter.  Both streams may do it for the same tile (zeros over zeros).
      if (!kInt8 && p.cu_seqlens_k != nullptr && k0 + kBN > si.k_len) {
        const int vpos = 2 * j + 1;
        ok = wait_bar(&sh->kv_full[vpos % C::kStages], (vpos / C::kStages) & 1, sh, 39);
        if (!ok) break;
        if (k0 + row_in_tile >= si.k_len) {
          unsigned char* vrow = tiles + C::kTileBytes * (2 + vpos % C::kStages) + row_in_tile * 128;
#pragma unroll
          for (int bx = 0; bx < C::kBoxes; ++bx) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
              reinterpret_cast<uint4*>(vrow + bx * (kBN * 128))[c] = make_uint4(0u, 0u, 0u, 0u);
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
      if (kInt8) mx *= sq_row;               // s_q > 0

#ifdef FA_PROF
      prof_acc[masked ? 3 : 2] += (unsigned int)(clock64() - prof_t1);   // load + score + max phase
      prof_t1 = clock64();
#endif
      // ---- lazy rescale ----------------------------------------------------------------
      if (t == 0) {
        m_used = mx;
      } else {
        const bool need = mx > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // The previous P V of this stream is its (t-1)-th; the one of this tile cannot
          // complete before P is written below, so the barrier is at most one phase ahead
          // of the parity waited for here.
          ok = wait_bar(&sh->o_ready[x], (t - 1) & 1, sh, 33 + x);
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
#ifdef FA_PROF
      prof_acc[4] += (unsigned int)(clock64() - prof_t1);                 // rescale (incl. its wait)
      prof_t1 = clock64();
#endif
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;

      // ---- P = exp2(s - m), row sum, P -> TMEM in place over S ----------------------------
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
      if (kInt8) {
        // Outlier keys make the rows peaky; with a stale reference maximum the dominant
        // probability is 2^x instead of exactly 1, so its rounding to T would not cancel
        // in O / l unless l sums the ROUNDED values that enter P@V.
        const float2 nm2 = make_float2(-m_safe, -m_safe), sq2 = make_float2(sq_row, sq_row);
        float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 a = f2fma(make_float2(__uint_as_float(r[cc][i]), __uint_as_float(r[cc][i + 1])), sq2, nm2);
            pk[i >> 1] = Elem<T>::pack(ex2(a.x), ex2(a.y));
            acc2[(i >> 1) & 1] = f2add(acc2[(i >> 1) & 1], Elem<T>::unpack(pk[i >> 1]));
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
        ps[0] = acc2[0].x; ps[1] = acc2[0].y; ps[2] = acc2[1].x; ps[3] = acc2[1].y;
      } else {
        // packed pairs: one FMA, two exponentials, one conversion and one add per two scores
        const float2 mul2 = make_float2(mul, mul), nm2 = make_float2(-m_safe, -m_safe);
        float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 a = f2fma(make_float2(__uint_as_float(r[cc][i]), __uint_as_float(r[cc][i + 1])), mul2, nm2);
            // the unmasked fast path holds no -inf scores: part of its exponentials may run on the FMA pipe
            const float2 pe = prescaled ? make_float2(ex2(a.x), ex2(a.y)) : ex2_pair<kPolyEvery>(a, i >> 1);
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
        ps[0] = acc2[0].x; ps[1] = acc2[0].y; ps[2] = acc2[1].x; ps[3] = acc2[1].y;
      }
      l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->p_ready[x]));
#ifdef FA_PROF
      prof_acc[5] += (unsigned int)(clock64() - prof_t1);                 // exp + store phase
#endif
    }

    // ---- epilogue: O / l -> global, base-2 LSE ------------------------------------------
    const int my_tiles = my_je - my_jb;
#ifdef FA_PROF
    prof_acc[6] = (unsigned int)(clock64() - prof_start);                 // start of role -> end of main loop
    prof_t1 = clock64();
#endif
    if (ok && my_tiles > 0) ok = wait_bar(&sh->o_ready[x], (my_tiles - 1) & 1, sh, 35 + x);
    // A stream without key tiles writes zeros over its Q tile straight away: the TMA load of
    // both Q tiles (issued whenever the CTA has steps) must have landed first, or it would
    // overwrite the staged zeros.
    if (ok && my_tiles == 0 && nsteps > 0) ok = wait_bar(&sh->q_full, 0, sh, 37);
    tc_fence_after();
    if (m0 < si.q_len && ok && sh->abort_flag == 0) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = row < si.q_len;
      // The tile is staged in shared memory (over this stream's Q tile, which no MMA reads any
      // more) in the swizzled box layout and written by the TMA unit as full rows; a packed
      // tile that reaches past the end of its sequence is stored row by row instead (the unit
      // would write the neighbour's rows).
      const bool via_tma = (p.cu_seqlens_q == nullptr) || (m0 + kBM <= si.q_len);
      const uint32_t sOx = sQ + x * C::kTileBytes;
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
#ifdef FA_PROF
    prof_acc[7] = (unsigned int)(clock64() - prof_t1);                    // epilogue
    prof_acc[10] = 1;
    PROF_FLUSH((tid & 127) == 0, (warp >> 2) * 16, 12);
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
  if (tid == 0) report_abort(sh->abort_flag, host_status);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
bool fwd_sm100_supported(const fa_attn_args& a) {
  if (a.head_dim != 128 && a.head_dim != 64) return false;
  if (a.softmax_scale < 0.f) return false;
  if (a.batch == 0 || a.seqlen_q == 0 || a.seqlen_k == 0) return false;
  // tiny problems are launch-bound; the warp-level kernel has less fixed cost
  if (a.impl == FA_IMPL_AUTO && a.seqlen_k < 256) return false;
  return true;
}

static bool make_map(CUtensorMap* m, const void* base, const int64_t* stride, int rows, int heads,
                     int batch, int D, bool packed) {
  // dims (innermost first): head_dim, heads, rows, batch
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)rows, (uint64_t)(packed ? 1 : batch)};
  const uint64_t strides[3] = {(uint64_t)stride[2] * 2, (uint64_t)stride[1] * 2,
                               (uint64_t)(packed ? (int64_t)rows * stride[1] : stride[0]) * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap(m, base, 2, 4, dims, strides, box);
}

template <typename T, int D>
static int launch(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st, int q_rows, int k_rows) {
  using C = Cfg<D>;
  CUtensorMap tq, tk, tv, to;
  const bool packed = a.cu_seqlens_q != nullptr;
  if (!make_map(&to, a.o, a.o_stride, q_rows, a.heads_q, a.batch, D, packed) ||
      !make_map(&tq, a.q, a.q_stride, q_rows, a.heads_q, a.batch, D, packed) ||
      !make_map(&tk, a.k, a.k_stride, k_rows, a.heads_kv, a.batch, D, packed) ||
      !make_map(&tv, a.v, a.v_stride, k_rows, a.heads_kv, a.batch, D, packed)) {
    set_error("fwd_sm100: cuTensorMapEncodeTiled failed");
    return FA_ERR_LAUNCH;
  }
  const bool extras = cfg.has_alibi || cfg.softcap > 0.f;
  auto kern = extras ? fwd_sm100_kernel<T, D, true, false> : fwd_sm100_kernel<T, D, false, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) {
    set_error("fwd_sm100: cudaFuncSetAttribute(%d): %s", C::kSmemBytes, cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  dim3 grid((a.seqlen_q + 2 * kBM - 1) / (2 * kBM), a.heads_q, a.batch);
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, to, a, cfg, nullptr, nullptr, host_wait_word(a.device));
  return check_launch("fwd_sm100");
}

// Two kernels.  The persistent one (fwd_persist_sm100.cu) takes the calls with long work items:
// measured with launches interleaved on one GPU it is 3-4 % faster at 4096-8192 keys (dense, GQA
// and the packed workload) and 9 % slower at 1024 keys, where an item is four or five steps and
// the hand-over between items costs more than a fresh CTA.  This file keeps the one-CTA-per-item
// kernel for those, and for the INT8 variant.
#ifndef FA_FWD_PERSISTENT_FROM
#define FA_FWD_PERSISTENT_FROM 2048   // keys (dense: seqlen_k, packed: max_seqlen_k); 0 = never
#endif
int fwd_persist_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st);
int fwd_persist_sm100_status();
int fwd_persist_sm100_clear_status();

int fwd_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  // FA_B200_FWD_PERSISTENT_FROM in the environment overrides the threshold (tests run the
  // persistent kernel on small shapes with it; 0 = never)
  int from = FA_FWD_PERSISTENT_FROM;
  if (const char* e = getenv("FA_B200_FWD_PERSISTENT_FROM")) from = atoi(e);
  if (from > 0 && a.seqlen_k >= from) return fwd_persist_sm100(a, cfg, st);
  // Row extents of the tensor maps.  Dense: the sequence length.  Packed: the caller does
  // not pass the total token count, so the map covers rows up to the int32 limit of the
  // cu_seqlens; tiles never start past cu_seqlens[batch], and rows past a sequence's end
  // are masked (keys) or not stored (queries).
  const bool packed = a.cu_seqlens_q != nullptr;
  const int q_rows = packed ? a.total_q : a.seqlen_q;
  const int k_rows = packed ? a.total_k : a.seqlen_k;
  if (a.head_dim == 128)
    return a.dtype == FA_BF16 ? launch<__nv_bfloat16, 128>(a, cfg, st, q_rows, k_rows)
                              : launch<__half, 128>(a, cfg, st, q_rows, k_rows);
  return a.dtype == FA_BF16 ? launch<__nv_bfloat16, 64>(a, cfg, st, q_rows, k_rows)
                            : launch<__half, 64>(a, cfg, st, q_rows, k_rows);
}

// ---------------------------------------------------------------------------------------
// INT8-QK^T forward on contiguous (batch, heads, seqlen, 128) tensors
// ---------------------------------------------------------------------------------------
int quantize_q(const void* q, int8_t* q8, float* s_q, int64_t rows, int head_dim, cudaStream_t st);

bool fwd_int8_sm100_supported(const fa_int8_args& a) {
  if (a.head_dim != 128 || a.softmax_scale < 0.f) return false;
  if (a.q8_scratch == nullptr || a.sq_scratch == nullptr) return false;
  if (a.impl == FA_IMPL_AUTO && a.seqlen < 256) return false;
  return true;
}

int fwd_int8_sm100(const fa_int8_args& a, cudaStream_t st) {
  constexpr int D = 128;
  using C = Cfg<D>;
  const int64_t rows = (int64_t)a.batch * a.heads * a.seqlen;
  if (int r = quantize_q(a.q, a.q8_scratch, a.sq_scratch, rows, D, st)) return r;
  const int B = a.batch, H = a.heads, S = a.seqlen;
  CUtensorMap tq, tk, tv, to;
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    const uint64_t s8[3] = {(uint64_t)S * D, (uint64_t)D, (uint64_t)H * S * D};
    const uint64_t s16[3] = {(uint64_t)S * D * 2, (uint64_t)D * 2, (uint64_t)H * S * D * 2};
    const uint32_t box8[4] = {128, 1, 128, 1}, box16[4] = {64, 1, 128, 1};
    if (!encode_tmap(&tq, a.q8_scratch, 1, 4, dims, s8, box8) || !encode_tmap(&tk, a.k8, 1, 4, dims, s8, box8) ||
        !encode_tmap(&tv, a.v, 2, 4, dims, s16, box16) || !encode_tmap(&to, a.o, 2, 4, dims, s16, box16)) {
      set_error("fwd_int8_sm100: cuTensorMapEncodeTiled failed");
      return FA_ERR_LAUNCH;
    }
  }
  fa_attn_args p;
  memset(&p, 0, sizeof(p));
  p.dtype = FA_F16;
  p.device = a.device;
  p.batch = B; p.seqlen_q = S; p.heads_q = H; p.heads_kv = H; p.head_dim = D;
  p.seqlen_k = a.seqlen_k_valid > 0 ? a.seqlen_k_valid : S;   // keys past it are padding (masked, tiles skipped)
  p.total_q = p.total_k = S;                                  // rows of q8 / k8 and of the scale arrays
  p.q_pos_offset = a.q_pos_offset;
  p.o = a.o;
  p.o_stride[0] = (int64_t)H * S * D; p.o_stride[1] = D; p.o_stride[2] = (int64_t)S * D;
  p.lse2 = a.lse2;
  p.lse_stride[0] = (int64_t)H * S; p.lse_stride[1] = 1; p.lse_stride[2] = S;
  p.softmax_scale = a.softmax_scale;
  p.causal = a.causal;
  p.window_left = p.window_right = -1;
  const ScoreCfg cfg = make_score_cfg(a.softmax_scale, 0.f, a.causal, -1, -1, false);
  auto kern = fwd_sm100_kernel<__half, D, false, true>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) {
    set_error("fwd_int8_sm100: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  dim3 grid((S + 2 * kBM - 1) / (2 * kBM), H, B);
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, to, p, cfg, a.sq_scratch, a.s_k, host_wait_word(a.device));
  return check_launch("fwd_int8_sm100");
}


int fwd_sm100_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_fwd_sm100_status, sizeof(int));
  return v != 0 ? v : fwd_persist_sm100_status();
}

void fwd_sm100_clear_status() {
  const int z = 0;
  cudaMemcpyToSymbol(g_fwd_sm100_status, &z, sizeof(int));
  fwd_persist_sm100_clear_status();
}

// One warp waits, for at most `clocks` cycles, on a barrier nothing arrives at: the time-out path
// of bounded_wait with nothing else in flight.
__global__ void wait_probe_kernel(long long clocks, int* host_status) {
  __shared__ uint64_t bar;
  __shared__ volatile int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncwarp();
  bounded_wait<0>(&bar, 0, &abort_flag, &g_fwd_sm100_status, 99, clocks);
  __syncwarp();
  if (threadIdx.x == 0) report_abort(abort_flag, host_status);
}

// Rate of the tensor pipe as this library drives it: every CTA (one per SM) issues `iters`
// back-to-back tcgen05.mma of shape M128 N128 (K16 fp16 or K32 int8) on operand tiles that sit
// in shared memory, into four accumulators in turn.  The host times the launch; the result is the
// denominator for kernels that mix int8 and fp16 GEMMs (cuBLAS only gives the bf16 figure).
template <bool kInt8>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t done;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  // operand tiles: 128 rows of 128 bytes each (A and B), filled with small pseudo-random values
  for (int i = tid; i < 2 * 128 * 128 / 4; i += 128) {
    uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x;
    reinterpret_cast<uint32_t*>(tiles)[i] = kInt8 ? (x & 0x0f0f0f0fu) : (0x2c002c00u | (x & 0x03ff03ffu));
  }
  if (tid == 0) {
    mbar_init(smem_u32(&done), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  fence_proxy_async();
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base;
  if (warp == 1) {
    const uint32_t leader = elect_one() ? 1u : 0u;
    const uint32_t sA = smem_u32(tiles), sB = sA + 128 * 128;
    const uint64_t da = make_smem_desc(sA, 16, 1024), db = make_smem_desc(sB, 16, 1024);
    constexpr uint32_t idesc = kInt8 ? make_idesc(2, 1, 0, 0, 128, 128) : make_idesc(1, 0, 0, 0, 128, 128);
    for (int it = 0; it < iters; ++it) {
      const uint32_t o = (uint32_t)((it & 3) * 32) >> 4;            // the four K steps of a 128-byte row
      if (kInt8) {
        if (leader) mma_i8_ss(tmem + ((it >> 2) & 3) * 128, da + o, db + o, idesc, 1u);
        __syncwarp();
      } else {
        mma_f16_ss_lp(tmem + ((it >> 2) & 3) * 128, da + o, db + o, idesc, 1u, leader);
      }
    }
    mma_commit_lp(smem_u32(&done), leader);
    bounded_wait(&done, 0, &abort_flag, &g_fwd_sm100_status, 98);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

int mma_peak_probe(int device, int kind, int iters, cudaStream_t st) {
  const int smem = 2 * 128 * 128 + 1024;
  const int grid = sm_count(device);
  if (kind == 1) mma_peak_kernel<true><<<grid, 128, smem, st>>>(iters);
  else mma_peak_kernel<false><<<grid, 128, smem, st>>>(iters);
  return check_launch("mma_peak_probe");
}

int wait_probe(int device, long long clocks, cudaStream_t st) {
  wait_probe_kernel<<<1, 32, 0, st>>>(clocks, host_wait_word(device));
  return check_launch("wait_probe");
}

}  // namespace fa
