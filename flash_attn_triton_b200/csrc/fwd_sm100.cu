// Forward attention on the 5th-generation tensor cores: TMA-staged tiles, tcgen05.mma with
// accumulators in tensor memory, warp-specialised online softmax.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles.  Keys are consumed
// in half-steps of 64; every Q tile has TWO score buffers in tensor memory, so the MMA of
// half-step i+1 is already queued while the softmax warps work on half-step i, and the
// tensor pipe and the exp units overlap instead of waiting for each other:
//
//   warps 0-3   softmax group of tile 0 : one query row per thread (TMEM lane = row)
//   warps 4-7   softmax group of tile 1
//   warp  8     TMA producer            : Q tiles once, then K/V tiles through a ring
//   warp  9     MMA issuer (one thread) : S_t = Q_t K^T (SS), O_t += P_t V (A = P from TMEM)
//   warps 10-11 idle; they complete the third warpgroup so that it can hand its registers
//               to the softmax groups (setmaxnreg)
//
// TMEM (512 columns): S0a S0b | S1a S1b | O0 | O1 (score buffers 64 fp32 columns each,
// O head_dim columns).  P (fp16/bf16) overwrites the first 32 columns of its score buffer.  The running row maximum is only
// raised when it grows by more than 2^8 ("lazy rescale"), so the O accumulator in TMEM is
// rarely touched by the softmax warps; exactness is kept because O and the row sum always
// share the same reference maximum.
//
// Shared memory: Q0,Q1 (128 x D each) + a ring of K/V tiles (128 keys x D), every tile
// written by TMA with the 128-byte swizzle the MMA descriptors expect.
//
// Every mbarrier wait is bounded; on timeout the CTA raises a device-side status word,
// releases its TMEM and returns.
#include "common.cuh"
#include "sm100.cuh"

namespace fa {

using namespace sm100;

__device__ int g_fwd_sm100_status = 0;

namespace {

constexpr int kBM = 128;          // rows per Q tile
constexpr int kBN = 128;          // keys per K/V tile
constexpr int kThreads = 384;     // 8 softmax warps + a warpgroup holding producer and MMA warps
constexpr float kRescaleThreshold = 8.0f;

template <int D> struct Cfg {
  static constexpr int kTileBytes = kBN * D * 2;                    // one Q/K/V tile
  static constexpr int kStages = (D == 128) ? 4 : 6;                // K/V ring depth
  static constexpr int kBoxes = D / 64;                             // TMA boxes per tile
  static constexpr int kSmemTiles = (2 + kStages) * kTileBytes;
  static constexpr int kSmemBytes = kSmemTiles + 1024 /*align slack*/ + 256 /*barriers*/;
};

constexpr int kHalf = 64;         // keys per half-step

struct Shared {
  uint64_t q_full[2];
  uint64_t kv_full[6];
  uint64_t kv_empty[6];
  uint64_t s_full[2][2];   // [tile][buffer]
  uint64_t p_ready[2][2];  // [tile][buffer]
  uint64_t o_ready[2][2];  // [tile][parity of the PV index]: see the note at the waits
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, Shared* sh, int code) {
  const uint32_t a = smem_u32(bar);
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(a, parity)) return true;
    if ((it & 255u) == 255u) {
      if (sh->abort_flag) return false;
      if (clock64() - t0 > 4000000000LL) {  // ~2 s
        sh->abort_flag = code;
        atomicExch(&g_fwd_sm100_status, code);
        return false;
      }
    }
  }
}

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr int code = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr int code = 1; };

}  // namespace

template <typename T, int D, bool kExtras>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const fa_attn_args p, const ScoreCfg cfg) {
  using C = Cfg<D>;
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Shared* sh = reinterpret_cast<Shared*>(tiles + C::kSmemTiles);
  const uint32_t sQ = smem_u32(tiles);
  const uint32_t sKV = sQ + 2 * C::kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int mblk = cfg.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;  // heavy blocks first
  const SeqInfo si = seq_info(p, b);
  const int m0 = mblk * 2 * kBM;
  if (m0 >= si.q_len) return;
  const int hk = h / (p.heads_q / p.heads_kv);
  const int off = p.q_pos_offset;

  // Half-step ranges [glo_t, ghi_t) of the two Q tiles (half-step g covers keys
  // [64g, 64g+64)), their union, and the K/V tiles (128 keys) the union touches.
  int glo_t[2], ghi_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r_first = m0 + t * kBM, r_last = min(r_first + kBM, si.q_len) - 1;
    if (r_last < r_first) {
      glo_t[t] = ghi_t[t] = 0;
    } else {
      int klo, khi;
      visible_key_range(cfg, r_first + off, r_last + off, si.k_len, klo, khi);
      glo_t[t] = klo / kHalf;
      ghi_t[t] = (khi + kHalf - 1) / kHalf;
      if (ghi_t[t] <= glo_t[t]) glo_t[t] = ghi_t[t] = 0;
    }
  }
  const bool any0 = ghi_t[0] > glo_t[0], any1 = ghi_t[1] > glo_t[1];
  const int glo = any0 ? (any1 ? min(glo_t[0], glo_t[1]) : glo_t[0]) : glo_t[1];
  const int ghi = max(any0 ? ghi_t[0] : 0, any1 ? ghi_t[1] : 0);
  const bool any = any0 || any1;
  const int T0 = glo >> 1;                       // first K/V tile
  const int T1 = any ? ((ghi - 1) >> 1) + 1 : T0;  // one past the last K/V tile

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sh->q_full[i]), 1);
      for (int k = 0; k < 2; ++k) {
        mbar_init(smem_u32(&sh->o_ready[i][k]), 1);
        mbar_init(smem_u32(&sh->s_full[i][k]), 1);
        mbar_init(smem_u32(&sh->p_ready[i][k]), 128);
      }
    }
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(smem_u32(&sh->kv_full[i]), 1);
      mbar_init(smem_u32(&sh->kv_empty[i]), 1);
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
    // idle warps of the producer/MMA warpgroup
    reg_dealloc<56>();
  } else if (warp == 8) {
    // ------------------------------- TMA producer ---------------------------------------
    reg_dealloc<56>();
    if (lane == 0 && any) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      const int qrow = (int)si.q_row0 + m0;
      const int krow0 = (int)si.k_row0;
      const int qb = (int)si.q_boff, kb = (int)si.k_boff;
      auto load_q = [&](int t) {
        const uint32_t bar = smem_u32(&sh->q_full[t]);
        mbar_expect_tx(bar, C::kTileBytes);
        for (int x = 0; x < C::kBoxes; ++x)
          tma_load_4d(sQ + t * C::kTileBytes + x * (kBM * 128), &tmQ, bar, x * 64, h, qrow + t * kBM, qb);
      };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // ring order: K[T0], V[T0], K[T0+1], V[T0+1], ...
      auto load_kv = [&](const CUtensorMap* tm, int tile) {
        if (!ok) return;
        ok = wait_bar(&sh->kv_empty[stage], phase ^ 1, sh, 11);
        if (!ok) return;
        const uint32_t bar = smem_u32(&sh->kv_full[stage]);
        mbar_expect_tx(bar, C::kTileBytes);
        for (int x = 0; x < C::kBoxes; ++x)
          tma_load_4d(sKV + stage * C::kTileBytes + x * (kBN * 128), tm, bar, x * 64, hk,
                      krow0 + tile * kBN, kb);
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      };
      load_q(0);
      load_kv(&tmK, T0);
      load_q(1);
      for (int tl = T0; tl < T1; ++tl) {
        load_kv(&tmV, tl);
        if (tl + 1 < T1) load_kv(&tmK, tl + 1);
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -----------------------------------------
    reg_dealloc<56>();
    if (lane == 0 && any) {
      constexpr uint32_t idesc_qk = make_idesc(1, Fmt<T>::code, 0, 0, kBM, kHalf);
      constexpr uint32_t idesc_pv = make_idesc(1, Fmt<T>::code, 0, 1, kBM, D);
      bool ok = true;
      int waited = 0;  // ring slots [0, waited) are known to be full
      // ring slot of K tile tl is 2*(tl-T0), of V tile tl 2*(tl-T0)+1
      auto slot_addr = [&](int slot) { return sKV + (slot % C::kStages) * C::kTileBytes; };
      auto wait_slot = [&](int slot) {
        while (ok && waited <= slot) {
          ok = wait_bar(&sh->kv_full[waited % C::kStages], (waited / C::kStages) & 1, sh, 22);
          ++waited;
        }
        if (ok) tc_fence_after();
      };
      auto release_slot = [&](int slot) { mma_commit(smem_u32(&sh->kv_empty[slot % C::kStages])); };
      int cqk[2] = {0, 0}, cpv[2] = {0, 0};
      // S_t[buf] = Q_t K[g]^T for half-step g
      auto issue_qk = [&](int t, int g) {
        const int slot = 2 * ((g >> 1) - T0);
        wait_slot(slot);
        if (!ok) return;
        const int buf = cqk[t] & 1;
        const uint32_t kbase = slot_addr(slot) + (g & 1) * (kHalf * 128);
        const uint32_t d = tmem + t * 128 + buf * kHalf;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk / 4) * (kBM * 128) + (kk % 4) * 32;
          mma_f16_ss(d, make_smem_desc(sQ + t * C::kTileBytes + o, 16, 1024),
                     make_smem_desc(kbase + o, 16, 1024), idesc_qk, kk > 0);
        }
        mma_commit(smem_u32(&sh->s_full[t][buf]));
        ++cqk[t];
      };
      // O_t += P_t[buf] V[g]
      auto issue_pv = [&](int t, int g) {
        const int slot = 2 * ((g >> 1) - T0) + 1;
        wait_slot(slot);
        if (!ok) return;
        const int buf = cpv[t] & 1;
        ok = wait_bar(&sh->p_ready[t][buf], (cpv[t] >> 1) & 1, sh, 25 + t);
        if (!ok) return;
        tc_fence_after();
        const uint32_t vbase = slot_addr(slot) + (g & 1) * (kHalf * 128);
        const uint32_t a = tmem + t * 128 + buf * kHalf;
#pragma unroll
        for (int kk = 0; kk < kHalf / 16; ++kk)
          mma_f16_ts(tmem + 256 + t * 128, a + kk * 8, make_smem_desc(vbase + kk * 2048, kBN * 128, 1024),
                     idesc_pv, (cpv[t] > 0 || kk > 0) ? 1u : 0u);
        mma_commit(smem_u32(&sh->o_ready[t][cpv[t] & 1]));
        ++cpv[t];
      };
      auto in_range = [&](int t, int g) { return g >= glo_t[t] && g < ghi_t[t]; };
      // A K (V) tile is free once both Q tiles have issued every QK (PV) that reads it; the
      // commit then covers all MMAs issued so far.  Tiles are released in ring order.
      int k_rel = T0, v_rel = T0;
      auto done_upto = [&](const int (&cnt)[2], int tl) {
        return glo_t[0] + cnt[0] >= min(ghi_t[0], 2 * tl + 2) &&
               glo_t[1] + cnt[1] >= min(ghi_t[1], 2 * tl + 2);
      };
      auto release_ready = [&]() {
        while (k_rel < T1 && done_upto(cqk, k_rel)) release_slot(2 * (k_rel++ - T0));
        while (v_rel < T1 && done_upto(cpv, v_rel)) release_slot(2 * (v_rel++ - T0) + 1);
      };

      ok = wait_bar(&sh->q_full[0], 0, sh, 21);
      // prologue: the first two half-steps of each tile
      for (int t = 0; t < 2 && ok; ++t) {
        if (t == 1) ok = wait_bar(&sh->q_full[1], 0, sh, 23);
        for (int g = glo_t[t]; g < min(glo_t[t] + 2, ghi_t[t]) && ok; ++g) {
          issue_qk(t, g);
          if (ok) release_ready();
        }
      }
      for (int g = glo; g < ghi && ok; ++g) {
        for (int t = 0; t < 2 && ok; ++t) {
          if (!in_range(t, g)) continue;
          issue_pv(t, g);
          if (ok && in_range(t, g + 2)) issue_qk(t, g + 2);
          if (ok) release_ready();
        }
      }
    }
  } else {
    // ------------------------------- softmax groups -------------------------------------
    reg_alloc<224>();
    const int t = warp >> 2;                        // Q tile of this group
    const int row_in_tile = (warp & 3) * 32 + lane; // TMEM lane
    const int row = m0 + t * kBM + row_in_tile;     // query row inside the sequence
    const int qpos = row + off;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tSb = tmem + t * 128 + lane_addr;
    const uint32_t tOt = tmem + 256 + t * 128 + lane_addr;
    const float slope = (kExtras && cfg.has_alibi) ? p.alibi_slopes[b * p.heads_q + h] : 0.f;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    const int tq_min = m0 + t * kBM + off, tq_max = tq_min + kBM - 1;
    const int cnt = ghi_t[t] - glo_t[t];

    for (int c = 0; c < cnt && ok; ++c) {
      const int g = glo_t[t] + c;
      const int buf = c & 1;
      const int k0 = g * kHalf;
      bool masked = (k0 + kHalf > si.k_len);
      if (cfg.causal) masked |= (k0 + kHalf - 1 > tq_min);
      if (cfg.wl >= 0) masked |= (k0 < tq_max - cfg.wl);
      if (cfg.wr >= 0) masked |= (k0 + kHalf - 1 > tq_min + cfg.wr);

      ok = wait_bar(&sh->s_full[t][buf], (c >> 1) & 1, sh, 31 + t);
      if (!ok) break;
      tc_fence_after();

      // ---- the 64 scores of this row into registers ---------------------------------------
      uint32_t r[2][32];
      tmem_ld32(tSb + buf * kHalf, r[0]);
      tmem_ld32(tSb + buf * kHalf + 32, r[1]);
      tmem_wait_ld();

      const bool prescaled = kExtras || masked;
      if (prescaled) {
        // score pipeline and mask applied once, in place; values end up in the log2 domain
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(r[cc][i]);
            const int col = k0 + cc * 32 + i;
            if (kExtras) {
              float th;
              v = score_log2(cfg, slope, v, qpos, col, th);
            } else {
              v *= cfg.scale_log2;
            }
            if (masked && !visible(cfg, qpos, col, si.k_len)) v = -INFINITY;
            r[cc][i] = __float_as_uint(v);
          }
        }
      }

      // ---- row maximum: four independent chains ------------------------------------------
      float mx4[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int cc = q4 >> 1, base = (q4 & 1) * 16;
        float a = fmaxf(__uint_as_float(r[cc][base]), __uint_as_float(r[cc][base + 1]));
#pragma unroll
        for (int i = 2; i < 16; i += 2)
          a = fmaxf(a, fmaxf(__uint_as_float(r[cc][base + i]), __uint_as_float(r[cc][base + i + 1])));
        mx4[q4] = a;
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      if (!prescaled) mx *= cfg.scale_log2;  // scale >= 0 on this path

      // ---- lazy rescale ----------------------------------------------------------------
      if (c == 0) {
        m_used = mx;
      } else {
        const bool need = mx > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // PV number c-1.  A parity wait cannot tell "k completions" from "k+2", and only
          // PV c-3 is known to be complete here (QK c-1 was queued behind it), so PVs
          // alternate between two barriers: on barrier (c-1)&1 at most one phase is open.
          ok = wait_bar(&sh->o_ready[t][(c - 1) & 1], ((c - 1) >> 1) & 1, sh, 33 + t);
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
            tmem_ld32(tOt + cc * 32, ro);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
            tmem_st32(tOt + cc * 32, ro);
          }
          tmem_wait_st();
        }
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      const float mul = prescaled ? 1.f : cfg.scale_log2;

      // ---- P = exp2(s - m), row sum (four chains), P -> TMEM in place over S -------------
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(r[cc][i]), mul, -m_safe));
          const float p1 = ex2(fmaf(__uint_as_float(r[cc][i + 1]), mul, -m_safe));
          ps[(i >> 1) & 3] += p0 + p1;
          pk[i >> 1] = Elem<T>::pack(p0, p1);
        }
        tmem_st16(tSb + buf * kHalf + cc * 16, pk);
      }
      l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->p_ready[t][buf]));
    }

    // ---- epilogue: O / l -> global, base-2 LSE ------------------------------------------
    if (ok && cnt > 0) ok = wait_bar(&sh->o_ready[t][(cnt - 1) & 1], ((cnt - 1) >> 1) & 1, sh, 35 + t);
    if (ok) {
      tc_fence_after();
      const bool row_ok = row < si.q_len;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* og = reinterpret_cast<T*>(p.o) + si.q_boff * p.o_stride[0] +
              (si.q_row0 + row) * p.o_stride[1] + (int64_t)h * p.o_stride[2];
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t ro[32];
        if (cnt > 0) {
          tmem_ld32(tOt + cc * 32, ro);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ro[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = Elem<T>::pack(__uint_as_float(ro[i]) * inv, __uint_as_float(ro[i + 1]) * inv);
            v.y = Elem<T>::pack(__uint_as_float(ro[i + 2]) * inv, __uint_as_float(ro[i + 3]) * inv);
            v.z = Elem<T>::pack(__uint_as_float(ro[i + 4]) * inv, __uint_as_float(ro[i + 5]) * inv);
            v.w = Elem<T>::pack(__uint_as_float(ro[i + 6]) * inv, __uint_as_float(ro[i + 7]) * inv);
            *reinterpret_cast<uint4*>(og + cc * 32 + i) = v;
          }
        }
      }
      if (row_ok && p.lse2 != nullptr)
        p.lse2[si.q_boff * p.lse_stride[0] + (si.q_row0 + row) * p.lse_stride[1] +
               (int64_t)h * p.lse_stride[2]] = l > 0.f ? m_used + log2f(l) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
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
  CUtensorMap tq, tk, tv;
  const bool packed = a.cu_seqlens_q != nullptr;
  if (!make_map(&tq, a.q, a.q_stride, q_rows, a.heads_q, a.batch, D, packed) ||
      !make_map(&tk, a.k, a.k_stride, k_rows, a.heads_kv, a.batch, D, packed) ||
      !make_map(&tv, a.v, a.v_stride, k_rows, a.heads_kv, a.batch, D, packed)) {
    set_error("fwd_sm100: cuTensorMapEncodeTiled failed");
    return FA_ERR_LAUNCH;
  }
  const bool extras = cfg.has_alibi || cfg.softcap > 0.f;
  auto kern = extras ? fwd_sm100_kernel<T, D, true> : fwd_sm100_kernel<T, D, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) {
    set_error("fwd_sm100: cudaFuncSetAttribute(%d): %s", C::kSmemBytes, cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  dim3 grid((a.seqlen_q + 2 * kBM - 1) / (2 * kBM), a.heads_q, a.batch);
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, a, cfg);
  return check_launch("fwd_sm100");
}

int fwd_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
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

int fwd_sm100_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_fwd_sm100_status, sizeof(int));
  return v;
}

}  // namespace fa
