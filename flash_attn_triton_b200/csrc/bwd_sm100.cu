// Backward attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), as two
// PERSISTENT kernels with one writer per output element (no atomics, deterministic):
//
//   bwd_dkdv_sm100_kernel  work item = 128 keys of one (batch, kv head); loops over the query
//                          tiles (and the query heads of the GQA group) that can see them.
//                          Works on the TRANSPOSED tiles  S^T = K Q^T,  dP^T = V dO^T  so
//                          that a TMEM lane is a key: P^T and dS^T are written back to TMEM
//                          and feed  dV += P^T dO,  dK += dS^T Q  as the A operand.
//   bwd_dq_sm100_kernel    work item = 128 query rows of one (batch, head); loops over key
//                          tiles: S = Q K^T, dP = dO V^T, dS in place over dP, dQ += dS K.
//
// One CTA per SM takes work items from a queue: a counter in global memory hands out candidates
// in an order in which the CTAs that run together work on the same heads (the tiles they stream
// stay in L2) and in which the heavy items of a causal mask come first.  The producer thread
// draws from the counter, one item ahead, and publishes what it drew to the other roles through
// a small ring in shared memory.  Barriers, tensor memory and tensor maps are set up once per CTA.  Every role runs ahead into the next item on
// its own: the producer fetches the next item's tiles as ring slots free up, the MMA warps issue
// its first products while the element-wise warps still store the previous item's result.  The
// result tiles are staged over the LAST streamed tiles of the item, whose ring slots are released
// by the store instead of by the MMAs that read them: the next item's first tiles are already in
// the other slots by then.
//
// Both kernels are software-pipelined through the ORDER in which the MMA warps feed the (in-
// order) tensor pipe, so that the element-wise warps always work while independent MMAs run:
//
//   dK/dV, per query tile i:   S(i) | dK += dS(i-1)^T Q(i-1) | dV += P(i-1)^T dO(i-1) | dP(i)
//       S(i) and dP(i) take turns in ONE fp32 TMEM region, P and dS (16-bit) share a second one.
//   dQ, per key tile k:        S(k+1) -> other S buffer | dQ += dS(k) K(k) | dP(k+1)
//
// Roles (384 threads):
//   warps 0-3 / 4-7  element-wise groups A / B: columns 0..63 / 64..127 of the 128 x 128
//                    tiles, one TMEM lane (row) per thread
//   warp 8           TMA producer
//   warp 9           MMA issuer (uniform control flow, one elected lane issues)
//   warp 10          dK/dV kernel: loads the per-row statistics (base-2 LSE, delta) of the
//                    streamed query tile and writes them as a 16-column GEMM operand
//   warp 11          dK/dV kernel: second MMA issuer (the accumulating GEMMs)
//
// TMEM, dK/dV kernel: S^T or dP^T (128 columns) | P^T or dS^T (64) | K (64) | dV (128) | dK (128).
// TMEM, dQ kernel:    S[0] | S[1] | dP | dQ    (4 x 128 columns).
// All operand tiles are written by TMA with the 128-byte swizzle; the same tile is read
// K-major (contraction over head_dim) or MN-major (contraction over its rows) through
// different descriptors.  Every mbarrier wait is bounded.
#include <cstddef>
#include <type_traits>

#include <cstdlib>
#include "common.cuh"
#define PROF_TAG bwd
#include "prof.cuh"
#include "sm100.cuh"

namespace fa {

using namespace sm100;

__device__ int g_bwd_sm100_status = 0;

namespace {

constexpr int kT = 128;        // tile edge: rows of Q / keys of K,V per tile
constexpr int kHalfT = 64;     // columns per element-wise group
constexpr int kBwdThreads = 384;
constexpr int kSched = 4;      // depth of the in-CTA ring of work-queue entries
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
  // dK/dV kernel: V resident, ring A of K / Q entries (Q(i) lives from S(i) to dK(i); dK is
  // staged over the last Q), ring B of dO entries (dO(i) lives from dP(i) to dV(i); dV is
  // staged over the last dO).
  static constexpr int kStagesQ = (D == 128) ? 3 : 4;
  static constexpr int kStagesO = (D == 128) ? 2 : 4;
  static constexpr int kSmemTiles = (1 + kStagesQ + kStagesO) * kTileBytes;
  // dK/dV kernel: 128 x 16 operand tiles that carry the row statistics into the GEMMs
  // (two constant ones on the key side, one per ring stage on the query side)
  static constexpr int kAugBytes = kT * 16 * 2;
  static constexpr int kAugTotal = (2 + kStagesQ) * kAugBytes;
  static constexpr int kSmemBytes = kSmemTiles + kAugTotal + 1024 + 4096;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  // dQ kernel: Q and dO resident, ring A of K tiles (dQ is staged over the last one), ring B of V tiles.  The K
  // ring is one stage deeper than the V ring: K(k+1) is needed by S(k+1) at the START of step k
  // while K(k) is still read by dQ(k) at its end.
  static constexpr int kStagesK = (D == 128) ? 3 : 4;
  static constexpr int kStagesV = (D == 128) ? 2 : 4;
  static constexpr int kSmemTilesDq = (2 + kStagesK + kStagesV) * kTileBytes;
  static constexpr int kSmemBytesDq = kSmemTilesDq + 1024 + 1024;
  static_assert(kSmemBytesDq <= 227 * 1024, "shared memory budget (dQ)");
};

struct BShared {
  uint64_t full_a[4];     // ring A entry landed (dK/dV: K, Q + statistics; dQ: K)
  uint64_t full_b[4];     // ring B entry landed (dK/dV: dO; dQ: V)
  uint64_t empty_a[4];    // ring A entry released
  uint64_t empty_b[4];    // ring B entry released
  uint64_t res_full;      // resident tiles of the item landed (dK/dV: V; dQ: Q and dO)
  uint64_t res_free;      // last MMA reading the resident tiles of the item finished
  uint64_t s_full[2];     // S computed ([buffer] in the dQ kernel, [0] in the dK/dV kernel)
  uint64_t dp_full;       // dP computed
  uint64_t p_ready;       // P written back (256 arrivals; dK/dV kernel)
  uint64_t ds_ready;      // dS written back (256 arrivals)
  uint64_t r_free;        // dK/dV kernel: scores, then dP, read out of their shared TMEM region (256 arrivals)
  uint64_t p_free;        // dK/dV kernel: dV MMA that read P finished
  uint64_t ds_free;       // dK/dV kernel: dK MMA that read dS finished
  uint64_t k_copied;      // dK/dV kernel: K of the item copied from its ring slot into TMEM (256 arrivals)
  uint64_t acc_done;      // every accumulation MMA of the item finished
  uint64_t sched_full[kSched];   // work-queue entry published by the producer thread
  uint64_t sched_empty[kSched];  // ... read by every consuming warp
  int4 sched_item[kSched][3];    // the item, decoded once by the producer thread (KItem / QItem)
  uint64_t stg_ready[2];  // [group] result tile of an item staged for the store lane (and its message written)
  uint64_t stg_taken[2];  // [group] the store lane has read the message
  // [group] message to the store lane: shared-memory address of the staged tile (0 = nothing to
  // store, -1 = no more items), tensor-map coordinates head / row / batch, barrier to release
  volatile int stg_msg[2][5];
  uint32_t tmem_base;
  volatile int abort_flag;
  alignas(16) float lse[4][kT];  // [stage][row of the streamed query tile]: MINUS the base-2 LSE (feature variant)
};
static_assert(sizeof(BShared) <= 4096, "BShared must fit its reserve");
static_assert(offsetof(BShared, lse) <= 1024, "the dQ kernel reserves 1024 bytes for the barriers and the work queue");

template <typename T> struct BFmt;
template <> struct BFmt<__half> { static constexpr int code = 0; };
template <> struct BFmt<__nv_bfloat16> { static constexpr int code = 1; };

__device__ __forceinline__ bool bwait(uint64_t* bar, uint32_t parity, BShared* sh, int code) {
  return bounded_wait(bar, parity, &sh->abort_flag, &g_bwd_sm100_status, code);
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

// Work queue.  `counter[0]` hands out candidate indices, `counter[1]` counts the CTAs that have
// finished; the last one to finish puts both back to zero, so a launch always finds them at zero.
// The producer thread draws a candidate, decodes it into an item (12 ints: KItem / QItem) and
// publishes the item to the other roles; entry number i of this CTA travels in ring slot
// i % kSched.  Candidates outside their sequence are skipped; an item with total < 0 ends the queue.
template <typename Item, typename F>
__device__ __forceinline__ Item sched_publish(BShared* sh, unsigned int* counter, int ncand, int& fidx, bool& ok,
                                              F decode) {
  static_assert(sizeof(Item) == 48, "an item travels as three 16-byte words");
  Item w;
  for (;;) {
    const unsigned int u = atomicAdd(&counter[0], 1u);
    if (u >= (unsigned int)ncand) {
      w.total = -1;
      break;
    }
    if (decode((int)u, w)) break;
  }
  const int slot = fidx % kSched;
  if (!bwait_relaxed(&sh->sched_empty[slot], ((fidx / kSched) & 1) ^ 1, sh, 60)) {
    ok = false;
    w.total = -1;
    return w;
  }
  const int4* src = reinterpret_cast<const int4*>(&w);
  sh->sched_item[slot][0] = src[0];
  sh->sched_item[slot][1] = src[1];
  sh->sched_item[slot][2] = src[2];
  mbar_arrive(smem_u32(&sh->sched_full[slot]));
  ++fidx;
  return w;
}
// Entry number idx as seen by a consuming warp (all lanes call this together).  `consume` releases
// the entry; without it the call only looks at an entry that will be consumed later.
template <typename Item>
__device__ __forceinline__ Item sched_get(BShared* sh, int idx, bool consume, bool& ok) {
  Item w;
  const int slot = idx % kSched;
  if (!bwait(&sh->sched_full[slot], (idx / kSched) & 1, sh, 61)) {
    ok = false;
    w.total = -1;
    return w;
  }
  int4* dst = reinterpret_cast<int4*>(&w);
  dst[0] = sh->sched_item[slot][0];
  dst[1] = sh->sched_item[slot][1];
  dst[2] = sh->sched_item[slot][2];
  if (consume) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&sh->sched_empty[slot]));
  }
  return w;
}
// Releases an entry that this warp has already looked at.
__device__ __forceinline__ void sched_release(BShared* sh, int idx) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&sh->sched_empty[idx % kSched]));
}

// Store lane: one thread that writes the result tiles the element-wise warps stage, so that none of
// them has to wait for the TMA unit.  Per item it waits for the tile (and the message that
// describes it), issues the store, waits until the unit has read the tile and releases the ring
// entry the tile was staged over (two stand-in arrivals, or one in the dQ kernel).
template <int D>
__device__ __forceinline__ void store_lane(BShared* sh, int x, const CUtensorMap* tm, uint32_t release_count) {
  for (uint32_t n = 0;; ++n) {
    // an item takes tens of microseconds: sleep between polls instead of spinning next to the
    // producer lane (a spinning lane of the same warp takes its issue slots)
    {
      const uint32_t bar = smem_u32(&sh->stg_ready[x]);
      const long long t0 = clock64();
      bool done = false;
      while (!(done = mbar_try_wait(bar, n & 1))) {
        __nanosleep(400);
        if (sh->abort_flag || *reinterpret_cast<volatile int*>(&g_bwd_sm100_status) != 0) break;
        if (clock64() - t0 > 4 * FA_WAIT_CLOCKS) {   // items differ in length by orders of magnitude
          sh->abort_flag = 62;
          atomicCAS(&g_bwd_sm100_status, 0, 62);
          break;
        }
      }
      if (!done) return;
    }
    const int addr = sh->stg_msg[x][0], head = sh->stg_msg[x][1], row = sh->stg_msg[x][2],
              batch = sh->stg_msg[x][3], rel = sh->stg_msg[x][4];
    mbar_arrive(smem_u32(&sh->stg_taken[x]));
    if (addr == -1) return;
    if (addr > 0) {
#pragma unroll
      for (int bx = 0; bx < D / 64; ++bx) tma_store_4d(tm, (uint32_t)addr + bx * (kT * 128), bx * 64, head, row, batch);
      tma_store_commit();
      tma_store_wait_read();
    }
    mbar_arrive_cnt((uint32_t)rel, release_count);
  }
}
// Element-wise side: thread `poster` of the group writes the message for item number n (after the
// store lane has taken the previous one); every thread of the group then arrives on stg_ready
// once its part of the tile is staged.
__device__ __forceinline__ bool post_store(BShared* sh, int x, int n, int addr, int head, int row, int batch,
                                           uint32_t release_bar) {
  if (n > 0 && !bwait(&sh->stg_taken[x], (n - 1) & 1, sh, 63)) return false;
  sh->stg_msg[x][0] = addr;
  sh->stg_msg[x][1] = head;
  sh->stg_msg[x][2] = row;
  sh->stg_msg[x][3] = batch;
  sh->stg_msg[x][4] = (int)release_bar;
  return true;
}

__device__ __forceinline__ void sched_finish(unsigned int* counter) {
  __threadfence();
  const unsigned int done = atomicAdd(&counter[1], 1u);
  if (done == gridDim.x - 1) {
    counter[0] = 0u;
    counter[1] = 0u;
    __threadfence();
  }
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

// TMEM accumulator (128 lanes x kCols fp32 columns starting at tsrc, this thread's lane) scaled
// by `mul`, converted to T and either staged in the swizzled box layout at `stg` (column
// `col0 + c` of the tile) or, when `direct` is set, stored to the row pointer `grow` (null = skip).
template <typename T, int kCols>
__device__ __forceinline__ void drain_acc(uint32_t tsrc, float mul, bool staged, uint32_t stg, int lrow,
                                          int col0, T* grow) {
#pragma unroll
  for (int cc = 0; cc < kCols / 32; ++cc) {
    uint32_t r[32];
    tmem_ld32(tsrc + cc * 32, r);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 v;
      v.x = Elem<T>::pack(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
      v.y = Elem<T>::pack(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
      v.z = Elem<T>::pack(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
      v.w = Elem<T>::pack(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
      const int col = col0 + cc * 32 + i;
      if (staged) st_shared_v4(sw128_addr(stg + (col / 64) * (kT * 128), lrow, (col % 64) / 8), v);
      else if (grow != nullptr) *reinterpret_cast<uint4*>(grow + cc * 32 + i) = v;
    }
  }
}

// ---------------------------------------------------------------------------------------
// work items
// ---------------------------------------------------------------------------------------
struct Geo {          // one sequence's geometry, as ints (tensor-map coordinates are 32-bit)
  int q_len, k_len, q_row0, k_row0, q_boff, k_boff;
};
__device__ __forceinline__ Geo geo_of(const fa_attn_args& p, int b) {
  const SeqInfo si = seq_info(p, b);
  Geo g;
  g.q_len = si.q_len; g.k_len = si.k_len;
  g.q_row0 = (int)si.q_row0; g.k_row0 = (int)si.k_row0;
  g.q_boff = (int)si.q_boff; g.k_boff = (int)si.k_boff;
  return g;
}

// dK/dV: candidate c = ((b * heads_kv + hk) * key_blocks + key block); key block 0 sees the most
// query tiles under a causal mask.  Returns false when the key block lies outside its sequence.
struct KItem {
  Geo g;
  int n0, hk, b;
  int m_lo, ntiles, total;   // query tiles [m_lo, m_lo + ntiles) per query head; total = ntiles * group
};
__device__ __forceinline__ bool dkdv_item(const fa_attn_args& p, const ScoreCfg& cfg, int cand, int nkb, KItem& w) {
  const int nblk = cand % nkb, rem = cand / nkb;
  w.hk = rem % p.heads_kv;
  w.b = rem / p.heads_kv;
  w.n0 = nblk * kT;
  w.g = geo_of(p, w.b);
  w.m_lo = w.ntiles = w.total = 0;
  if (w.n0 >= w.g.k_len) return false;
  const int off = p.q_pos_offset;
  int qlo, qhi;
  visible_query_range(cfg, w.n0, min(w.n0 + kT, w.g.k_len) - 1, off, w.g.q_len + off, qlo, qhi);
  w.m_lo = max(qlo - off, 0) / kT;
  const int m_hi = (max(qhi - off, 0) + kT - 1) / kT;
  w.ntiles = max(m_hi - w.m_lo, 0);
  w.total = w.ntiles * (p.heads_q / p.heads_kv);
  return true;
}

// dQ: candidate c = ((b * heads_q + h) * query_blocks + i); with a causal mask block i counts
// down from the last (heaviest) query block.  Returns false when the block lies outside its sequence.
struct QItem {
  Geo g;
  int m0, h, b;
  int n_hi, total;           // step j works on key tile n_hi - 1 - j (masked tiles first)
  int pad;
};
__device__ __forceinline__ bool dq_item(const fa_attn_args& p, const ScoreCfg& cfg, int cand, int nmb, QItem& w) {
  const int i = cand % nmb, rem = cand / nmb;
  w.h = rem % p.heads_q;
  w.b = rem / p.heads_q;
  w.m0 = (cfg.causal ? (nmb - 1 - i) : i) * kT;
  w.g = geo_of(p, w.b);
  w.n_hi = w.total = w.pad = 0;
  if (w.m0 >= w.g.q_len) return false;
  const int off = p.q_pos_offset;
  int klo, khi;
  visible_key_range(cfg, w.m0 + off, min(w.m0 + kT, w.g.q_len) - 1 + off, w.g.k_len, klo, khi);
  const int n_lo = klo / kT;
  w.n_hi = (khi + kT - 1) / kT;
  w.total = max(w.n_hi - n_lo, 0);
  return true;
}

}  // namespace

// =======================================================================================
// dK, dV
// =======================================================================================
template <typename T, int D, bool kExtras>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                      const fa_attn_args p, const ScoreCfg cfg, const int nkb, const int ncand,
                      unsigned int* const queue, int* const host_status) {
  using C = BCfg<D>;
  constexpr int SQ = C::kStagesQ, SO = C::kStagesO;
  constexpr int kConsumers = 11;   // warps that read the work queue: 8 element-wise, 2 issuers, statistics
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  BShared* sh = reinterpret_cast<BShared*>(tiles + C::kSmemTiles + C::kAugTotal);
  const uint32_t sV = smem_u32(tiles);
  const uint32_t sRingQ = sV + C::kTileBytes, sRingO = sRingQ + SQ * C::kTileBytes;
  // statistics operands: [0] key side of the score GEMM, [1] key side of the dP GEMM,
  // [2 + stage] query side (written per streamed query tile by the statistics warp)
  unsigned char* aug = tiles + C::kSmemTiles;
  const uint32_t sAug = sV + C::kSmemTiles;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.heads_q / p.heads_kv;
  const int off = p.q_pos_offset;

  auto slotA = [&](int pos) { return sRingQ + (pos % SQ) * C::kTileBytes; };
  auto slotB = [&](int pos) { return sRingO + (pos % SO) * C::kTileBytes; };

  if (tid == 0) {
    mbar_init(smem_u32(&sh->res_full), 1);
    mbar_init(smem_u32(&sh->res_free), 1);
    mbar_init(smem_u32(&sh->s_full[0]), 1);
    mbar_init(smem_u32(&sh->s_full[1]), 1);
    mbar_init(smem_u32(&sh->dp_full), 1);
    mbar_init(smem_u32(&sh->p_ready), 256);
    mbar_init(smem_u32(&sh->ds_ready), 256);
    mbar_init(smem_u32(&sh->r_free), 256);
    mbar_init(smem_u32(&sh->p_free), 1);
    mbar_init(smem_u32(&sh->ds_free), 1);
    mbar_init(smem_u32(&sh->acc_done), 1);
    mbar_init(smem_u32(&sh->k_copied), 256);
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&sh->full_a[i]), 2);   // the TMA load and the statistics warp (or two stand-in arrivals)
      mbar_init(smem_u32(&sh->full_b[i]), 1);
      mbar_init(smem_u32(&sh->empty_a[i]), 2);  // one commit from each of the two issuer warps (or a stand-in)
      mbar_init(smem_u32(&sh->empty_b[i]), 2);
    }
    for (int i = 0; i < kSched; ++i) {
      mbar_init(smem_u32(&sh->sched_full[i]), 1);
      mbar_init(smem_u32(&sh->sched_empty[i]), kConsumers);
    }
    mbar_init(smem_u32(&sh->stg_ready[0]), 128);
    mbar_init(smem_u32(&sh->stg_ready[1]), 128);
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
  // TMEM: R (128 fp32 columns: S^T, then dP^T of a tile) | X (64: P^T, then dS^T) | K (64) | dV | dK
  const uint32_t tR = tmem, tX = tmem + 128, tK = tmem + 192, tdV = tmem + 256, tdK = tmem + 384;

  // Ring bookkeeping shared by every role.  An item with `total` query tiles takes, in order,
  //   ring A:  K | Q(0) ... Q(total-1)        (total + 1 entries)
  //   ring B:  dO(0) ... dO(total-1)          (total entries)
  // and every role advances the same two position counters; entry `pos` lives in slot
  // pos % stages and completes phase (pos / stages) & 1 of that slot's barriers.  The entries of
  // the LAST tile are released by the epilogue (which stages dK and dV over them), the others
  // by the commits of the two issuer warps.

  if (warp == 8) {
    // ------------------------------- TMA producer ---------------------------------------
    reg_dealloc<kRegsService>();
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      prefetch_tmap(&tmdO);
      prefetch_tmap(&tmdK);
      prefetch_tmap(&tmdV);
      int posA = 0, posB = 0, wi = 0, fidx = 0;
      bool ok = true;
      auto acquire_a = [&]() { return bwait_relaxed(&sh->empty_a[posA % SQ], ((posA / SQ) & 1) ^ 1, sh, 41); };
      auto acquire_b = [&]() { return bwait_relaxed(&sh->empty_b[posB % SO], ((posB / SO) & 1) ^ 1, sh, 41); };
      auto decode = [&](int c, KItem& w) { return dkdv_item(p, cfg, c, nkb, w); };
      // An item is drawn from the queue as late as possible -- when the loads of the previous one
      // are all issued, a tile or two before it ends -- so that the CTAs share the work evenly;
      // the other roles look one entry ahead only at the end of an item.
      PROF_VARS(4);
      for (;;) {
        PROF_T0();
        const KItem w = sched_publish<KItem>(sh, queue, ncand, fidx, ok, decode);
        PROF_ADD(0);
        if (!ok || w.total < 0) break;
        if (w.total == 0) continue;
        PROF_T0();
        // K: a ring A entry; the second arrival of its barrier is made here
        if (!(ok = acquire_a())) break;
        {
          const uint32_t bar = smem_u32(&sh->full_a[posA % SQ]);
          mbar_expect_tx(bar, C::kTileBytes);
          load_tile<D>(slotA(posA), &tmK, bar, w.g.k_row0 + w.n0, w.hk, w.g.k_boff);
          mbar_arrive(bar);
          ++posA;
        }
        for (int it = 0; it < w.total; ++it) {
          const int hq = w.hk * G + it / w.ntiles, m = w.m_lo + it % w.ntiles;
          if (!(ok = acquire_a())) break;
          {
            const uint32_t bar = smem_u32(&sh->full_a[posA % SQ]);
            mbar_expect_tx(bar, C::kTileBytes);
            load_tile<D>(slotA(posA), &tmQ, bar, w.g.q_row0 + m * kT, hq, w.g.q_boff);
            ++posA;
          }
          if (!(ok = acquire_b())) break;
          {
            const uint32_t bar = smem_u32(&sh->full_b[posB % SO]);
            mbar_expect_tx(bar, C::kTileBytes);
            load_tile<D>(slotB(posB), &tmdO, bar, w.g.q_row0 + m * kT, hq, w.g.q_boff);
            ++posB;
          }
          if (it == 0) {
            // V (first needed by dP(0), after the first score tile): its slot is free once the last
            // dP GEMM of the previous item has read it.  Requested after the first Q and dO tiles so
            // that those never queue behind this wait.
            if (wi > 0 && !(ok = bwait_relaxed(&sh->res_free, (wi - 1) & 1, sh, 41))) break;
            const uint32_t bar = smem_u32(&sh->res_full);
            mbar_expect_tx(bar, C::kTileBytes);
            load_tile<D>(sV, &tmV, bar, w.g.k_row0 + w.n0, w.hk, w.g.k_boff);
          }
        }
        if (!ok) break;
        ++wi;
        PROF_ADD(1);
      }
      PROF_FLUSH(true, 28, 4);
    }
  } else if (warp == 10) {
    // ------------------------------- statistics loader ----------------------------------
    // The loads of the next tile are ISSUED right after the current one has been written and only
    // consumed after the wait for the next slot, so their latency hides behind that wait.
    reg_dealloc<kRegsService>();
    float rl[kT / 32], rd[kT / 32];                  // statistics of rows lane, lane + 32, ... as loaded
    auto fetch = [&](const KItem& w, int it) {
      const int hq = w.hk * G + it / w.ntiles, m = w.m_lo + it % w.ntiles;
#pragma unroll
      for (int k = 0; k < kT / 32; ++k) {
        const int row = m * kT + lane + 32 * k;
        rl[k] = INFINITY;
        rd[k] = 0.f;
        if (row < w.g.q_len) {
          const int64_t idx = (int64_t)w.g.q_boff * p.lse_stride[0] + (int64_t)(w.g.q_row0 + row) * p.lse_stride[1] +
                              (int64_t)hq * p.lse_stride[2];
          rl[k] = p.lse2[idx];
          rd[k] = p.delta[idx];
        }
      }
    };
    int posA = 0, sidx = 0;
    bool ok = true, fetched = false;                 // fetched: tile 0 of the item about to run is in rl/rd
    KItem w = sched_get<KItem>(sh, sidx++, true, ok);
    while (ok && w.total >= 0) {
      if (w.total == 0) {
        w = sched_get<KItem>(sh, sidx++, true, ok);
        continue;
      }
      bool haven = false;
      if (!fetched) fetch(w, 0);
      ++posA;                                        // the K entry
      for (int it = 0; it < w.total; ++it, ++posA) {
        const int stage = posA % SQ;
        bool wt = true;
        if (lane == 0) wt = bwait_relaxed(&sh->empty_a[stage], ((posA / SQ) & 1) ^ 1, sh, 42);
        if (!__all_sync(0xffffffffu, wt)) { ok = false; break; }
        uint4* q4 = reinterpret_cast<uint4*>(aug + (2 + stage) * C::kAugBytes);
#pragma unroll
        for (int k = 0; k < kT / 32; ++k) {
          const int i = lane + 32 * k;
          // NEGATED; rows that do not exist or see no key get a large finite value instead of
          // infinity (an infinity would meet the zeros of the other GEMM's key-side operand): P = 0.
          // delta is clamped into the 16-bit range for the same reason.
          float nl2 = -rl[k];
          float ndl = fminf(fmaxf(-rd[k], -60000.f), 60000.f);
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
        if (it + 1 < w.total) {
          fetch(w, it + 1);
        } else {
          // the entry after this one (published once the loads of this item are issued), if it
          // has work, gets its first tile fetched ahead
          const KItem wn = sched_get<KItem>(sh, sidx, false, ok);
          if (!ok) break;
          haven = wn.total > 0;
          if (haven) fetch(wn, 0);
        }
      }
      if (!ok) break;
      fetched = haven;
      w = sched_get<KItem>(sh, sidx++, true, ok);
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer, GEMMs into the fp32 region -------------
    // This warp issues dP(i), then S(i+1) -- each once the element-wise warps have read its
    // predecessor out of R (r_free).  Warp 11 issues the accumulating GEMMs dV(i), dK(i) that
    // read P, dS from region X.
    reg_dealloc<kRegsService>();
    constexpr uint32_t idesc_s = make_idesc(1, BFmt<T>::code, 0, 0, kT, kT);
    const uint32_t leader = elect_one() ? 1u : 0u;
    bool ok = true;
    // every lane polls (uniform control flow, no vote needed: a completed phase is seen by all)
    auto wq = [&](uint64_t* bar, uint32_t parity, int code) {
      if (ok) ok = bwait(bar, parity, sh, code);
      tc_fence_after();
    };
    const uint64_t dstat_s = make_smem_desc_noswizzle(sAug, 2048, 128);
    const uint64_t dstat_dp = make_smem_desc_noswizzle(sAug + C::kAugBytes, 2048, 128);
    auto stat_desc = [&](int pos) {
      return make_smem_desc_noswizzle(sAug + (2 + pos % SQ) * C::kAugBytes, 2048, 128);
    };
    PROF_VARS(8);
    int posA = 0, posB = 0, wi = 0, tg = 0;          // tg: tiles issued so far by this CTA
    // The last query tile of a packed sequence also stages rows of the NEXT sequence.  Their P is
    // 0 (the statistics say so), but 0 * inf is NaN and dS^T Q, P^T dO contract over those rows:
    // this warp, the first reader of every staged Q and dO tile, zeroes them once the tile has
    // landed (scores and dP of those rows then are 0 too).
    // S^T = K Q^T (K from TMEM) - lse2 / scale_log2 for the tile at ring position qpos
    auto issue_s = [&](int qpos, int tile_no, int tail) {
      PROF_T0();
      wq(&sh->full_a[qpos % SQ], (qpos / SQ) & 1, 44);
      PROF_ADD(1);
      if (ok && tail < kT) zero_tile_tail<C::kBoxes, kT>(slotA(qpos), tail, lane);
      PROF_T0();
      if (tile_no > 0) wq(&sh->r_free, 1, 49);                                  // the previous dP read out
      PROF_ADD(2);
      if (!ok) return;
      mma_kmajor_ts<D>(tR, tK, slotA(qpos), idesc_s, leader);
      if (!kExtras) mma_f16_ss_lp(tR, dstat_s, stat_desc(qpos), idesc_s, 1u, leader);
      mma_commit_lp(smem_u32(&sh->s_full[0]), leader);
    };
    int sidx = 0;
    for (;;) {
      PROF_T0();
      const KItem w = sched_get<KItem>(sh, sidx++, true, ok);
      if (!ok || w.total < 0) break;
      PROF_ADD(6);
      if (w.total == 0) continue;
      // K is in TMEM: its ring slot may be refilled (stand-in for the two MMA commits of a Q entry)
      PROF_T0();
      wq(&sh->k_copied, wi & 1, 43);
      PROF_ADD(0);
      if (!ok) break;
      if (leader) mbar_arrive_cnt(smem_u32(&sh->empty_a[posA % SQ]), 2);
      __syncwarp();
      const int q0pos = posA + 1;
      // the query tile that crosses the end of its sequence (-1: none) and its first row to zero;
      // m_cur / m_nxt: query tile of stream position i / i + 1 (the tiles repeat per query head)
      const int tail_m = (p.cu_seqlens_q != nullptr && (w.g.q_len % kT) != 0) ? w.g.q_len / kT : -1;
      const int tail_first = w.g.q_len % kT, m_end = w.m_lo + w.ntiles;
      int m_cur = w.m_lo, m_nxt = (w.m_lo + 1 == m_end) ? w.m_lo : w.m_lo + 1;
      issue_s(q0pos, tg, m_cur == tail_m ? tail_first : kT);
      for (int i = 0; i < w.total && ok; ++i, ++tg, m_cur = m_nxt, m_nxt = (m_nxt + 1 == m_end) ? w.m_lo : m_nxt + 1) {
        const int qpos = q0pos + i, opos = posB + i;
        PROF_T0();
        wq(&sh->full_b[opos % SO], (opos / SO) & 1, 44);
        PROF_ADD(3);
        if (ok && m_cur == tail_m) zero_tile_tail<C::kBoxes, kT>(slotB(opos), tail_first, lane);
        PROF_T0();
        if (i == 0) wq(&sh->res_full, wi & 1, 43);                              // V of this item
        PROF_ADD(4);
        PROF_T0();
        wq(&sh->r_free, 0, 49);                                                 // S(i) read out
        PROF_ADD(5);
        if (!ok) break;
        mma_kmajor<D>(tR, sV, slotB(opos), idesc_s, leader);                    // dP^T(i) = V dO(i)^T
        mma_f16_ss_lp(tR, dstat_dp, stat_desc(qpos), idesc_s, 1u, leader);      //           - delta
        mma_commit_lp(smem_u32(&sh->dp_full), leader);
        if (i + 1 < w.total) {
          mma_commit_lp(smem_u32(&sh->empty_b[opos % SO]), leader);   // this warp's last reads of dO(i) and of
          mma_commit_lp(smem_u32(&sh->empty_a[qpos % SQ]), leader);   // Q(i) and its statistics
          issue_s(qpos + 1, tg + 1, m_nxt == tail_m ? tail_first : kT);
        } else {
          mma_commit_lp(smem_u32(&sh->res_free), leader);             // ... and of V (the epilogue releases
        }                                                             // the last tile's ring entries)
      }
      posA += w.total + 1;
      posB += w.total;
      ++wi;
    }
    PROF_FLUSH(lane == 0, 16, 8);
    __syncwarp();
  } else if (warp == 11) {
    // ------------------------------- MMA issuer, accumulations --------------------------
    reg_dealloc<kRegsService>();
    constexpr uint32_t idesc_acc = make_idesc(1, BFmt<T>::code, 0, 1, kT, D);
    const uint32_t leader = elect_one() ? 1u : 0u;
    bool ok = true;
    auto wq = [&](uint64_t* bar, uint32_t parity, int code) {
      if (ok) ok = bwait(bar, parity, sh, code);
      tc_fence_after();
    };
    int posA = 0, posB = 0, tg = 0, sidx = 0, wi = 0;
    PROF_VARS(4);
    for (;;) {
      PROF_T0();
      const KItem w = sched_get<KItem>(sh, sidx++, true, ok);
      if (!ok || w.total < 0) break;
      PROF_ADD(3);
      if (w.total == 0) continue;
      for (int i = 0; i < w.total && ok; ++i, ++tg) {
        const int qpos = posA + 1 + i, opos = posB + i;
        // dO(i) may land after P(i) is ready; Q(i) has been read by S(i) long before dS(i) exists
        PROF_T0();
        wq(&sh->full_b[opos % SO], (opos / SO) & 1, 44);
        PROF_ADD(0);
        PROF_T0();
        wq(&sh->p_ready, tg & 1, 45);
        PROF_ADD(1);
        if (!ok) break;
        const bool last = i + 1 == w.total;          // its ring entries are released by the epilogue
        mma_from_tmem<D, 32>(tdV, tX, slotB(opos), idesc_acc, i > 0, leader);   // dV += P(i)^T dO(i)
        if (!last) mma_commit_lp(smem_u32(&sh->empty_b[opos % SO]), leader);
        mma_commit_lp(smem_u32(&sh->p_free), leader);
        PROF_T0();
        wq(&sh->ds_ready, tg & 1, 46);
        PROF_ADD(2);
        if (!ok) break;
        mma_from_tmem<D, 32>(tdK, tX, slotA(qpos), idesc_acc, i > 0, leader);   // dK += dS(i)^T Q(i)
        if (!last) mma_commit_lp(smem_u32(&sh->empty_a[qpos % SQ]), leader);
        mma_commit_lp(smem_u32(&sh->ds_free), leader);
      }
      if (ok) mma_commit_lp(smem_u32(&sh->acc_done), leader);
      // The element-wise warps now stage dV and dK over the item's last dO and Q tiles.  This warp
      // has nothing to issue until the first P of the next item exists, so it hands the staged
      // tiles to the TMA unit and releases the two ring entries once the unit has read them.
      {
        const int stgA = posA + w.total, stgB = posB + w.total - 1;
        const bool via_tma = (p.cu_seqlens_k == nullptr) || (w.n0 + kT <= w.g.k_len);
        wq(&sh->stg_ready[0], wi & 1, 62);
        if (ok && via_tma && leader) {
#pragma unroll
          for (int bx = 0; bx < D / 64; ++bx)
            tma_store_4d(&tmdV, slotB(stgB) + bx * (kT * 128), bx * 64, w.hk, w.g.k_row0 + w.n0, w.g.k_boff);
        }
        wq(&sh->stg_ready[1], wi & 1, 62);
        if (ok && leader) {
          if (via_tma) {
#pragma unroll
            for (int bx = 0; bx < D / 64; ++bx)
              tma_store_4d(&tmdK, slotA(stgA) + bx * (kT * 128), bx * 64, w.hk, w.g.k_row0 + w.n0, w.g.k_boff);
            tma_store_commit();
            tma_store_wait_read();
          }
          // released like tiles whose two readers have finished
          mbar_arrive_cnt(smem_u32(&sh->empty_b[stgB % SO]), 2);
          mbar_arrive_cnt(smem_u32(&sh->empty_a[stgA % SQ]), 2);
        }
        __syncwarp();
      }
      posA += w.total + 1;
      posB += w.total;
      ++wi;
    }
    PROF_FLUSH(lane == 0, 24, 4);
    __syncwarp();
  } else {
    // ------------------------------- element-wise groups --------------------------------
    reg_alloc<kRegsEw>();
    const int x = warp >> 2;                         // column half
    const int lrow = (warp & 3) * 32 + lane;         // TMEM lane = key inside the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tRx = tR + lane_addr + x * kHalfT;            // fp32 scores / dP: this group's 64 columns
    const uint32_t tXx = tX + lane_addr + x * (kHalfT / 2);      // P^T, then dS^T, as 16-bit pairs: 32 columns
    bool ok = true;
    int posA = 0, posB = 0, wi = 0, tg = 0, sidx = 0;
    bool k_in_tmem = false;                          // K of the item about to run is already in TMEM
    PROF_VARS(16);
#ifdef FA_PROF
    const long long prof_start = clock64();
    long long prof_t1 = 0;
#endif

    // K of an item: from its ring slot into TMEM, where the score GEMM reads it as the A operand.
    // This thread copies its key row, group x the x-th half of it.
    auto copy_k = [&](int kpos) {
      ok = bwait(&sh->full_a[kpos % SQ], (kpos / SQ) & 1, sh, 43);
      if (!ok) return;
      constexpr int kChunks = D / 16;                // 16-byte chunks per group
      const uint32_t src = slotA(kpos);
      uint32_t kr[kChunks / 4][16];
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        const int g = x * kChunks + c;
        const uint4 v = ld_shared_v4(sw128_addr(src + (g / 8) * (kT * 128), lrow, g % 8));
        kr[c / 4][(c % 4) * 4] = v.x; kr[c / 4][(c % 4) * 4 + 1] = v.y;
        kr[c / 4][(c % 4) * 4 + 2] = v.z; kr[c / 4][(c % 4) * 4 + 3] = v.w;
      }
#pragma unroll
      for (int c = 0; c < kChunks / 4; ++c) tmem_st16(tK + lane_addr + x * (D / 4) + c * 16, kr[c]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(smem_u32(&sh->k_copied));
    };

    KItem w, wn;                                     // wn: the entry after the current one, once looked at
    bool peeked = false;
    for (;;) {
      PROF_T0();
      if (peeked) {
        sched_release(sh, sidx++);
        w = wn;
      } else {
        w = sched_get<KItem>(sh, sidx++, true, ok);
      }
      if (!ok || w.total < 0) break;
      peeked = false;
      PROF_ADD(7);
      const int key = w.n0 + lrow;
      // group A stores dV, group B stores dK * softmax_scale
      T* grow = nullptr;
      if (key < w.g.k_len)
        grow = (x == 0) ? reinterpret_cast<T*>(p.dv) + (int64_t)w.g.k_boff * p.dv_stride[0] +
                              (int64_t)(w.g.k_row0 + key) * p.dv_stride[1] + (int64_t)w.hk * p.dv_stride[2]
                        : reinterpret_cast<T*>(p.dk) + (int64_t)w.g.k_boff * p.dk_stride[0] +
                              (int64_t)(w.g.k_row0 + key) * p.dk_stride[1] + (int64_t)w.hk * p.dk_stride[2];
      if (w.total == 0) {
        // no query can see these keys: their gradients are zero
        if (grow != nullptr) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(grow)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      int vq_lo, vq_hi;                              // query positions that see this thread's key
      visible_q_interval(cfg, key, vq_lo, vq_hi);
      PROF_T0();
      if (!k_in_tmem) copy_k(posA);
      PROF_ADD(4);
      if (!ok) break;
      const int q0pos = posA + 1;
      PROF_COUNT(9, w.total);
      PROF_COUNT(10, 1);

      for (int it = 0; it < w.total && ok; ++it, ++tg) {
        const int stage = (q0pos + it) % SQ;
        const int hq = w.hk * G + it / w.ntiles, m = w.m_lo + it % w.ntiles;
        const int q0 = m * kT + x * kHalfT;            // first query row of this thread's columns
        const float slope = (kExtras && cfg.has_alibi) ? p.alibi_slopes[w.b * p.heads_q + hq] : 0.f;
        bool masked = false;
        if (cfg.causal) masked |= (w.n0 + kT - 1 > q0 + off);
        if (cfg.wl >= 0) masked |= (w.n0 < q0 + kHalfT - 1 + off - cfg.wl);
        if (cfg.wr >= 0) masked |= (w.n0 + kT - 1 > q0 + off + cfg.wr);

        // Only the feature path still needs the LSE per column (it is added after the soft cap);
        // it is fetched into registers BEFORE the wait for the scores: shared-memory loads issued
        // while the tensor pipe streams its operands take hundreds of cycles, and here that
        // latency hides behind the wait.  Otherwise the GEMMs deliver S - lse and dP - delta.
        float st[kHalfT];                              // -lse, later the soft cap's tanh factor
        if (kExtras) {
          ok = bwait(&sh->full_a[stage], ((q0pos + it) / SQ) & 1, sh, 47);
          if (!ok) break;
          const float4* L4 = reinterpret_cast<const float4*>(&sh->lse[stage][x * kHalfT]);
#pragma unroll
          for (int i4 = 0; i4 < kHalfT / 4; ++i4) {
            const float4 l4 = L4[i4];
            st[i4 * 4] = l4.x; st[i4 * 4 + 1] = l4.y; st[i4 * 4 + 2] = l4.z; st[i4 * 4 + 3] = l4.w;
          }
        }
        PROF_T0();
        ok = bwait(&sh->s_full[0], tg & 1, sh, 46);
#ifdef FA_PROF
        if (it == 0) PROF_ADD(11); else PROF_ADD(0);
        prof_t1 = clock64();
#endif
        if (!ok) break;
        tc_fence_after();

        // ---- exp phase: P = exp2(score - lse), written back as T pairs ---------------------
        uint32_t r0[32], r1[32];
        tmem_ld32(tRx, r0);
        tmem_ld32(tRx + 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh->r_free));            // the scores are in registers: dP may take the region
        float pf[kHalfT];                              // P in fp32, kept for the dS phase
        const float dist0 = (float)(q0 + off - key);   // query position - key position of column 0
        // columns (query rows) of this tile that see this thread's key
        const ColMask cm = make_col_mask(vq_lo - (q0 + off), vq_hi - (q0 + off));
        // One body, compiled per (masked tile, soft cap): no branch inside the unrolled loops.
        uint32_t pkx[kExtras ? 32 : 1];                // feature variant: P as T pairs, packed inside the loop
        auto exp_body = [&](auto mask_tag, auto cap_tag, auto abs_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
          constexpr bool kCap = decltype(cap_tag)::value;
          constexpr bool kAbs = decltype(abs_tag)::value;
          if constexpr (kExtras) {
            // Packed pairs throughout (the loop body is what the instruction cache has to hold:
            // as 64 scalar chains this variant stalled more on instruction fetch than on anything
            // else).  The distance of a pair's columns advances by (2, 2); under the causal mask
            // every visible element has distance >= 0 and |.| is not needed.
            const float ka = kCap ? -(slope * cfg.inv_softcap) : -(slope * FA_LOG2E);
            const float kb = kCap ? cfg.scale * cfg.inv_softcap : cfg.scale_log2;
            const float cl = cfg.softcap * FA_LOG2E;
            const float2 ka2 = make_float2(ka, ka), kb2 = make_float2(kb, kb), cl2 = make_float2(cl, cl);
            const float2 one2 = make_float2(1.f, 1.f), none2 = make_float2(-1.f, -1.f), two2 = make_float2(2.f, 2.f);
            float2 d2 = make_float2(dist0, dist0 + 1.f);
#pragma unroll
            for (int i = 0; i < kHalfT; i += 2) {
              const uint32_t* rr = i < 32 ? r0 : r1;
              const float2 sv2 = make_float2(__uint_as_float(rr[i & 31]), __uint_as_float(rr[(i & 31) + 1]));
              const float2 da = kAbs ? make_float2(fabsf(d2.x), fabsf(d2.y)) : d2;
              const float2 st2 = make_float2(st[i], st[i + 1]);
              float2 pe;
              if (kCap) {
                const float2 y2 = f2fma(ka2, da, f2mul(sv2, kb2));
                const float2 th2 = make_float2(tanh_approx(y2.x), tanh_approx(y2.y));
                const float2 a2 = f2fma(th2, cl2, st2);
                pe = make_float2(ex2(a2.x), ex2(a2.y));
                if (kMask) {
                  pe.x = col_visible(cm, i) ? pe.x : 0.f;
                  pe.y = col_visible(cm, i + 1) ? pe.y : 0.f;
                }
                pkx[i >> 1] = Elem<T>::pack(pe.x, pe.y);
                // the tanh factor of the soft cap goes into the copy kept for dS
                pe = f2mul(pe, f2fma(f2mul(th2, th2), none2, one2));
              } else {
                const float2 a2 = f2fma(ka2, da, f2fma(sv2, kb2, st2));
                pe = make_float2(ex2(a2.x), ex2(a2.y));
                if (kMask) {
                  pe.x = col_visible(cm, i) ? pe.x : 0.f;
                  pe.y = col_visible(cm, i + 1) ? pe.y : 0.f;
                }
                pkx[i >> 1] = Elem<T>::pack(pe.x, pe.y);
              }
              pf[i] = pe.x;
              pf[i + 1] = pe.y;
              d2 = f2add(d2, two2);
            }
          } else {
            const float2 c2 = make_float2(cfg.scale_log2, cfg.scale_log2);
#pragma unroll
            for (int i = 0; i < kHalfT; i += 2) {
              const uint32_t* rr = i < 32 ? r0 : r1;
              const float2 a = f2mul(make_float2(__uint_as_float(rr[i & 31]), __uint_as_float(rr[(i & 31) + 1])), c2);
              float2 pe = ex2_pair<kPolyEvery>(a, i >> 1);
              if (kMask) {
                pe.x = col_visible(cm, i) ? pe.x : 0.f;
                pe.y = col_visible(cm, i + 1) ? pe.y : 0.f;
              }
              pf[i] = pe.x;
              pf[i + 1] = pe.y;
            }
          }
        };
        const bool cap = kExtras && cfg.softcap > 0.f;
        // |distance| only where a visible element can lie on the other side of the diagonal
        const bool need_abs = kExtras && !cfg.causal;
        auto run_exp = [&](auto mask_tag) {
          if (cap) {
            if (need_abs) exp_body(mask_tag, std::true_type{}, std::true_type{});
            else exp_body(mask_tag, std::true_type{}, std::false_type{});
          } else {
            if (need_abs) exp_body(mask_tag, std::false_type{}, std::true_type{});
            else exp_body(mask_tag, std::false_type{}, std::false_type{});
          }
        };
        if (masked) run_exp(std::true_type{});
        else run_exp(std::false_type{});
#ifdef FA_PROF
        prof_acc[masked ? 13 : 12] += (unsigned int)(clock64() - prof_t1);
        if (masked) prof_acc[14] += 1;
#endif
        // X holds dS of the previous tile until its dK MMA has finished (ds_free)
        if (tg > 0) {
          PROF_T0();
          ok = bwait(&sh->ds_free, (tg - 1) & 1, sh, 50);
          PROF_ADD(1);
          if (!ok) break;
          tc_fence_after();
        }
        if constexpr (kExtras) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = pkx[c * 16 + i];
            tmem_st16(tXx + c * 16, pk);
          }
        } else {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = Elem<T>::pack(pf[c * 32 + 2 * i], pf[c * 32 + 2 * i + 1]);
            tmem_st16(tXx + c * 16, pk);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh->p_ready));

        // ---- dS phase: dS = P (dP - delta) -------------------------------------------------
        PROF_T0();
        ok = bwait(&sh->dp_full, tg & 1, sh, 48);
        PROF_ADD(2);
#ifdef FA_PROF
        prof_t1 = clock64();
#endif
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
#ifdef FA_PROF
        prof_acc[15] += (unsigned int)(clock64() - prof_t1);
#endif
        // X holds P of this tile until its dV MMA has finished (p_free)
        PROF_T0();
        ok = bwait(&sh->p_free, tg & 1, sh, 51);
        PROF_ADD(3);
        if (!ok) break;
        tc_fence_after();
        tmem_st16(tXx, pk0);
        tmem_st16(tXx + 16, pk1);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh->ds_ready));
      }
      if (!ok) break;

      // ---- end of the item ------------------------------------------------------------------
      // K of the next item goes into TMEM first (every score GEMM of this item has finished, and
      // the last dK GEMM still runs), so that the issuer can start on it during the epilogue.
      const int stgA = posA + w.total, stgB = posB + w.total - 1;   // the last Q and dO tiles of the item
      {
        PROF_T0();
        wn = sched_get<KItem>(sh, sidx, false, ok);
        if (!ok) break;
        peeked = true;
        k_in_tmem = wn.total > 0;
        PROF_ADD(7);
        PROF_T0();
        if (k_in_tmem) copy_k(stgA + 1);
        PROF_ADD(4);
        if (!ok) break;
      }
      // Epilogue: each group stages its tile over the item's last dO / Q tile (every MMA is done;
      // swizzled box layout) and hands it to the second issuer warp, which lets the TMA unit write
      // full rows; a packed tile that reaches past the end of its sequence is stored row by row instead.
      PROF_T0();
      ok = bwait(&sh->acc_done, wi & 1, sh, 49);
      PROF_ADD(5);
      if (!ok) break;
      tc_fence_after();
      PROF_T0();
      const uint32_t stg = (x == 0) ? slotB(stgB) : slotA(stgA);
      const bool via_tma = (p.cu_seqlens_k == nullptr) || (w.n0 + kT <= w.g.k_len);
      drain_acc<T, D>((x == 0 ? tdV : tdK) + lane_addr, (x == 0) ? 1.f : cfg.scale, via_tma, stg, lrow, 0, grow);
      tc_fence_before();
      if (via_tma) fence_proxy_async();
      mbar_arrive(smem_u32(&sh->stg_ready[x]));
      PROF_ADD(6);
      posA += w.total + 1;
      posB += w.total;
      ++wi;
    }
#ifdef FA_PROF
    prof_acc[8] = (unsigned int)(clock64() - prof_start);
#endif
    PROF_FLUSH(tid == 0, 0, 12);
#ifdef FA_PROF
    if (tid == 0) for (int pi = 11; pi < 16; ++pi) atomicAdd(&PROF_ARRAY[32 + pi], (unsigned long long)prof_acc[pi]);
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
  if (tid == 0) {
    if (sh->abort_flag == 0) sched_finish(queue);
    report_abort(sh->abort_flag, host_status);
  }
}

// =======================================================================================
// dQ
// =======================================================================================
template <typename T, int D, bool kExtras>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmdQ, const fa_attn_args p, const ScoreCfg cfg,
                    const int nmb, const int ncand, unsigned int* const queue,
                    int* const host_status) {
  using C = BCfg<D>;
  constexpr int SK = C::kStagesK, SV = C::kStagesV;
  constexpr int kConsumers = 9;    // warps that read the work queue: 8 element-wise and the issuer
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  BShared* sh = reinterpret_cast<BShared*>(tiles + C::kSmemTilesDq);
  const uint32_t sQ = smem_u32(tiles), sdO = sQ + C::kTileBytes;
  const uint32_t sRingK = sdO + C::kTileBytes, sRingV = sRingK + SK * C::kTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int off = p.q_pos_offset;

  auto slotK = [&](int pos) { return sRingK + (pos % SK) * C::kTileBytes; };
  auto slotV = [&](int pos) { return sRingV + (pos % SV) * C::kTileBytes; };

  if (tid == 0) {
    mbar_init(smem_u32(&sh->res_full), 1);
    mbar_init(smem_u32(&sh->res_free), 2);    // the last S GEMM and the last dP GEMM of the item
    mbar_init(smem_u32(&sh->s_full[0]), 1);
    mbar_init(smem_u32(&sh->s_full[1]), 1);
    mbar_init(smem_u32(&sh->dp_full), 1);
    mbar_init(smem_u32(&sh->ds_ready), 256);
    mbar_init(smem_u32(&sh->acc_done), 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&sh->full_a[i]), 1);
      mbar_init(smem_u32(&sh->full_b[i]), 1);
      mbar_init(smem_u32(&sh->empty_a[i]), 1);
      mbar_init(smem_u32(&sh->empty_b[i]), 1);
    }
    for (int i = 0; i < kSched; ++i) {
      mbar_init(smem_u32(&sh->sched_full[i]), 1);
      mbar_init(smem_u32(&sh->sched_empty[i]), kConsumers);
    }
    mbar_init(smem_u32(&sh->stg_ready[0]), 256);
    mbar_init(smem_u32(&sh->stg_taken[0]), 1);
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
  const uint32_t tS = tmem /* + buffer * 128 */, tdP = tmem + 256, tdQ = tmem + 384;

  // Ring bookkeeping: an item with `total` key tiles takes ring A entries K(0) ... K(total-1) and
  // ring B entries V(0) ... V(total-1); the last K entry is released by the epilogue, which
  // stages dQ over it.

  if (warp >= 10) {
    reg_dealloc<kRegsService>();
    if (warp == 10 && lane == 0) {
      prefetch_tmap(&tmdQ);
      store_lane<D>(sh, 0, &tmdQ, 1);                 // the store lane of dQ
    }
  } else if (warp == 8) {
    // ------------------------------- TMA producer ---------------------------------------
    reg_dealloc<kRegsService>();
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      prefetch_tmap(&tmdO);
      int posA = 0, posB = 0, wi = 0, fidx = 0;
      bool ok = true;
      auto decode = [&](int c, QItem& w) { return dq_item(p, cfg, c, nmb, w); };
      // an item is drawn from the queue only when the loads of the previous one are all issued
      for (;;) {
        const QItem w = sched_publish<QItem>(sh, queue, ncand, fidx, ok, decode);
        if (!ok || w.total < 0) break;
        if (w.total == 0) continue;
        const int hk = w.h / (p.heads_q / p.heads_kv);
        // Q and dO: their slots are free once the last S and dP GEMMs of the previous item are done
        if (wi > 0 && !(ok = bwait_relaxed(&sh->res_free, (wi - 1) & 1, sh, 51))) break;
        {
          const uint32_t bar = smem_u32(&sh->res_full);
          mbar_expect_tx(bar, 2 * C::kTileBytes);
          load_tile<D>(sQ, &tmQ, bar, w.g.q_row0 + w.m0, w.h, w.g.q_boff);
          load_tile<D>(sdO, &tmdO, bar, w.g.q_row0 + w.m0, w.h, w.g.q_boff);
        }
        // K runs one tile ahead of V: K(j+1) is requested before V(j)
        auto load_k = [&](int j) {
          const int pos = posA + j;
          if (!bwait_relaxed(&sh->empty_a[pos % SK], ((pos / SK) & 1) ^ 1, sh, 51)) return false;
          const uint32_t bar = smem_u32(&sh->full_a[pos % SK]);
          mbar_expect_tx(bar, C::kTileBytes);
          load_tile<D>(slotK(pos), &tmK, bar, w.g.k_row0 + (w.n_hi - 1 - j) * kT, hk, w.g.k_boff);
          return true;
        };
        auto load_v = [&](int j) {
          const int pos = posB + j;
          if (!bwait_relaxed(&sh->empty_b[pos % SV], ((pos / SV) & 1) ^ 1, sh, 51)) return false;
          const uint32_t bar = smem_u32(&sh->full_b[pos % SV]);
          mbar_expect_tx(bar, C::kTileBytes);
          load_tile<D>(slotV(pos), &tmV, bar, w.g.k_row0 + (w.n_hi - 1 - j) * kT, hk, w.g.k_boff);
          return true;
        };
        ok = load_k(0);
        for (int j = 0; j < w.total && ok; ++j) {
          if (j + 1 < w.total) ok = load_k(j + 1);
          if (ok) ok = load_v(j);
        }
        if (!ok) break;
        posA += w.total;
        posB += w.total;
        ++wi;
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -----------------------------------------
    reg_dealloc<kRegsService>();
    constexpr uint32_t idesc_s = make_idesc(1, BFmt<T>::code, 0, 0, kT, kT);
    constexpr uint32_t idesc_acc = make_idesc(1, BFmt<T>::code, 0, 1, kT, D);
    const uint32_t leader = elect_one() ? 1u : 0u;
    bool ok = true;
    auto wq = [&](uint64_t* bar, uint32_t parity, int code) {
      if (ok) ok = bwait(bar, parity, sh, code);
      tc_fence_after();
    };
    int posA = 0, posB = 0, wi = 0, tg = 0, sidx = 0; // tg: key tiles issued so far by this CTA
    for (;;) {
      const QItem w = sched_get<QItem>(sh, sidx++, true, ok);
      if (!ok || w.total < 0) break;
      if (w.total == 0) continue;
      const int last = w.total - 1;
      // The last key tile of a packed sequence (the first one visited) also stages rows of the NEXT
      // sequence.  Their P is 0, but 0 * inf is NaN and dS K contracts over those rows: this warp,
      // the first reader of every staged K and V tile, zeroes them once the tile has landed.
      const int tail = p.cu_seqlens_k == nullptr ? kT : max(0, min(kT, w.g.k_len - (w.n_hi - 1) * kT));
      wq(&sh->res_full, wi & 1, 53);
      wq(&sh->full_a[posA % SK], (posA / SK) & 1, 54);
      if (ok && tail < kT) zero_tile_tail<C::kBoxes, kT>(slotK(posA), tail, lane);
      if (ok) {
        mma_kmajor<D>(tS + (tg & 1) * kT, sQ, slotK(posA), idesc_s, leader);      // S(0) = Q K(0)^T
        mma_commit_lp(smem_u32(&sh->s_full[tg & 1]), leader);
        if (last == 0) mma_commit_lp(smem_u32(&sh->res_free), leader);
      }
      wq(&sh->full_b[posB % SV], (posB / SV) & 1, 54);
      if (ok && tail < kT) zero_tile_tail<C::kBoxes, kT>(slotV(posB), tail, lane);
      if (ok) {
        mma_kmajor<D>(tdP, sdO, slotV(posB), idesc_s, leader);                    // dP(0) = dO V(0)^T
        mma_commit_lp(smem_u32(&sh->dp_full), leader);
        mma_commit_lp(smem_u32(&sh->empty_b[posB % SV]), leader);
        if (last == 0) mma_commit_lp(smem_u32(&sh->res_free), leader);
      }
      for (int k = 0; k < w.total && ok; ++k, ++tg) {
        const int kpos = posA + k, k1pos = kpos + 1, v1pos = posB + k + 1;
        const bool more = k < last;
        if (more) {
          wq(&sh->full_a[k1pos % SK], (k1pos / SK) & 1, 54);
          if (!ok) break;
          mma_kmajor<D>(tS + ((tg + 1) & 1) * kT, sQ, slotK(k1pos), idesc_s, leader);   // S(k+1)
          mma_commit_lp(smem_u32(&sh->s_full[(tg + 1) & 1]), leader);
          if (k + 1 == last) mma_commit_lp(smem_u32(&sh->res_free), leader);      // Q's last reader
        }
        wq(&sh->ds_ready, tg & 1, 55);
        if (!ok) break;
        mma_from_tmem<D>(tdQ, tdP, slotK(kpos), idesc_acc, k > 0, leader);        // dQ += dS(k) K(k)
        if (more) mma_commit_lp(smem_u32(&sh->empty_a[kpos % SK]), leader);       // (the epilogue releases the last)
        if (more) {
          wq(&sh->full_b[v1pos % SV], (v1pos / SV) & 1, 54);
          if (!ok) break;
          mma_kmajor<D>(tdP, sdO, slotV(v1pos), idesc_s, leader);                 // dP(k+1)
          mma_commit_lp(smem_u32(&sh->dp_full), leader);
          mma_commit_lp(smem_u32(&sh->empty_b[v1pos % SV]), leader);
          if (k + 1 == last) mma_commit_lp(smem_u32(&sh->res_free), leader);      // dO's last reader
        }
      }
      if (ok) mma_commit_lp(smem_u32(&sh->acc_done), leader);
      posA += w.total;
      posB += w.total;
      ++wi;
    }
    __syncwarp();
  } else {
    // ------------------------------- element-wise groups --------------------------------
    reg_alloc<kRegsEw>();
    const int x = warp >> 2;
    const int lrow = (warp & 3) * 32 + lane;  // TMEM lane = query row inside the tile
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tdPx = tdP + lane_addr + x * kHalfT;
    constexpr int DH = D / 2;                 // each group stores half of the head_dim columns
    bool ok = true;
    int posA = 0, wi = 0, tg = 0, sidx = 0;
    // statistics of this thread's row: base-2 LSE (+inf for rows that do not exist or see no
    // key: P = 0) and delta; those of the next item are fetched before the epilogue of this one
    auto row_stats = [&](const QItem& w, float& l2, float& dl) {
      l2 = INFINITY;
      dl = 0.f;
      const int row = w.m0 + lrow;
      if (row < w.g.q_len) {
        const int64_t idx = (int64_t)w.g.q_boff * p.lse_stride[0] + (int64_t)(w.g.q_row0 + row) * p.lse_stride[1] +
                            (int64_t)w.h * p.lse_stride[2];
        l2 = p.lse2[idx];
        dl = p.delta[idx];
        if (l2 == -INFINITY) l2 = INFINITY;
      }
    };
    float l2n = INFINITY, dln = 0.f;
    bool stats_ready = false;

    QItem w, wn;                                     // wn: the entry after the current one, once looked at
    bool peeked = false;
    for (;;) {
      if (peeked) {
        sched_release(sh, sidx++);
        w = wn;
      } else {
        w = sched_get<QItem>(sh, sidx++, true, ok);
      }
      if (!ok || w.total < 0) break;
      peeked = false;
      const int row = w.m0 + lrow;
      const int qpos = row + off;
      T* grow = nullptr;
      if (row < w.g.q_len)
        grow = reinterpret_cast<T*>(p.dq) + (int64_t)w.g.q_boff * p.dq_stride[0] +
               (int64_t)(w.g.q_row0 + row) * p.dq_stride[1] + (int64_t)w.h * p.dq_stride[2] + x * DH;
      if (w.total == 0) {
        // no key is visible from these rows: their gradient is zero
        if (grow != nullptr) {
#pragma unroll
          for (int c = 0; c < DH / 8; ++c) reinterpret_cast<uint4*>(grow)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      float l2, dl;
      if (stats_ready) { l2 = l2n; dl = dln; }
      else row_stats(w, l2, dl);
      const float slope = (kExtras && cfg.has_alibi) ? p.alibi_slopes[w.b * p.heads_q + w.h] : 0.f;
      int vk_lo, vk_hi;                              // key positions this thread's query row sees
      visible_k_interval(cfg, qpos, w.g.k_len, vk_lo, vk_hi);

      for (int j = 0; j < w.total && ok; ++j, ++tg) {
        const int k0 = (w.n_hi - 1 - j) * kT + x * kHalfT;   // first key of this thread's columns
        bool masked = (k0 + kHalfT > w.g.k_len);
        if (cfg.causal) masked |= (k0 + kHalfT - 1 > w.m0 + off);
        if (cfg.wl >= 0) masked |= (k0 < w.m0 + kT - 1 + off - cfg.wl);
        if (cfg.wr >= 0) masked |= (k0 + kHalfT - 1 > w.m0 + off + cfg.wr);

        ok = bwait(&sh->s_full[tg & 1], (tg >> 1) & 1, sh, 56);
        if (!ok) break;
        tc_fence_after();
        uint32_t r0[32], r1[32];
        const uint32_t tSx = tS + (tg & 1) * kT + lane_addr + x * kHalfT;
        tmem_ld32(tSx, r0);
        tmem_ld32(tSx + 32, r1);
        tmem_wait_ld();
        // ---- exp phase: P (times the soft cap's tanh factor) in fp32 registers -------------
        const float dist0 = (float)(qpos - k0);        // query position - key position of column 0
        float pf[kHalfT];
        // columns (keys) of this tile that this thread's query row sees
        const ColMask cm = make_col_mask(vk_lo - k0, vk_hi - k0);
        // One body, compiled per (masked tile, soft cap): no branch inside the unrolled loops.
        auto exp_body = [&](auto mask_tag, auto cap_tag, auto abs_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
          constexpr bool kCap = decltype(cap_tag)::value;
          constexpr bool kAbs = decltype(abs_tag)::value;
          if (kExtras) {
            // packed pairs; the distance of a pair's columns goes down by (2, 2)
            const FeatK fk = feat_k<kCap>(cfg, slope);
            const float cl = cfg.softcap * FA_LOG2E;
            const float2 cl2 = make_float2(cl, cl), nl2 = make_float2(-l2, -l2);
            const float2 one2 = make_float2(1.f, 1.f), none2 = make_float2(-1.f, -1.f), step2 = make_float2(-2.f, -2.f);
            float2 d2 = make_float2(dist0, dist0 - 1.f);
#pragma unroll
            for (int i = 0; i < kHalfT; i += 2) {
              const uint32_t* rr = i < 32 ? r0 : r1;
              const float2 sv2 = make_float2(__uint_as_float(rr[i & 31]), __uint_as_float(rr[(i & 31) + 1]));
              const float2 u2 = score_unit_feat2<kCap, kAbs>(fk, sv2, d2);
              const float2 a2 = kCap ? f2fma(u2, cl2, nl2) : f2add(u2, nl2);
              float2 pe = make_float2(ex2(a2.x), ex2(a2.y));
              if (kMask) {
                pe.x = col_visible(cm, i) ? pe.x : 0.f;
                pe.y = col_visible(cm, i + 1) ? pe.y : 0.f;
              }
              if (kCap) pe = f2mul(pe, f2fma(f2mul(u2, u2), none2, one2));   // times 1 - tanh^2
              pf[i] = pe.x;
              pf[i + 1] = pe.y;
              d2 = f2add(d2, step2);
            }
          } else {
            const float2 c2 = make_float2(cfg.scale_log2, cfg.scale_log2), nl = make_float2(-l2, -l2);
#pragma unroll
            for (int i = 0; i < kHalfT; i += 2) {
              const uint32_t* rr = i < 32 ? r0 : r1;
              const float2 a = f2fma(make_float2(__uint_as_float(rr[i & 31]), __uint_as_float(rr[(i & 31) + 1])), c2, nl);
              float2 pe = ex2_pair<kPolyEvery>(a, i >> 1);
              if (kMask) {
                pe.x = col_visible(cm, i) ? pe.x : 0.f;
                pe.y = col_visible(cm, i + 1) ? pe.y : 0.f;
              }
              pf[i] = pe.x;
              pf[i + 1] = pe.y;
            }
          }
        };
        const bool cap = kExtras && cfg.softcap > 0.f;
        const bool need_abs = kExtras && !cfg.causal;    // under the causal mask visible keys lie at distance >= 0
        auto run_exp = [&](auto mask_tag) {
          if (cap) {
            if (need_abs) exp_body(mask_tag, std::true_type{}, std::true_type{});
            else exp_body(mask_tag, std::true_type{}, std::false_type{});
          } else {
            if (need_abs) exp_body(mask_tag, std::false_type{}, std::true_type{});
            else exp_body(mask_tag, std::false_type{}, std::false_type{});
          }
        };
        if (masked) run_exp(std::true_type{});
        else run_exp(std::false_type{});

        // ---- dS phase --------------------------------------------------------------------
        ok = bwait(&sh->dp_full, tg & 1, sh, 57);
        if (!ok) break;
        tc_fence_after();
        tmem_ld32(tdPx, r0);
        tmem_ld32(tdPx + 32, r1);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[16];
          const uint32_t* rr = c == 0 ? r0 : r1;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 d = f2add(make_float2(__uint_as_float(rr[2 * i]), __uint_as_float(rr[2 * i + 1])),
                                   make_float2(-dl, -dl));
            const float2 ds = f2mul(make_float2(pf[c * 32 + 2 * i], pf[c * 32 + 2 * i + 1]), d);
            pk[i] = Elem<T>::pack(ds.x, ds.y);
          }
          tmem_st16(tdPx + c * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sh->ds_ready));
      }
      if (!ok) break;

      // ---- end of the item: fetch the next item's row statistics, then store dQ * softmax_scale --
      {
        wn = sched_get<QItem>(sh, sidx, false, ok);
        if (!ok) break;
        peeked = true;
        stats_ready = wn.total > 0;
        if (stats_ready) row_stats(wn, l2n, dln);
      }
      // The tile is staged over the item's last K tile (every MMA is done) and handed to the store
      // lane, which lets the TMA unit write it; a packed tile that crosses the end of its sequence
      // is stored row by row instead.
      const int spos = posA + w.total - 1;
      ok = bwait(&sh->acc_done, wi & 1, sh, 58);
      if (!ok) break;
      tc_fence_after();
      const bool via_tma = (p.cu_seqlens_q == nullptr) || (w.m0 + kT <= w.g.q_len);
      const uint32_t stg = slotK(spos);
      if (tid == 0)
        ok = post_store(sh, 0, wi, via_tma ? (int)stg : 0, w.h, w.g.q_row0 + w.m0, w.g.q_boff,
                        smem_u32(&sh->empty_a[spos % SK]));
      drain_acc<T, DH>(tdQ + lane_addr + x * DH, cfg.scale, via_tma, stg, lrow, x * DH, grow);
      tc_fence_before();
      if (via_tma) fence_proxy_async();
      mbar_arrive(smem_u32(&sh->stg_ready[0]));
      posA += w.total;
      ++wi;
    }
    // no more items: the store lane may leave
    if (ok) {
      if (tid == 0) ok = post_store(sh, 0, wi, -1, 0, 0, 0, 0);
      mbar_arrive(smem_u32(&sh->stg_ready[0]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
  if (tid == 0) {
    if (sh->abort_flag == 0) sched_finish(queue);
    report_abort(sh->abort_flag, host_status);
  }
}

// =======================================================================================
// host side
// =======================================================================================
bool bwd_sm100_supported(const fa_attn_args& a) {
  if (a.head_dim != 128 && a.head_dim != 64) return false;
  if (a.softmax_scale < 0.f) return false;
  if (a.batch == 0 || a.seqlen_q == 0 || a.seqlen_k == 0) return false;
  if (a.impl == FA_IMPL_AUTO && (a.seqlen_k < 256 || a.seqlen_q < 128)) return false;
  return true;
}

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

// candidates of a launch: blocks x heads x batch must stay a 32-bit count
bool candidate_count(int64_t blocks, int64_t heads, int64_t batch, int* out) {
  const int64_t n = blocks * heads * batch;
  if (n <= 0 || n > 0x7fffffff) return false;
  *out = (int)n;
  return true;
}

template <typename T, int D>
int launch_dkdv(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  Maps m{};
  if (!make_maps(m, a)) {
    set_error("bwd_dkdv_sm100: cuTensorMapEncodeTiled failed");
    return FA_ERR_LAUNCH;
  }
  // The plain variant folds -lse2 / scale_log2 into the score GEMM through 16-bit operands; a
  // scale so small that its reciprocal leaves the fp16 range takes the feature variant, whose
  // element-wise warps add the LSE themselves.
  const bool extras = cfg.has_alibi || cfg.softcap > 0.f || !(cfg.scale_log2 > 2e-5f);
  auto kern = extras ? bwd_dkdv_sm100_kernel<T, D, true> : bwd_dkdv_sm100_kernel<T, D, false>;
  if (int r = set_smem_attr(kern, BCfg<D>::kSmemBytes, "bwd_dkdv_sm100")) return r;
  const int nkb = (a.seqlen_k + kT - 1) / kT;
  int ncand = 0;
  if (!candidate_count(nkb, a.heads_kv, a.batch, &ncand)) {
    set_error("bwd_dkdv_sm100: too many work items");
    return FA_ERR_UNSUPPORTED;
  }
  unsigned int* queue = work_queue(a.device);
  if (queue == nullptr) return FA_ERR_LAUNCH;
  const int grid = ncand < sm_count(a.device) ? ncand : sm_count(a.device);
  kern<<<grid, kBwdThreads, BCfg<D>::kSmemBytes, st>>>(m.q, m.k, m.v, m.dout, m.dk, m.dv, a, cfg, nkb, ncand, queue,
                                                           host_wait_word(a.device));
  return check_launch("bwd_dkdv_sm100");
}

template <typename T, int D>
int launch_dq(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  Maps m{};
  if (!make_maps(m, a)) {
    set_error("bwd_dq_sm100: cuTensorMapEncodeTiled failed");
    return FA_ERR_LAUNCH;
  }
  const bool extras = cfg.has_alibi || cfg.softcap > 0.f;
  auto kern = extras ? bwd_dq_sm100_kernel<T, D, true> : bwd_dq_sm100_kernel<T, D, false>;
  if (int r = set_smem_attr(kern, BCfg<D>::kSmemBytesDq, "bwd_dq_sm100")) return r;
  const int nmb = (a.seqlen_q + kT - 1) / kT;
  int ncand = 0;
  if (!candidate_count(nmb, a.heads_q, a.batch, &ncand)) {
    set_error("bwd_dq_sm100: too many work items");
    return FA_ERR_UNSUPPORTED;
  }
  unsigned int* queue = work_queue(a.device);
  if (queue == nullptr) return FA_ERR_LAUNCH;
  const int grid = ncand < sm_count(a.device) ? ncand : sm_count(a.device);
  kern<<<grid, kBwdThreads, BCfg<D>::kSmemBytesDq, st>>>(m.q, m.k, m.v, m.dout, m.dq, a, cfg, nmb, ncand, queue,
                                                             host_wait_word(a.device));
  return check_launch("bwd_dq_sm100");
}

}  // namespace

int bwd_dkdv_cta_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st);

#ifndef FA_DKDV_CTA_BELOW
#define FA_DKDV_CTA_BELOW 1e9    // plain dense work items shorter than this many tiles go to the one-CTA-per-key-block kernel
#endif
// Average number of query tiles a block of 128 keys meets (times the GQA group): what one work
// item of the dK/dV kernels amounts to.  Dense layout only (the lengths of a packed batch live
// on the device).
static double dkdv_tiles_per_item(const fa_attn_args& a, const ScoreCfg& cfg) {
  const int nkb = (a.seqlen_k + kT - 1) / kT, off = a.q_pos_offset;
  long long sum = 0;
  for (int n = 0; n < nkb; ++n) {
    int qlo, qhi;
    const int k_last = (n * kT + kT < a.seqlen_k ? n * kT + kT : a.seqlen_k) - 1;
    visible_query_range(cfg, n * kT, k_last, off, a.seqlen_q + off, qlo, qhi);
    const int m_lo = (qlo - off > 0 ? qlo - off : 0) / kT, m_hi = ((qhi - off > 0 ? qhi - off : 0) + kT - 1) / kT;
    if (m_hi > m_lo) sum += m_hi - m_lo;
  }
  return (double)sum / nkb * (a.heads_q / a.heads_kv);
}

int bwd_dkdv_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  // Two kernels (see bwd_dkdv_cta_sm100.cu): a plain dense problem goes to the one-CTA-per-key-block
  // kernel (since it keeps K in shared memory and P, dS apart it wins at every item length: 2-7 %
  // without a mask, 10-15 % with the causal mask or GQA, measured at 16-66 tiles per item),
  // packed batches and the feature variants to the persistent one.
  const bool features = cfg.has_alibi || cfg.softcap > 0.f || !(cfg.scale_log2 > 2e-5f);
  double below = FA_DKDV_CTA_BELOW;
  if (const char* e = getenv("FA_B200_DKDV_CTA_BELOW")) below = atof(e);   // tuning / tests: 0 = never
  if (!features && a.cu_seqlens_q == nullptr && dkdv_tiles_per_item(a, cfg) < below)
    return bwd_dkdv_cta_sm100(a, cfg, st);
  if (a.head_dim == 128)
    return a.dtype == FA_BF16 ? launch_dkdv<__nv_bfloat16, 128>(a, cfg, st) : launch_dkdv<__half, 128>(a, cfg, st);
  return a.dtype == FA_BF16 ? launch_dkdv<__nv_bfloat16, 64>(a, cfg, st) : launch_dkdv<__half, 64>(a, cfg, st);
}

int bwd_dq_sm100(const fa_attn_args& a, const ScoreCfg& cfg, cudaStream_t st) {
  if (a.head_dim == 128)
    return a.dtype == FA_BF16 ? launch_dq<__nv_bfloat16, 128>(a, cfg, st) : launch_dq<__half, 128>(a, cfg, st);
  return a.dtype == FA_BF16 ? launch_dq<__nv_bfloat16, 64>(a, cfg, st) : launch_dq<__half, 64>(a, cfg, st);
}

int bwd_dkdv_cta_status();
void bwd_dkdv_cta_clear_status();

void bwd_sm100_clear_status() {
  const int z = 0;
  cudaMemcpyToSymbol(g_bwd_sm100_status, &z, sizeof(int));
  bwd_dkdv_cta_clear_status();
}

int bwd_sm100_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_bwd_sm100_status, sizeof(int));
  return v != 0 ? v : bwd_dkdv_cta_status();
}

}  // namespace fa
