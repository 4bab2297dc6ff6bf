// Stall accounting for kernel tuning.  Compiled in only with -DFA_PROF (a tagged side build,
// never the shipped library): chosen threads add up the clock64 cycles they spend in each kind of
// wait and flush the sums to a global array that fa_debug_prof_<tag>() copies out.  Without
// FA_PROF every macro is empty and no symbol is exported.  A translation unit defines PROF_TAG
// (its array and accessor are named after it) before including this header.
#pragma once

#ifdef FA_PROF
#define PROF_CAT2(a, b) a##b
#define PROF_CAT(a, b) PROF_CAT2(a, b)
#define PROF_ARRAY PROF_CAT(g_prof_, PROF_TAG)
namespace fa {
__device__ unsigned long long PROF_ARRAY[64];
}
extern "C" int PROF_CAT(fa_debug_prof_, PROF_TAG)(unsigned long long* out, int reset) {
  int r = (int)cudaMemcpyFromSymbol(out, fa::PROF_ARRAY, sizeof(unsigned long long) * 64);
  if (reset) {
    unsigned long long z[64] = {0};
    cudaMemcpyToSymbol(fa::PROF_ARRAY, z, sizeof(z));
  }
  return r;
}
#define PROF_VARS(n) unsigned int prof_acc[n] = {0}; long long prof_t0 = 0; (void)prof_t0
#define PROF_T0() prof_t0 = clock64()
#define PROF_ADD(slot) prof_acc[slot] += (unsigned int)(clock64() - prof_t0)
#define PROF_COUNT(slot, v) prof_acc[slot] += (unsigned int)(v)
#define PROF_FLUSH(cond, base, n)                                                    \
  do {                                                                               \
    if (cond) {                                                                      \
      for (int pi = 0; pi < (n); ++pi) atomicAdd(&fa::PROF_ARRAY[(base) + pi], (unsigned long long)prof_acc[pi]); \
    }                                                                                \
  } while (0)
#else
#define PROF_VARS(n) do {} while (0)
#define PROF_T0() do {} while (0)
#define PROF_ADD(slot) do {} while (0)
#define PROF_COUNT(slot, v) do {} while (0)
#define PROF_FLUSH(cond, base, n) do {} while (0)
#endif
