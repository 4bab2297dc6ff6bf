// C ABI: argument validation, kernel-family dispatch, error strings.  See include/fa_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace fa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  return FA_OK;
}

int ensure_device(int device) {
  int cur = -1;
  cudaError_t e = cudaGetDevice(&cur);
  if (e == cudaSuccess && cur == device) return FA_OK;
  e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    set_error("cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  return FA_OK;
}

int sm_count(int device) {
  static int cached[64] = {0};
  const bool slot = device >= 0 && device < 64;
  if (slot && cached[device] > 0) return cached[device];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
  if (slot) cached[device] = n;
  return n;
}

// One word per device ordinal, in a page of its own that is registered (pinned and mapped) on
// first use: no allocation, the kernels write it through the mapping, the host just reads it.
alignas(4096) static volatile int g_host_wait[1024];
static std::mutex g_host_wait_mu;
static int g_host_wait_registered = 0;   // 0 not tried, 1 mapped, -1 unavailable

int* host_wait_word(int device) {
  if (device < 0 || device >= 1024) return nullptr;
  std::lock_guard<std::mutex> lock(g_host_wait_mu);
  if (g_host_wait_registered == 0) {
    cudaError_t e = cudaHostRegister(const_cast<int*>(g_host_wait), sizeof(g_host_wait),
                                     cudaHostRegisterPortable | cudaHostRegisterMapped);
    g_host_wait_registered = (e == cudaSuccess) ? 1 : -1;
    if (e != cudaSuccess) cudaGetLastError();
  }
  if (g_host_wait_registered != 1) return nullptr;
  int* dptr = nullptr;
  if (cudaHostGetDevicePointer(&dptr, const_cast<int*>(&g_host_wait[device]), 0) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return dptr;
}

int host_wait_status(int device) { return (device >= 0 && device < 1024) ? g_host_wait[device] : 0; }

static __device__ unsigned int g_work_queues[kWorkQueues][2];

unsigned int* work_queue(int device) {
  static unsigned int* base[64] = {nullptr};
  static std::mutex mu;
  static unsigned int turn = 0;
  if (device < 0 || device >= 64) {
    set_error("device ordinal %d out of range for the work queues", device);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (base[device] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_work_queues);
    if (e != cudaSuccess || p == nullptr) {
      set_error("cudaGetSymbolAddress(work queues) on device %d: %s", device, cudaGetErrorString(e));
      return nullptr;
    }
    base[device] = static_cast<unsigned int*>(p);
  }
  return base[device] + 2 * (turn++ % kWorkQueues);
}

// kernel families (defined in the other translation units)
int fwd_mma(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
int attn_probs(const fa_attn_args&, const ScoreCfg&, float*, const int64_t*, float*, int64_t, cudaStream_t);
int bwd_preprocess(const fa_attn_args&, cudaStream_t);
int bwd_dq_mma(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
int bwd_dkdv_mma(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
bool fwd_sm100_supported(const fa_attn_args&);
int fwd_sm100(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
bool bwd_sm100_supported(const fa_attn_args&);
int bwd_dq_sm100(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
int bwd_dkdv_sm100(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
int decode_paged(const fa_decode_args&, cudaStream_t);
size_t decode_workspace_bytes(const fa_decode_args&);
int decode_paged_static(const fa_decode_args&, cudaStream_t);
size_t decode_static_scratch_bytes();
int quantize_k(const void*, int8_t*, float*, int64_t, int, cudaStream_t);
int fwd_int8_mma(const fa_int8_args&, cudaStream_t);
bool fwd_int8_sm100_supported(const fa_int8_args&);
int fwd_int8_sm100(const fa_int8_args&, cudaStream_t);
int rotary(const fa_rotary_args&, cudaStream_t);
int gather_rows(const void*, void*, const int64_t*, int64_t, int64_t, int64_t, int, cudaStream_t);
int scatter_rows(const void*, void*, const int64_t*, int64_t, int64_t, int64_t, int, int, cudaStream_t);
int fwd_sm100_status();
int bwd_sm100_status();
void fwd_sm100_clear_status();
void bwd_sm100_clear_status();
int wait_probe(int device, long long clocks, cudaStream_t st);
int mma_peak_probe(int device, int kind, int iters, cudaStream_t st);

static bool mult8(const int64_t* s, int n) {
  for (int i = 0; i < n; ++i)
    if (s[i] % 8 != 0) return false;
  return true;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int validate_common(const fa_attn_args* a, bool need_cu) {
  FA_REQUIRE(a != nullptr, "args is NULL");
  FA_REQUIRE(a->dtype == FA_F16 || a->dtype == FA_BF16, "dtype must be FA_F16 or FA_BF16");
  FA_REQUIRE(a->batch >= 0 && a->seqlen_q >= 0 && a->seqlen_k >= 0, "negative size");
  FA_REQUIRE(a->heads_q > 0 && a->heads_kv > 0 && a->heads_q % a->heads_kv == 0,
             "heads_q (%d) must be a positive multiple of heads_kv (%d)", a->heads_q, a->heads_kv);
  FA_REQUIRE(a->head_dim == 16 || a->head_dim == 32 || a->head_dim == 64 || a->head_dim == 128 ||
                 a->head_dim == 256,
             "head dimension must be one of 16, 32, 64, 128, or 256 (got %d)", a->head_dim);
  FA_REQUIRE(a->softcap >= 0.f, "softcap must be non-negative");
  FA_REQUIRE(a->dropout_p >= 0.f && a->dropout_p < 1.f, "dropout_p must be in the range [0, 1)");
  FA_REQUIRE(a->dropout_p == 0.f || a->dropout_row_stride > 0, "dropout needs dropout_row_stride > 0");
  FA_REQUIRE(a->attn_bias == nullptr || a->cu_seqlens_q == nullptr, "attn_bias is for the dense layout only");
  FA_REQUIRE((a->seqused_q == nullptr && a->seqused_k == nullptr) || a->cu_seqlens_q != nullptr,
             "seqused_q/seqused_k need the packed layout");
  FA_REQUIRE((a->cu_seqlens_q == nullptr) == (a->cu_seqlens_k == nullptr),
             "cu_seqlens_q and cu_seqlens_k must be given together");
  if (need_cu) FA_REQUIRE(a->cu_seqlens_q != nullptr, "packed layout needs cu_seqlens_q/k");
  if (a->cu_seqlens_q) {
    FA_REQUIRE(a->q_pos_offset == 0, "q_pos_offset is dense-only");
    FA_REQUIRE(a->total_q >= 0 && a->total_k >= 0, "total_q/total_k must be the packed row counts");
  }
  const bool empty = a->batch == 0 || a->seqlen_q == 0;
  if (!empty) {
    FA_REQUIRE(a->q && a->o, "q/o is NULL");
    FA_REQUIRE(a->seqlen_k == 0 || (a->k && a->v), "k/v is NULL");
    FA_REQUIRE(aligned16(a->q) && aligned16(a->k) && aligned16(a->v) && aligned16(a->o),
               "q/k/v/o must be 16-byte aligned");
    FA_REQUIRE(mult8(a->q_stride, 3) && mult8(a->k_stride, 3) && mult8(a->v_stride, 3) &&
                   mult8(a->o_stride, 3),
               "strides must be multiples of 8 elements (16-byte rows)");
  }
  return FA_OK;
}

static int validate_bwd(const fa_attn_args* a) {
  if (a->batch == 0 || a->seqlen_q == 0) return FA_OK;
  FA_REQUIRE(a->dout && a->lse2 && a->delta, "backward needs dout, lse2 and delta");
  FA_REQUIRE(aligned16(a->dout) && mult8(a->do_stride, 3), "dout alignment/stride");
  return FA_OK;
}

static ScoreCfg cfg_of(const fa_attn_args* a) {
  ScoreCfg c = make_score_cfg(a->softmax_scale, a->softcap, a->causal, a->window_left, a->window_right,
                              a->alibi_slopes != nullptr);
  c.bias = a->attn_bias;
  for (int i = 0; i < 4; ++i) c.bias_stride[i] = a->bias_stride[i];
  if (a->dropout_p > 0.f) {
    c.dropout_p = a->dropout_p;
    c.dropout_scale = 1.f / (1.f - a->dropout_p);
    c.seed_lo = (uint32_t)(a->dropout_seed & 0xffffffffull);
    c.seed_hi = (uint32_t)(a->dropout_seed >> 32);
    c.drop_stride = (uint32_t)a->dropout_row_stride;
  }
  return c;
}

// Bias and dropout are features of the mma.sync kernels.
static bool needs_mma(const fa_attn_args* a) { return a->attn_bias != nullptr || a->dropout_p > 0.f; }

// A bounded wait that ran out earlier on this device (host mirror of the status word): the tcgen05
// kernels would return at their first wait, so the call is refused before anything is launched.
static int refuse_after_timeout(int device, const char* what) {
  if (const int c = host_wait_status(device)) {
    set_error("%s: a bounded device-side wait ran out earlier on device %d (code %d); the tcgen05 kernels stay "
              "off until fa_device_wait_clear()", what, device, c);
    return FA_ERR_DEVICE_WAIT;
  }
  return FA_OK;
}

static int fwd_impl(const fa_attn_args* a, void* stream, bool need_cu) {
  if (int r = validate_common(a, need_cu)) return r;
  if (a->impl != FA_IMPL_MMA && fwd_sm100_supported(*a) && !needs_mma(a))
    if (int r = refuse_after_timeout(a->device, "fa_fwd")) return r;
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const ScoreCfg cfg = cfg_of(a);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!fwd_sm100_supported(*a) || needs_mma(a)) {
      set_error("no tcgen05 forward kernel for this shape/feature set");
      return FA_ERR_UNSUPPORTED;
    }
    return fwd_sm100(*a, cfg, st);
  }
  if (a->impl == FA_IMPL_AUTO && fwd_sm100_supported(*a) && !needs_mma(a)) return fwd_sm100(*a, cfg, st);
  return fwd_mma(*a, cfg, st);
}

static int dq_impl(const fa_attn_args* a, void* stream, bool need_cu) {
  if (int r = validate_common(a, need_cu)) return r;
  if (int r = validate_bwd(a)) return r;
  if (a->batch && a->seqlen_q) {
    FA_REQUIRE(a->dq && aligned16(a->dq) && mult8(a->dq_stride, 3), "dq pointer/alignment/stride");
  }
  if (a->impl != FA_IMPL_MMA && bwd_sm100_supported(*a) && !needs_mma(a))
    if (int r = refuse_after_timeout(a->device, "fa_bwd_dq")) return r;
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const ScoreCfg cfg = cfg_of(a);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!bwd_sm100_supported(*a) || needs_mma(a)) {
      set_error("no tcgen05 backward kernel for this shape/feature set");
      return FA_ERR_UNSUPPORTED;
    }
    return bwd_dq_sm100(*a, cfg, st);
  }
  if (a->impl == FA_IMPL_AUTO && bwd_sm100_supported(*a) && !needs_mma(a)) return bwd_dq_sm100(*a, cfg, st);
  return bwd_dq_mma(*a, cfg, st);
}

static int dkdv_impl(const fa_attn_args* a, void* stream, bool need_cu) {
  if (int r = validate_common(a, need_cu)) return r;
  if (int r = validate_bwd(a)) return r;
  if (a->batch && a->seqlen_k) {
    FA_REQUIRE(a->dk && a->dv && aligned16(a->dk) && aligned16(a->dv) && mult8(a->dk_stride, 3) &&
                   mult8(a->dv_stride, 3),
               "dk/dv pointer/alignment/stride");
  }
  if (a->impl != FA_IMPL_MMA && bwd_sm100_supported(*a) && !needs_mma(a))
    if (int r = refuse_after_timeout(a->device, "fa_bwd_dkdv")) return r;
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const ScoreCfg cfg = cfg_of(a);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!bwd_sm100_supported(*a) || needs_mma(a)) {
      set_error("no tcgen05 backward kernel for this shape/feature set");
      return FA_ERR_UNSUPPORTED;
    }
    return bwd_dkdv_sm100(*a, cfg, st);
  }
  if (a->impl == FA_IMPL_AUTO && bwd_sm100_supported(*a) && !needs_mma(a)) return bwd_dkdv_sm100(*a, cfg, st);
  return bwd_dkdv_mma(*a, cfg, st);
}

}  // namespace fa

using namespace fa;

extern "C" {

int fa_fwd(const fa_attn_args* a, void* stream) { return fwd_impl(a, stream, false); }
int fa_varlen_fwd(const fa_attn_args* a, void* stream) { return fwd_impl(a, stream, true); }

int fa_attn_probs(const fa_attn_args* a, float* probs, const int64_t* probs_stride, float* lse_nat,
                  int64_t lse_nat_stride, void* stream) {
  if (int r = validate_common(a, false)) return r;
  if (a->batch == 0 || a->seqlen_q == 0 || a->seqlen_k == 0) return FA_OK;
  FA_REQUIRE(probs != nullptr && probs_stride != nullptr && a->lse2 != nullptr, "probs, probs_stride and lse2 are required");
  if (int r = ensure_device(a->device)) return r;
  return attn_probs(*a, cfg_of(a), probs, probs_stride, lse_nat, lse_nat_stride, reinterpret_cast<cudaStream_t>(stream));
}

int fa_bwd_preprocess(const fa_attn_args* a, void* stream) {
  if (int r = validate_common(a, false)) return r;
  if (int r = validate_bwd(a)) return r;
  if (int r = ensure_device(a->device)) return r;
  return bwd_preprocess(*a, reinterpret_cast<cudaStream_t>(stream));
}

int fa_bwd_dq(const fa_attn_args* a, void* stream) { return dq_impl(a, stream, false); }
int fa_varlen_bwd_dq(const fa_attn_args* a, void* stream) { return dq_impl(a, stream, true); }
int fa_bwd_dkdv(const fa_attn_args* a, void* stream) { return dkdv_impl(a, stream, false); }
int fa_varlen_bwd_dkdv(const fa_attn_args* a, void* stream) { return dkdv_impl(a, stream, true); }

static int validate_decode(const fa_decode_args* a) {
  FA_REQUIRE(a != nullptr, "args is NULL");
  FA_REQUIRE(a->dtype == FA_F16 || a->dtype == FA_BF16, "dtype must be FA_F16 or FA_BF16");
  FA_REQUIRE(a->batch >= 0 && a->seqlen_q >= 0, "negative size");
  FA_REQUIRE(a->heads_q > 0 && a->heads_kv > 0 && a->heads_q % a->heads_kv == 0,
             "heads_q must be a positive multiple of heads_kv");
  FA_REQUIRE(a->head_dim == 16 || a->head_dim == 32 || a->head_dim == 64 || a->head_dim == 128 ||
                 a->head_dim == 256,
             "head dimension must be one of 16, 32, 64, 128, or 256 (got %d)", a->head_dim);
  if (a->batch == 0 || a->seqlen_q == 0) return FA_OK;
  FA_REQUIRE(a->q && a->o && a->k_cache && a->v_cache && a->cache_seqlens,
             "q, o, k_cache, v_cache and cache_seqlens are required");
  FA_REQUIRE(a->page_size > 0, "page_size must be positive");
  FA_REQUIRE(aligned16(a->k_cache) && aligned16(a->v_cache) && mult8(a->kc_stride, 3) &&
                 mult8(a->vc_stride, 3),
             "cache rows must be 16-byte aligned");
  FA_REQUIRE(aligned16(a->q) && aligned16(a->o), "q and o must be 16-byte aligned");
  FA_REQUIRE(mult8(a->q_stride, 3) && mult8(a->o_stride, 3), "q/o strides must be multiples of 8 elements");
  FA_REQUIRE(a->workspace == nullptr || aligned16(a->workspace), "workspace must be 16-byte aligned");
  FA_REQUIRE(a->num_splits >= 0, "num_splits must be non-negative");
  FA_REQUIRE(a->block_table == nullptr || a->block_table_stride > 0,
             "block_table_stride must be positive when a block table is given");
  FA_REQUIRE(!(a->block_table && a->cache_batch_idx), "cache_batch_idx cannot be combined with paged KV caches");
  FA_REQUIRE(!(a->block_table && a->cache_leftpad), "cache_leftpad cannot be combined with paged KV caches");
  FA_REQUIRE((a->k_new == nullptr) == (a->v_new == nullptr), "k and v must be supplied together");
  FA_REQUIRE((a->rotary_cos == nullptr) == (a->rotary_sin == nullptr),
             "rotary_cos and rotary_sin must be supplied together");
  if (a->rotary_cos) {
    FA_REQUIRE(a->rotary_dim > 0 && a->rotary_dim % 2 == 0 && a->rotary_dim <= a->head_dim,
               "rotary tables exceed the head dimension");
    FA_REQUIRE(a->rotary_seqlen > 0, "rotary_seqlen must be the number of rows of the rotary tables");
  }
  if (a->k_new) {
    FA_REQUIRE(a->seqlen_new > 0, "seqlen_new must be positive when k/v are given");
    FA_REQUIRE(aligned16(a->k_new) && aligned16(a->v_new) && mult8(a->kn_stride, 3) && mult8(a->vn_stride, 3),
               "new k/v rows must be 16-byte aligned");
  }
  return FA_OK;
}

int fa_decode_paged(const fa_decode_args* a, void* stream) {
  if (int r = validate_decode(a)) return r;
  if (int r = ensure_device(a->device)) return r;
  return decode_paged(*a, reinterpret_cast<cudaStream_t>(stream));
}

int fa_decode_paged_static(const fa_decode_args* a, void* stream) {
  if (int r = validate_decode(a)) return r;
  if (int r = ensure_device(a->device)) return r;
  return decode_paged_static(*a, reinterpret_cast<cudaStream_t>(stream));
}

size_t fa_decode_static_scratch_bytes(void) { return decode_static_scratch_bytes(); }

size_t fa_decode_workspace_bytes(const fa_decode_args* a) {
  if (a == nullptr || a->heads_kv <= 0 || a->heads_q <= 0 || a->page_size <= 0) return 0;
  return decode_workspace_bytes(*a);
}

int fa_quantize_k_int8(const void* k, int8_t* k8, float* s_k, int64_t rows, int32_t head_dim,
                       int32_t device, void* stream) {
  FA_REQUIRE(rows >= 0, "negative rows");
  if (rows == 0) return FA_OK;
  FA_REQUIRE(k && k8 && s_k, "NULL pointer");
  FA_REQUIRE(aligned16(k) && (reinterpret_cast<uintptr_t>(k8) & 7) == 0, "k must be 16-byte, k8 8-byte aligned");
  FA_REQUIRE(head_dim >= 32 && (head_dim & (head_dim - 1)) == 0,
             "The INT8 kernel requires a power-of-two head dim of at least 32");
  if (int r = ensure_device(device)) return r;
  return quantize_k(k, k8, s_k, rows, head_dim, reinterpret_cast<cudaStream_t>(stream));
}

int fa_fwd_int8(const fa_int8_args* a, void* stream) {
  FA_REQUIRE(a != nullptr, "args is NULL");
  FA_REQUIRE(a->batch >= 0 && a->heads >= 0 && a->seqlen >= 0, "negative size");
  FA_REQUIRE(a->head_dim >= 32 && (a->head_dim & (a->head_dim - 1)) == 0,
             "The INT8 kernel requires a power-of-two head dim of at least 32");
  if (a->batch * a->heads == 0 || a->seqlen == 0) return FA_OK;
  FA_REQUIRE(a->q && a->k8 && a->s_k && a->v && a->o, "NULL pointer");
  FA_REQUIRE(a->seqlen_k_valid >= 0 && a->seqlen_k_valid <= a->seqlen, "seqlen_k_valid must lie in [0, seqlen]");
  FA_REQUIRE(aligned16(a->q) && aligned16(a->k8) && aligned16(a->v) && aligned16(a->o), "16-byte alignment");
  if (a->impl != FA_IMPL_MMA && fwd_int8_sm100_supported(*a))
    if (int r = refuse_after_timeout(a->device, "fa_fwd_int8")) return r;
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!fwd_int8_sm100_supported(*a)) {
      set_error("no tcgen05 INT8 kernel for this shape");
      return FA_ERR_UNSUPPORTED;
    }
    return fwd_int8_sm100(*a, st);
  }
  if (a->impl == FA_IMPL_AUTO && fwd_int8_sm100_supported(*a)) return fwd_int8_sm100(*a, st);
  return fwd_int8_mma(*a, st);
}

int fa_rotary(const fa_rotary_args* a, void* stream) {
  FA_REQUIRE(a != nullptr, "args is NULL");
  FA_REQUIRE(a->dtype == FA_F16 || a->dtype == FA_BF16 || a->dtype == FA_F32, "dtype must be FA_F16, FA_BF16 or FA_F32");
  FA_REQUIRE(a->batch >= 0 && a->seqlen >= 0 && a->heads >= 0 && a->head_dim > 0, "negative size");
  FA_REQUIRE(a->head_dim <= 256, "Only support headdim <= 256");
  FA_REQUIRE(a->rotary_dim >= 0 && a->rotary_dim % 2 == 0 && a->rotary_dim <= a->head_dim,
             "rotary_dim must be even and <= headdim");
  FA_REQUIRE(a->rotary_seqlen >= 0, "negative rotary table length");
  if (a->batch == 0 || a->seqlen == 0 || a->heads == 0) return FA_OK;
  FA_REQUIRE(a->x && a->out, "x/out is NULL");
  FA_REQUIRE(a->rotary_dim == 0 || (a->cos && a->sin), "cos/sin is NULL");
  if (int r = ensure_device(a->device)) return r;
  return rotary(*a, reinterpret_cast<cudaStream_t>(stream));
}

static int validate_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                         int64_t rows) {
  FA_REQUIRE(n_idx >= 0 && row_bytes >= 0 && rows >= 0, "negative size");
  if (n_idx == 0 || row_bytes == 0) return FA_OK;
  FA_REQUIRE(src && dst && idx, "NULL pointer");
  FA_REQUIRE(row_bytes % 16 == 0 && aligned16(src) && aligned16(dst), "rows must be 16-byte multiples, 16-byte aligned");
  FA_REQUIRE(row_bytes / 16 <= 0x7fffffff, "row too long");
  return FA_OK;
}

int fa_gather_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                   int64_t src_rows, int32_t device, void* stream) {
  if (int r = validate_rows(src, dst, idx, n_idx, row_bytes, src_rows)) return r;
  if (n_idx == 0 || row_bytes == 0) return FA_OK;
  if (int r = ensure_device(device)) return r;
  return gather_rows(src, dst, idx, n_idx, row_bytes, src_rows, device, reinterpret_cast<cudaStream_t>(stream));
}

int fa_scatter_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                    int64_t dst_rows, int32_t add_dtype, int32_t device, void* stream) {
  if (int r = validate_rows(src, dst, idx, n_idx, row_bytes, dst_rows)) return r;
  FA_REQUIRE(add_dtype >= -1 && add_dtype <= FA_F32, "add_dtype must be -1 or an fa_dtype");
  if (n_idx == 0 || row_bytes == 0) return FA_OK;
  if (int r = ensure_device(device)) return r;
  return scatter_rows(src, dst, idx, n_idx, row_bytes, dst_rows, add_dtype, device,
                      reinterpret_cast<cudaStream_t>(stream));
}

const char* fa_version(void) { return "fa_b200 0.1 (sm_100a)"; }
const char* fa_last_error(void) { return g_err; }
int fa_fwd_uses_tcgen05(const fa_attn_args* a) {
  return a != nullptr && a->impl != FA_IMPL_MMA && fwd_sm100_supported(*a) ? 1 : 0;
}

int fa_device_wait_status(int device) {
  if (int r = ensure_device(device)) return r;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  int s = fwd_sm100_status();
  if (s == 0) s = bwd_sm100_status();
  if (s == 0) s = host_wait_status(device);
  if (s != 0 && device >= 0 && device < 1024) g_host_wait[device] = s;   // remembered for the launchers
  return s;
}

int fa_device_wait_clear(int device) {
  if (int r = ensure_device(device)) return r;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    return FA_ERR_LAUNCH;
  }
  fwd_sm100_clear_status();
  bwd_sm100_clear_status();
  if (device >= 0 && device < 1024) g_host_wait[device] = 0;
  return FA_OK;
}

int fa_wait_probe(int32_t device, int64_t clocks, void* stream) {
  FA_REQUIRE(clocks > 0 && clocks <= 2000000000LL, "clocks must be in (0, 2e9]");
  if (int r = ensure_device(device)) return r;
  return wait_probe(device, clocks, reinterpret_cast<cudaStream_t>(stream));
}

int fa_mma_peak_probe(int32_t device, int32_t kind, int32_t iters, void* stream) {
  FA_REQUIRE(kind == 0 || kind == 1, "kind: 0 = fp16 operands, 1 = int8 operands");
  FA_REQUIRE(iters > 0 && iters <= (1 << 24), "iters must be in (0, 2^24]");
  if (int r = ensure_device(device)) return r;
  return mma_peak_probe(device, kind, iters, reinterpret_cast<cudaStream_t>(stream));
}

int fa_debug_set_wait_status(int32_t device, int32_t code) {
  FA_REQUIRE(device >= 0 && device < 1024, "device ordinal out of range");
  g_host_wait[device] = code;
  return FA_OK;
}

size_t fa_sizeof_args(int which) {
  switch (which) {
    case 0: return sizeof(fa_attn_args);
    case 1: return sizeof(fa_decode_args);
    case 2: return sizeof(fa_int8_args);
    case 3: return sizeof(fa_rotary_args);
  }
  return 0;
}

}  // extern "C"
