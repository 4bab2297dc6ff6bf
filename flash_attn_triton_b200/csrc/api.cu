// C ABI: argument validation, kernel-family dispatch, error strings.  See include/fa_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

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

// kernel families (defined in the other translation units)
int fwd_mma(const fa_attn_args&, const ScoreCfg&, cudaStream_t);
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
int fwd_sm100_status();
int bwd_sm100_status();

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
  return make_score_cfg(a->softmax_scale, a->softcap, a->causal, a->window_left, a->window_right,
                        a->alibi_slopes != nullptr);
}

static int fwd_impl(const fa_attn_args* a, void* stream, bool need_cu) {
  if (int r = validate_common(a, need_cu)) return r;
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const ScoreCfg cfg = cfg_of(a);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!fwd_sm100_supported(*a)) {
      set_error("no tcgen05 forward kernel for this shape/feature set");
      return FA_ERR_UNSUPPORTED;
    }
    return fwd_sm100(*a, cfg, st);
  }
  if (a->impl == FA_IMPL_AUTO && fwd_sm100_supported(*a)) return fwd_sm100(*a, cfg, st);
  return fwd_mma(*a, cfg, st);
}

static int dq_impl(const fa_attn_args* a, void* stream, bool need_cu) {
  if (int r = validate_common(a, need_cu)) return r;
  if (int r = validate_bwd(a)) return r;
  if (a->batch && a->seqlen_q) {
    FA_REQUIRE(a->dq && aligned16(a->dq) && mult8(a->dq_stride, 3), "dq pointer/alignment/stride");
  }
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const ScoreCfg cfg = cfg_of(a);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!bwd_sm100_supported(*a)) {
      set_error("no tcgen05 backward kernel for this shape/feature set");
      return FA_ERR_UNSUPPORTED;
    }
    return bwd_dq_sm100(*a, cfg, st);
  }
  if (a->impl == FA_IMPL_AUTO && bwd_sm100_supported(*a)) return bwd_dq_sm100(*a, cfg, st);
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
  if (int r = ensure_device(a->device)) return r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const ScoreCfg cfg = cfg_of(a);
  if (a->impl == FA_IMPL_TCGEN05) {
    if (!bwd_sm100_supported(*a)) {
      set_error("no tcgen05 backward kernel for this shape/feature set");
      return FA_ERR_UNSUPPORTED;
    }
    return bwd_dkdv_sm100(*a, cfg, st);
  }
  if (a->impl == FA_IMPL_AUTO && bwd_sm100_supported(*a)) return bwd_dkdv_sm100(*a, cfg, st);
  return bwd_dkdv_mma(*a, cfg, st);
}

}  // namespace fa

using namespace fa;

extern "C" {

int fa_fwd(const fa_attn_args* a, void* stream) { return fwd_impl(a, stream, false); }
int fa_varlen_fwd(const fa_attn_args* a, void* stream) { return fwd_impl(a, stream, true); }

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
  FA_REQUIRE(!(a->block_table && a->cache_batch_idx), "cache_batch_idx cannot be combined with paged KV caches");
  FA_REQUIRE(!(a->block_table && a->cache_leftpad), "cache_leftpad cannot be combined with paged KV caches");
  FA_REQUIRE((a->k_new == nullptr) == (a->v_new == nullptr), "k and v must be supplied together");
  FA_REQUIRE((a->rotary_cos == nullptr) == (a->rotary_sin == nullptr),
             "rotary_cos and rotary_sin must be supplied together");
  if (a->rotary_cos)
    FA_REQUIRE(a->rotary_dim > 0 && a->rotary_dim % 2 == 0 && a->rotary_dim <= a->head_dim,
               "rotary tables exceed the head dimension");
  if (a->k_new) FA_REQUIRE(a->seqlen_new > 0, "seqlen_new must be positive when k/v are given");
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
  FA_REQUIRE(aligned16(a->q) && aligned16(a->k8) && aligned16(a->v) && aligned16(a->o), "16-byte alignment");
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
  if (int s = fwd_sm100_status()) return s;
  return bwd_sm100_status();
}

size_t fa_sizeof_args(int which) {
  switch (which) {
    case 0: return sizeof(fa_attn_args);
    case 1: return sizeof(fa_decode_args);
    case 2: return sizeof(fa_int8_args);
  }
  return 0;
}

}  // extern "C"
