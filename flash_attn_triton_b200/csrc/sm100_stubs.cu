// Placeholders for kernel families that have no tcgen05 implementation yet: the
// dispatcher asks `*_supported` first, so these are never launched.
#include "common.cuh"
namespace fa {
#ifndef FA_HAVE_FWD_SM100
bool fwd_sm100_supported(const fa_attn_args&) { return false; }
int fwd_sm100(const fa_attn_args&, const ScoreCfg&, cudaStream_t) { set_error("not built"); return FA_ERR_UNSUPPORTED; }
int fwd_sm100_status() { return 0; }
#endif
#ifndef FA_HAVE_BWD_SM100
bool bwd_sm100_supported(const fa_attn_args&) { return false; }
int bwd_dq_sm100(const fa_attn_args&, const ScoreCfg&, cudaStream_t) { set_error("not built"); return FA_ERR_UNSUPPORTED; }
int bwd_dkdv_sm100(const fa_attn_args&, const ScoreCfg&, cudaStream_t) { set_error("not built"); return FA_ERR_UNSUPPORTED; }
int bwd_sm100_status() { return 0; }
#endif
#ifndef FA_HAVE_FWD_SM100  // the INT8 tcgen05 forward lives in fwd_sm100.cu
bool fwd_int8_sm100_supported(const fa_int8_args&) { return false; }
int fwd_int8_sm100(const fa_int8_args&, cudaStream_t) { set_error("not built"); return FA_ERR_UNSUPPORTED; }
#endif
}  // namespace fa
