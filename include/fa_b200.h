/*
 * fa_b200.h -- C ABI of the B200 (sm_100a) attention kernels.
 *
 * The reference (luyanaa/flash-attn-triton) has no FFI: its operator boundary is the
 * Python layer that launches Triton kernels.  Each entry point below replaces one of
 * those launch sites; the citation gives the reference file:line it stands in for.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller.  The library allocates
 *     nothing and keeps no state between calls (besides a thread-local error string
 *     and one-time function-attribute set-up per device).
 *   - Strides are in ELEMENTS.  The innermost (head_dim) stride is always 1.
 *   - All work is enqueued on `stream` (a cudaStream_t passed as void*); calls return
 *     without synchronising.
 *   - Return value: 0 on success, a negative fa_status otherwise; fa_last_error() gives
 *     a message for the calling thread.
 *   - Row-wise log-sum-exp values are BASE-2 (lse2 = log2(sum exp(score))), -inf for a
 *     row with no visible key, as the reference saves them
 *     (flash_attn_triton/triton_kernel/attention_kernel.py:522-533).
 *   - Score pipeline, in this order (flash_attn_triton/flash_attn_interface.py:26-43):
 *       s = q.k * softmax_scale;  s -= slope * |qpos - kpos|;  s = softcap*tanh(s/softcap);
 *       mask (causal: kpos <= qpos; window: qpos-left <= kpos <= qpos+right) -> -inf
 *     with qpos = row + q_pos_offset (0 = upper-left alignment) and kpos = column.
 */
#ifndef FA_B200_H
#define FA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fa_status {
  FA_OK = 0,
  FA_ERR_INVALID = -1,     /* bad argument (null pointer, bad shape, bad stride)       */
  FA_ERR_UNSUPPORTED = -2, /* valid but no kernel is instantiated for it               */
  FA_ERR_LAUNCH = -3,      /* CUDA reported an error at launch                         */
  FA_ERR_WORKSPACE = -4,   /* caller's workspace is too small                          */
  FA_ERR_DEVICE_WAIT = -5  /* a bounded device-side wait ran out (kernel set its flag) */
} fa_status;

typedef enum fa_dtype { FA_F16 = 0, FA_BF16 = 1, FA_F32 = 2 /* rotary / row movers only */ } fa_dtype;

/* Kernel family selector (fa_attn_args.impl). */
typedef enum fa_impl {
  FA_IMPL_AUTO = 0,   /* tcgen05/TMA kernel when the shape has one, else the mma.sync one */
  FA_IMPL_MMA = 1,    /* warp-level mma.sync kernels (every head_dim, every feature)      */
  FA_IMPL_TCGEN05 = 2 /* tcgen05 + TMEM + TMA kernels; FA_ERR_UNSUPPORTED if none fits    */
} fa_impl;

/*
 * One argument block for dense and packed variable-length attention, forward and
 * backward.  Tensors are addressed as  base + b*stride[0] + row*stride[1] + head*stride[2] + d.
 * Dense:   q (batch, seqlen_q, heads_q, head_dim), k/v (batch, seqlen_k, heads_kv, head_dim).
 * Varlen:  cu_seqlens_* non-null; sequence b owns rows [cu[b], cu[b+1]) of the packed
 *          tensors, stride[0] is ignored, seqlen_q/seqlen_k are the MAXIMA over the batch.
 * GQA:     query head h reads kv head h / (heads_q / heads_kv)
 *          (attention_kernel.py:446, :49).
 */
typedef struct fa_attn_args {
  int32_t dtype;  /* fa_dtype */
  int32_t device; /* CUDA device ordinal that owns the pointers */
  int32_t impl;   /* fa_impl */
  int32_t batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim;
  int32_t total_q, total_k; /* packed layout only: rows of q and of k/v (= cu_seqlens[batch]) */

  const void* q;
  const void* k;
  const void* v;
  void* o; /* forward: output; backward: the forward's output (read only) */
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];

  float* lse2; /* forward: written when non-null; backward: read */
  int64_t lse_stride[3]; /* (batch, row, head); varlen ignores [0] */

  const int32_t* cu_seqlens_q; /* (batch+1) or NULL */
  const int32_t* cu_seqlens_k;

  float softmax_scale;
  float softcap;             /* 0 = off */
  const float* alibi_slopes; /* (batch, heads_q) fp32 or NULL */
  int32_t causal;
  int32_t window_left, window_right; /* -1 = unbounded */
  int32_t q_pos_offset;              /* added to the query row index; dense only */

  /* backward only */
  const void* dout;
  int64_t do_stride[3];
  float* delta; /* rowsum(o * dout), same layout as lse2 */
  void* dq;
  void* dk;
  void* dv;
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];

  /* Per-sequence length overrides of a packed batch (flash_attn_interface.py:552-581): sequence b
   * uses only its first seqused_q[b] query rows / seqused_k[b] keys.  NULL = use all.  Rows past
   * the used length are neither read nor written. */
  const int32_t* seqused_q;
  const int32_t* seqused_k;

  /* Additive score bias, fp32, element (b, h, row, col) at attn_bias[b*s0 + h*s1 + row*s2 + col*s3]
   * (a stride of 0 broadcasts); added after ALiBi, before the soft cap
   * (flash_attn_interface.py:39-40).  Dense layout only; no gradient is produced for it.  NULL = none.
   * Taken by the mma.sync kernels. */
  const float* attn_bias;
  int64_t bias_stride[4];

  /* Dropout on the probabilities with the reference's random stream (attention_kernel.py:345-358,
   * :91-93): element (row, col) is kept when philox4x32-10(key = dropout_seed, counter =
   * (row0 + row) * dropout_row_stride + col) mapped to [0, 1) exceeds dropout_p; kept
   * probabilities are scaled by 1 / (1 - p); row0 = cu_seqlens_q[b] in the packed layout, else 0.
   * The same mask for every batch entry and head, as in the reference.  0 = off.
   * Taken by the mma.sync kernels. */
  float dropout_p;
  int32_t dropout_row_stride;
  uint64_t dropout_seed;
} fa_attn_args;

/* Forward: o and (optionally) lse2.
 * Replaces _launch_dense_forward/_attn_fwd (attention_kernel.py:1057-1101, :419-533) and
 * _attention_varlen.forward/_varlen_fwd (attention_kernel.py:1284-1320, :27-104). */
int fa_fwd(const fa_attn_args* args, void* stream);

/* delta[b,h,row] = sum_d o*dout in fp32.
 * Replaces _attn_bwd_preprocess (attention_kernel.py:536-563, launched at :1127). */
int fa_bwd_preprocess(const fa_attn_args* args, void* stream);

/* dq from q,k,v,dout,lse2,delta; one writer per element, no atomics.
 * Replaces the dQ half of _attn_bwd (attention_kernel.py:677-772, :975-1054) and
 * _varlen_bwd (attention_kernel.py:107-186). */
int fa_bwd_dq(const fa_attn_args* args, void* stream);

/* dk, dv; a CTA owns a key block of one KV head and loops its query heads, so every
 * element has one writer (deterministic).
 * Replaces the dK/dV half of _attn_bwd (attention_kernel.py:567-673, :873-962) and
 * _varlen_bwd_dkdv (attention_kernel.py:188-272). */
int fa_bwd_dkdv(const fa_attn_args* args, void* stream);

/*
 * Attention probabilities as a matrix (the `return_attn_probs` surface,
 * flash_attn_interface.py:139-143, :642-659): probs[b, h, i, j] = exp2(score_log2(i, j) - lse2[i])
 * with the score pipeline, mask and dropout of `args`, for i < q_len(b), j < k_len(b); other
 * elements are left untouched (zero-fill the buffer first).  lse2 is the forward's.  When
 * lse_nat is non-NULL the natural-log LSE of row i goes to lse_nat[(b*heads_q + h)*lse_nat_stride + i].
 * probs_stride: element strides of (batch, head, row, col).
 */
int fa_attn_probs(const fa_attn_args* args, float* probs, const int64_t* probs_stride, float* lse_nat,
                  int64_t lse_nat_stride, void* stream);

/* Same three operations, but cu_seqlens_q/k are mandatory (the packed layout). */
int fa_varlen_fwd(const fa_attn_args* args, void* stream);
int fa_varlen_bwd_dq(const fa_attn_args* args, void* stream);
int fa_varlen_bwd_dkdv(const fa_attn_args* args, void* stream);

/*
 * KV-cache decode: append (optional) -> rotary (optional) -> attend, one launch chain.
 * Replaces the Python per-batch loop of flash_attn_with_kvcache
 * (flash_attn_interface.py:468-525) including _apply_rotary (:52-66), the cache append
 * (:482-492, performed IN PLACE here) and the page gather (:510-512).
 *
 * Cache layout: (num_pages, page_size, heads_kv, head_dim); a contiguous cache is the same
 * thing with page_size = capacity and block_table = NULL (sequence b uses "page"
 * cache_batch_idx[b], or b).  Token t of sequence b lives in page
 * block_table[b*block_table_stride + (t+leftpad)/page_size] at row (t+leftpad)%page_size.
 * The query rows sit at the END of the sequence: row i has position len_after-seqlen_q+i
 * (flash_attn_interface.py:517, :523).
 */
typedef struct fa_decode_args {
  int32_t dtype, device;
  int32_t batch, seqlen_q, heads_q, heads_kv, head_dim;
  const void* q;
  void* o;
  int64_t q_stride[3], o_stride[3];

  void* k_cache;
  void* v_cache;
  int64_t kc_stride[3], vc_stride[3]; /* (page, row, head) */
  int32_t page_size, num_pages;
  const int32_t* block_table; /* (batch, block_table_stride) or NULL */
  int32_t block_table_stride;
  const int32_t* cache_batch_idx; /* (batch) or NULL; contiguous cache only */
  const int32_t* cache_seqlens;   /* (batch) tokens already cached, BEFORE the append  */
  const int32_t* cache_leftpad;   /* (batch) or NULL */

  const void* k_new; /* (batch, seqlen_new, heads_kv, head_dim) or NULL */
  const void* v_new;
  int64_t kn_stride[3], vn_stride[3];
  int32_t seqlen_new;

  const void* rotary_cos; /* (rotary_seqlen, rotary_dim/2), same dtype as q; or NULL */
  const void* rotary_sin;
  int32_t rotary_dim, rotary_seqlen, rotary_interleaved;

  float softmax_scale;
  const float* alibi_slopes; /* (batch, heads_q) or NULL */
  int32_t causal, window_left, window_right;

  void* workspace; /* split-KV partials; size from fa_decode_workspace_bytes */
  size_t workspace_bytes;
  int32_t num_splits; /* 0 = choose */
} fa_decode_args;

int fa_decode_paged(const fa_decode_args* args, void* stream);

/* Bytes of workspace fa_decode_paged needs for this problem (host-only, no CUDA call). */
size_t fa_decode_workspace_bytes(const fa_decode_args* args);

/*
 * fa_decode_paged for callers that cannot allocate device memory and cannot get any from
 * their host (no counterpart in the reference).  Think of a serving loop that has frozen
 * its memory pool, a plugin running inside another runtime's callback where cudaMalloc is
 * forbidden or would synchronise the device, or a process whose whole HBM budget is already
 * spoken for by the KV cache.  The split-KV partial results go to a fixed 16 MiB array
 * inside the library image (fa_decode_static_scratch_bytes() reports the size; every GPU
 * that loads the library keeps those 16 MiB until the process exits).  args->workspace and
 * args->workspace_bytes are ignored; q, o, the caches and every other buffer are still the
 * caller's.  The call makes no cudaMalloc/cudaFree and calls no allocating library routine.
 *
 *  - A problem whose partials exceed the array (fa_decode_workspace_bytes(args) >
 *    fa_decode_static_scratch_bytes()) is refused with FA_ERR_WORKSPACE and a message;
 *    a smaller args->num_splits shrinks the need.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
 *    outside any stream capture.
 *  - All calls on one GPU share the array and it keeps whatever the last call left.  Nothing
 *    in it has to start at zero (each call writes every partial it later reads), but two
 *    calls that overlap on the GPU -- different streams, or different host threads --
 *    overwrite each other's partials: serialise them.
 */
int fa_decode_paged_static(const fa_decode_args* args, void* stream);
size_t fa_decode_static_scratch_bytes(void);

/*
 * Per-key-token INT8 quantisation: k (rows, head_dim) fp16 contiguous ->
 * k8 (rows, head_dim) int8, s_k (rows) fp32, with
 *   s = max(absmax, 1)/127;  code = round_half_away(k * (1/s))  in IEEE fp32,
 * bit-exact with _quantize_k_rows (attention_kernel_int8.py:58-79, :27-30).
 */
int fa_quantize_k_int8(const void* k, int8_t* k8, float* s_k, int64_t rows, int32_t head_dim,
                       int32_t device, void* stream);

/*
 * INT8-QK^T forward on contiguous (batch, heads, seqlen, head_dim) fp16 tensors:
 * q is quantised per row in-kernel, k8/s_k come from fa_quantize_k_int8, P@V stays fp16.
 * Replaces _attn_fwd_int8 (attention_kernel_int8.py:167-217, launched at :237).
 */
typedef struct fa_int8_args {
  int32_t device, impl;
  int32_t batch, heads, seqlen, head_dim;
  const void* q;    /* fp16 */
  const int8_t* k8; /* (batch*heads, seqlen, head_dim) */
  const float* s_k; /* (batch*heads, seqlen) */
  const void* v;    /* fp16 */
  void* o;          /* fp16 */
  float* lse2;      /* (batch, heads, seqlen) or NULL */
  float softmax_scale;
  int32_t causal;
  /* Scratch for the tcgen05 kernel, which stages the query codes with TMA: int8
   * (batch*heads, seqlen, head_dim) and fp32 (batch*heads, seqlen).  When either is NULL the
   * mma.sync kernel (which quantises q in shared memory) is used. */
  int8_t* q8_scratch;
  float* sq_scratch;
  /* Padded calls (attention_kernel_int8.py:108-118, :245): keys at or past seqlen_k_valid are
   * masked (0 = all seqlen keys are valid), and query row i sits at position i + q_pos_offset for
   * the causal mask (the reference passes SEQ_LEN_K - SEQ_LEN_Q). */
  int32_t seqlen_k_valid;
  int32_t q_pos_offset;
} fa_int8_args;

int fa_fwd_int8(const fa_int8_args* args, void* stream);

/*
 * Rotary position embedding on x (batch, seqlen, heads, head_dim) -- or packed (tokens, heads,
 * head_dim) with cu_seqlens -- into out (same layout; out == x rotates in place):
 *   non-interleaved: pairs (x[i], x[i + rotary_dim/2]);  interleaved: pairs (x[2i], x[2i+1])
 *   o0 = x0 cos - x1 sin,  o1 = x0 sin + x1 cos   in fp32, rounded once;  conjugate negates sin
 * Row r of sequence b uses table row r + seqlen_offsets[b] (or + seqlen_offset); rows past the
 * table read cos = 1, sin = 0; columns >= rotary_dim are copied.  cos/sin have x's dtype.
 * Replaces rotary_kernel / apply_rotary (flash_attn/ops/triton/rotary.py:11-130, :133-234).
 */
typedef struct fa_rotary_args {
  int32_t dtype, device; /* fa_dtype incl. FA_F32 */
  int32_t batch, seqlen, heads, head_dim; /* seqlen = the longest sequence when packed */
  const void* x;
  void* out;
  int64_t x_stride[3], out_stride[3]; /* (batch, row, head) in elements; packed ignores [0] */
  const void* cos; /* (rotary_seqlen, rotary_dim/2) contiguous */
  const void* sin;
  int32_t rotary_dim, rotary_seqlen;
  int32_t interleaved, conjugate;
  int32_t seqlen_offset;          /* used when seqlen_offsets is NULL */
  const int32_t* seqlen_offsets;  /* (batch) or NULL */
  const int32_t* cu_seqlens;      /* (batch+1) or NULL */
} fa_rotary_args;

int fa_rotary(const fa_rotary_args* args, void* stream);

/*
 * Row movers for un-padding / re-padding a batch.  Rows are row_bytes long (a multiple of 16),
 * src/dst 16-byte aligned, idx int64 on the device.
 *   fa_gather_rows:   dst[i] = src[idx[i]]            (an index outside [0, src_rows) yields zeros)
 *   fa_scatter_rows:  dst[idx[i]] = src[i], or += in element type add_dtype (fa_dtype; -1 = plain
 *                     store).  Indices of one call must be distinct; one outside [0, dst_rows) is
 *                     dropped.  Rows of dst that no index names keep their contents.
 * Replace IndexFirstAxis / IndexPutFirstAxis / IndexFirstAxisResidual
 * (flash_attn/bert_padding.py:8-96).
 */
int fa_gather_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                   int64_t src_rows, int32_t device, void* stream);
int fa_scatter_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                    int64_t dst_rows, int32_t add_dtype, int32_t device, void* stream);

/* Host-only helpers. */
const char* fa_version(void);
const char* fa_last_error(void);
/* 1 when fa_fwd with FA_IMPL_AUTO would pick the tcgen05 kernel for these arguments. */
int fa_fwd_uses_tcgen05(const fa_attn_args* args);
/*
 * Time-outs of bounded device-side waits.  Every wait inside the tcgen05 kernels gives up after
 * about a second; the kernel that gave up raises a status word (device memory, and a mirror in
 * mapped host memory), releases its tensor memory and returns early, leaving its outputs
 * incomplete.  From then on
 *   - every tcgen05 launch on that device returns at its first wait, and
 *   - fa_fwd / fa_bwd_* / fa_varlen_* / fa_fwd_int8 return FA_ERR_DEVICE_WAIT instead of launching
 *     a tcgen05 kernel, as soon as the host mirror shows the code (no synchronisation needed),
 * until fa_device_wait_clear() is called.
 *
 * fa_device_wait_status: 0, or the code of the wait that ran out.  Synchronises the device.
 * fa_device_wait_clear:  synchronises, then puts the words of `device` back to zero.
 * fa_wait_probe:         launches ONE warp that waits, for at most `clocks` cycles, on a barrier
 *                        nothing ever arrives at (no copy or MMA in flight): exercises the
 *                        time-out path for bring-up and tests.  Leaves the status set (code 99).
 * fa_debug_set_wait_status: writes the host mirror only (host-side tests of the refusal).
 */
int fa_device_wait_status(int device);
int fa_device_wait_clear(int device);
int fa_wait_probe(int32_t device, int64_t clocks, void* stream);
int fa_debug_set_wait_status(int32_t device, int32_t code);
/* Measurement aid: one CTA per SM issues `iters` back-to-back tcgen05.mma (M128 N128; K16 with fp16
 * operands for kind 0, K32 with int8 operands for kind 1) from shared memory into tensor memory.
 * Timed by the caller, it gives the tensor-pipe rate this library's own issue path reaches
 * (2*128*128*K*iters*SMs FLOP per launch): the int8 denominator for the INT8 forward. */
int fa_mma_peak_probe(int32_t device, int32_t kind, int32_t iters, void* stream);
/* sizeof of an argument block as this library was compiled: 0 = fa_attn_args,
 * 1 = fa_decode_args, 2 = fa_int8_args.  Lets a foreign-language binding check its
 * struct layout before the first call.  3 = fa_rotary_args. */
size_t fa_sizeof_args(int which);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H */
