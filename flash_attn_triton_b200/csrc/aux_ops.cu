// The steps either side of attention in a transformer block, as plain HBM-bound kernels:
//   rotary_kernel        rotary position embedding on (batch, seqlen, heads, headdim) or packed
//                        (tokens, heads, headdim) tensors, rotate-half or interleaved pairs,
//                        optional per-sequence position offsets, conjugate form for the backward
//   gather_rows_kernel   out[i, :] = src[idx[i], :]            (un-padding a batch)
//   scatter_rows_kernel  out[idx[i], :] (+)= src[i, :]         (re-padding; gradient of a gather)
// Each thread moves 16-byte chunks; the grids are sized to the data, there is no reuse to exploit.
#include "common.cuh"

namespace fa {

namespace {

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32(float x) { return x; }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ float from_f32(float x) { return x; }

// One thread per (row, head, pair index); fp32 arithmetic, one rounding per output element:
//   o0 = x0 cos - x1 sin,  o1 = x0 sin + x1 cos      (sin negated when conjugate)
// with (x0, x1) = (x[i], x[i + rot/2]) or, interleaved, (x[2i], x[2i+1]).  Positions past the
// table read cos = 1, sin = 0.  Columns >= rotary_dim are copied when out != x.
template <typename T>
__global__ void __launch_bounds__(256) rotary_kernel(const fa_rotary_args p) {
  const int half = p.rotary_dim >> 1;
  const int tail = p.head_dim - p.rotary_dim;          // columns that pass through
  const int per_head = half + ((p.out != p.x) ? tail : 0);
  const int64_t per_row = (int64_t)p.heads * per_head;
  const int b = blockIdx.y;
  int64_t row0 = 0;
  int len = p.seqlen;
  if (p.cu_seqlens) {
    row0 = p.cu_seqlens[b];
    len = p.cu_seqlens[b + 1] - (int)row0;
  }
  const int64_t offset = p.seqlen_offsets ? (int64_t)p.seqlen_offsets[b] : (int64_t)p.seqlen_offset;
  const T* cosb = reinterpret_cast<const T*>(p.cos);
  const T* sinb = reinterpret_cast<const T*>(p.sin);
  const int64_t total = (int64_t)len * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / per_row);
    const int rem = (int)(i - (int64_t)r * per_row);
    const int h = rem / per_head, c = rem - h * per_head;
    const T* x = reinterpret_cast<const T*>(p.x) + (p.cu_seqlens ? 0 : (int64_t)b * p.x_stride[0]) +
                 (row0 + r) * p.x_stride[1] + (int64_t)h * p.x_stride[2];
    T* o = reinterpret_cast<T*>(p.out) + (p.cu_seqlens ? 0 : (int64_t)b * p.out_stride[0]) +
           (row0 + r) * p.out_stride[1] + (int64_t)h * p.out_stride[2];
    if (c >= half) {                                    // pass-through column
      const int d = p.rotary_dim + (c - half);
      o[d] = x[d];
      continue;
    }
    const int d0 = p.interleaved ? 2 * c : c, d1 = p.interleaved ? 2 * c + 1 : c + half;
    const int64_t pos = r + offset;
    float cs = 1.f, sn = 0.f;
    if (pos >= 0 && pos < p.rotary_seqlen) {
      cs = to_f32(cosb[pos * half + c]);
      sn = to_f32(sinb[pos * half + c]);
    }
    if (p.conjugate) sn = -sn;
    const float x0 = to_f32(x[d0]), x1 = to_f32(x[d1]);
    o[d0] = from_f32<T>(x0 * cs - x1 * sn);
    o[d1] = from_f32<T>(x0 * sn + x1 * cs);
  }
}

// Rows of `row_bytes` bytes (a multiple of 16, rows 16-byte aligned) moved as uint4 chunks.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                          const int64_t* __restrict__ idx, int64_t n_idx,
                                                          int chunks, int64_t src_rows) {
  const int64_t total = n_idx * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks;
    const int c = (int)(i - r * chunks);
    const int64_t s = idx[r];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (s >= 0 && s < src_rows) v = src[s * chunks + c];   // an index outside the source reads zeros
    dst[i] = v;
  }
}

template <typename T> __device__ __forceinline__ uint4 add16(uint4 a, uint4 b);
template <> __device__ __forceinline__ uint4 add16<__half>(uint4 a, uint4 b) {
  uint4 r;
  __half2* pr = reinterpret_cast<__half2*>(&r);
  const __half2* pa = reinterpret_cast<const __half2*>(&a);
  const __half2* pb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) pr[i] = __hadd2(pa[i], pb[i]);
  return r;
}
template <> __device__ __forceinline__ uint4 add16<__nv_bfloat16>(uint4 a, uint4 b) {
  uint4 r;
  __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&r);
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) pr[i] = __hadd2(pa[i], pb[i]);
  return r;
}
template <> __device__ __forceinline__ uint4 add16<float>(uint4 a, uint4 b) {
  uint4 r;
  r.x = __float_as_uint(__uint_as_float(a.x) + __uint_as_float(b.x));
  r.y = __float_as_uint(__uint_as_float(a.y) + __uint_as_float(b.y));
  r.z = __float_as_uint(__uint_as_float(a.z) + __uint_as_float(b.z));
  r.w = __float_as_uint(__uint_as_float(a.w) + __uint_as_float(b.w));
  return r;
}

// kAcc < 0: dst[idx[r]] = src[r]; otherwise dst[idx[r]] += src[r] in the element type (the
// indices of one call are distinct, so a row has a single writer and no atomics are needed).
template <typename T, bool kAdd>
__global__ void __launch_bounds__(256) scatter_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                           const int64_t* __restrict__ idx, int64_t n_idx,
                                                           int chunks, int64_t dst_rows) {
  const int64_t total = n_idx * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks;
    const int c = (int)(i - r * chunks);
    const int64_t d = idx[r];
    if (d < 0 || d >= dst_rows) continue;                  // an index outside the destination is dropped
    uint4 v = src[i];
    if (kAdd) v = add16<T>(dst[d * chunks + c], v);
    dst[d * chunks + c] = v;
  }
}

unsigned grid_for(int64_t items, int device) {
  const int64_t blocks = (items + 255) / 256;
  const int64_t cap = (int64_t)sm_count(device) * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace

int rotary(const fa_rotary_args& a, cudaStream_t st) {
  if (a.batch == 0 || a.seqlen == 0 || a.heads == 0) return FA_OK;
  const int half = a.rotary_dim / 2;
  const int per_head = half + ((a.out != a.x) ? a.head_dim - a.rotary_dim : 0);
  if (per_head == 0) return FA_OK;
  const int64_t items = (int64_t)a.seqlen * a.heads * per_head;
  dim3 grid(grid_for(items, a.device), a.batch);
  switch (a.dtype) {
    case FA_F16: rotary_kernel<__half><<<grid, 256, 0, st>>>(a); break;
    case FA_BF16: rotary_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a); break;
    default: rotary_kernel<float><<<grid, 256, 0, st>>>(a); break;
  }
  return check_launch("rotary");
}

int gather_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                int64_t src_rows, int device, cudaStream_t st) {
  if (n_idx == 0 || row_bytes == 0) return FA_OK;
  const int chunks = (int)(row_bytes / 16);
  gather_rows_kernel<<<grid_for(n_idx * chunks, device), 256, 0, st>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), idx, n_idx, chunks, src_rows);
  return check_launch("gather_rows");
}

int scatter_rows(const void* src, void* dst, const int64_t* idx, int64_t n_idx, int64_t row_bytes,
                 int64_t dst_rows, int add_dtype, int device, cudaStream_t st) {
  if (n_idx == 0 || row_bytes == 0) return FA_OK;
  const int chunks = (int)(row_bytes / 16);
  const unsigned grid = grid_for(n_idx * chunks, device);
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  switch (add_dtype) {
    case FA_F16: scatter_rows_kernel<__half, true><<<grid, 256, 0, st>>>(s, d, idx, n_idx, chunks, dst_rows); break;
    case FA_BF16: scatter_rows_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(s, d, idx, n_idx, chunks, dst_rows); break;
    case FA_F32: scatter_rows_kernel<float, true><<<grid, 256, 0, st>>>(s, d, idx, n_idx, chunks, dst_rows); break;
    default: scatter_rows_kernel<float, false><<<grid, 256, 0, st>>>(s, d, idx, n_idx, chunks, dst_rows); break;
  }
  return check_launch("scatter_rows");
}

}  // namespace fa
