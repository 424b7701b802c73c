// Vectorised elementwise kernels: GELU (erf / tanh) forward and backward, dropout, bias-gradient
// column sums and dtype casts.
//
// GELU replaces `torch::gelu` (flodl-sys/ops_tensor.cpp:329-345) where it is not already folded
// into a GEMM epilogue; the column sum replaces the bias-gradient reduction libtorch's autograd
// runs for `torch::linear`.
#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

// `kFast` (bf16 tensors): the one-MUFU formulas of common.cuh, whose error is below bf16 resolution;
// fp32 tensors keep libdevice's erff / tanhf.
template <bool kFast>
__device__ __forceinline__ float gelu_fwd_f(float x, int tanh_approx) {
  if (kFast) return tanh_approx ? gelu_tanh_fast(x) : gelu_erf_fast(x);
  if (tanh_approx) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
  }
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}
template <bool kFast>
__device__ __forceinline__ float gelu_bwd_f(float x, int tanh_approx) {
  if (kFast) return tanh_approx ? dgelu_tanh_fast(x) : dgelu_erf_fast(x);
  if (tanh_approx) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float t = tanhf(u);
    const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
  }
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}

template <typename T>
__global__ void gelu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, int tanh_approx) {
  pdl_entry();
  constexpr int V = VecIO<T>::kVec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * V;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    if (i + V <= n) {
      float v[V];
      VecIO<T>::load(x + i, v);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = gelu_fwd_f<sizeof(T) == 2>(v[j], tanh_approx);
      VecIO<T>::store(y + i, v);
    } else {
      for (long long k = i; k < n; ++k) VecIO<T>::put(y + k, gelu_fwd_f<sizeof(T) == 2>(VecIO<T>::get(x + k), tanh_approx));
    }
  }
}

template <typename T>
__global__ void gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                                long long n, int tanh_approx) {
  pdl_entry();
  constexpr int V = VecIO<T>::kVec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * V;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    if (i + V <= n) {
      float a[V], b[V];
      VecIO<T>::load(dy + i, a);
      VecIO<T>::load(x + i, b);
#pragma unroll
      for (int j = 0; j < V; ++j) a[j] *= gelu_bwd_f<sizeof(T) == 2>(b[j], tanh_approx);
      VecIO<T>::store(dx + i, a);
    } else {
      for (long long k = i; k < n; ++k)
        VecIO<T>::put(dx + k, VecIO<T>::get(dy + k) * gelu_bwd_f<sizeof(T) == 2>(VecIO<T>::get(x + k), tanh_approx));
    }
  }
}

// y = x * mask(seed, idx) / (1 - p); used for forward and (with dy as x) for backward.
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p,
                               unsigned long long seed_in, const unsigned long long* __restrict__ seed_dev) {
  pdl_entry();
  constexpr int V = VecIO<T>::kVec;
  const unsigned long long seed = seed_in + (seed_dev ? *seed_dev : 0ull);
  const float inv_keep = 1.f / (1.f - p);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * V;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    if (i + V <= n) {
      float v[V];
      VecIO<T>::load(x + i, v);
#pragma unroll
      for (int j = 0; j < V; j += 4) {
        float s[4];
        dropout_scale4(seed, static_cast<uint64_t>(i + j), p, inv_keep, s);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[j + k] *= s[k];
      }
      VecIO<T>::store(y + i, v);
    } else {
      for (long long k = i; k < n; ++k)
        VecIO<T>::put(y + k, VecIO<T>::get(x + k) * dropout_scale(seed, static_cast<uint64_t>(k), p, inv_keep));
    }
  }
}

// out[c] (+)= sum_r x[r][c]; a 32x32 tile per block so reads stay coalesced.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ out, int rows, int cols,
                              long long ld, int rows_per_block, const int* __restrict__ rows_dyn) {
  pdl_entry();
  if (rows_dyn) rows = min(rows, *rows_dyn);
  __shared__ float tile[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float acc = 0.f;
  if (c < cols)
    for (int r = r0 + threadIdx.y; r < r1; r += blockDim.y) acc += VecIO<T>::get(x + static_cast<long long>(r) * ld + c);
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) s += (i < blockDim.y) ? tile[i][threadIdx.x] : 0.f;
    atomicAdd(out + c, s);
  }
}

// Vectorised form: a lane owns V consecutive columns (16 bytes), a warp 32*V columns, the 8 warps of
// a block different rows; partials meet in shared memory, one atomicAdd per column per block.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const T* __restrict__ x, float* __restrict__ out, int rows, int cols, long long ld, int rows_per_block,
                  const int* __restrict__ rows_dyn) {
  pdl_entry();
  if (rows_dyn) rows = min(rows, *rows_dyn);
  constexpr int V = VecIO<T>::kVec;
  __shared__ float red[8][32 * V + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + lane) * V;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  if (c0 + V <= cols) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float v[V];
      VecIO<T>::load(x + static_cast<long long>(r) * ld + c0, v);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += v[j];
    }
  } else if (c0 < cols) {   // ragged last vector of the row
    for (int r = r0 + warp; r < r1; r += 8) {
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (c0 + j < cols) acc[j] += VecIO<T>::get(x + static_cast<long long>(r) * ld + c0 + j);
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) red[warp][lane * V + j] = acc[j];
  __syncthreads();
  for (int c = threadIdx.x; c < 32 * V; c += blockDim.x) {
    const int col = blockIdx.x * 32 * V + c;
    if (col < cols) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w][c];
      atomicAdd(out + col, s);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Row compaction for losses that ignore most rows (masked-LM: ~15 % of the positions carry a label).
// The vocabulary projection, the softmax and their backward GEMMs then run on the active rows only;
// ignored rows contribute neither loss nor gradient, so the result is the same as for the full matrix.
// Counts stay on the device, buffers keep their full static size: the sequence is graph-capturable.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
compact_targets_kernel(const long long* __restrict__ targets, int rows, long long ignore_index, int* __restrict__ idx,
                       long long* __restrict__ targets_c, int* __restrict__ counts) {
  pdl_entry();
  __shared__ int warp_tot[32];
  __shared__ int base_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base_sh = 0;
  __syncthreads();
  for (int r0 = 0; r0 < rows; r0 += 1024) {
    const int r = r0 + threadIdx.x;
    const long long t = (r < rows) ? targets[r] : ignore_index;
    const bool act = (r < rows) && t != ignore_index;
    const unsigned m = __ballot_sync(0xffffffffu, act);
    const int before = __popc(m & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int woff = 0, tot = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = warp_tot[w];
      if (w < warp) woff += c;
      tot += c;
    }
    const int base = base_sh;
    if (act) {
      const int o = base + woff + before;
      idx[o] = r;
      targets_c[o] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) base_sh = base + tot;
    __syncthreads();
  }
  const int n = base_sh;
  int n_pad = (n + 255) / 256 * 256;
  if (n_pad > rows) n_pad = rows;
  for (int i = n + threadIdx.x; i < rows; i += 1024) {   // the tail: no row, no label
    idx[i] = 0;
    targets_c[i] = ignore_index;
  }
  if (threadIdx.x == 0) {
    counts[0] = n;
    counts[1] = n_pad;
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
gather_rows_kernel(const T* __restrict__ x, long long ld, const int* __restrict__ idx, const int* __restrict__ counts,
                   T* __restrict__ xc, long long ldc, int cols) {
  pdl_entry();
  const int i = blockIdx.x;
  const int n = counts[0], n_pad = counts[1];
  if (i >= n_pad) return;
  constexpr int V = VecIO<T>::kVec;
  T* dst = xc + static_cast<long long>(i) * ldc;
  const int rows_total = static_cast<int>(gridDim.x);
  if (!FB_INDEX_OK(n, rows_total + 1, 102) || !FB_INDEX_OK(n_pad, rows_total + 1, 103)) return;
  if (i < n && !FB_INDEX_OK(idx[i], rows_total, 104)) return;
  const T* src = x + static_cast<long long>(i < n ? idx[i] : 0) * ld;
  const bool vec = (cols % V == 0) && (ld % V == 0) && (ldc % V == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(xc) & 15) == 0);
  if (vec) {
    for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (i < n) v = *reinterpret_cast<const uint4*>(src + c);
      *reinterpret_cast<uint4*>(dst + c) = v;
    }
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) VecIO<T>::put(dst + c, i < n ? VecIO<T>::get(src + c) : 0.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
scatter_rows_kernel(const T* __restrict__ dxc, long long ldc, const int* __restrict__ idx, const int* __restrict__ counts,
                    T* __restrict__ dx, long long ld, int cols) {
  pdl_entry();
  const int i = blockIdx.x;
  if (i >= counts[0]) return;
  if (!FB_INDEX_OK(counts[0], static_cast<long long>(gridDim.x) + 1, 105) || !FB_INDEX_OK(idx[i], gridDim.x, 106)) return;
  constexpr int V = VecIO<T>::kVec;
  const T* src = dxc + static_cast<long long>(i) * ldc;
  T* dst = dx + static_cast<long long>(idx[i]) * ld;
  const bool vec = (cols % V == 0) && (ld % V == 0) && (ldc % V == 0) && ((reinterpret_cast<uintptr_t>(dx) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(dxc) & 15) == 0);
  if (vec) {
    for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) VecIO<T>::put(dst + c, VecIO<T>::get(src + c));
  }
}

// dW[ids[t]][:] += dy[t][:] for an embedding table (fp32 accumulation, rows equal to padding_idx skipped).
template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dy, const long long* __restrict__ ids, float* __restrict__ dw,
                                     long long tokens, int dim, long long vocab, long long padding_idx) {
  pdl_entry();
  const long long t = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const long long id = ids[t];
  if (id == padding_idx) return;
  if (!FB_INDEX_OK(id, vocab, 101) || id < 0 || id >= vocab) return;
  const T* src = dy + t * dim;
  float* dst = dw + id * dim;
  for (int c = threadIdx.x & 31; c < dim; c += 32) atomicAdd(dst + c, VecIO<T>::get(src + c));
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y, long long n, float scale) {
  pdl_entry();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    VecIO<TO>::put(y + i, VecIO<TI>::get(x + i) * scale);
}

static inline int grid_for(long long n, int per_thread, int block) {
  long long g = (n + static_cast<long long>(per_thread) * block - 1) / (static_cast<long long>(per_thread) * block);
  if (g > 148 * 16) g = 148 * 16;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace fb

extern "C" int fb_gelu_fwd(const void* x, void* y, long long n, int tanh_approx, int is_bf16, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::launch_pdl(fb::gelu_fwd_kernel<__nv_bfloat16>, dim3(fb::grid_for(n, 8, 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, tanh_approx);
  else
    fb::launch_pdl(fb::gelu_fwd_kernel<float>, dim3(fb::grid_for(n, 4, 256)), dim3(256), 0, st, static_cast<const float*>(x),
                                                                        static_cast<float*>(y), n, tanh_approx);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int tanh_approx, int is_bf16,
                           void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::launch_pdl(fb::gelu_bwd_kernel<__nv_bfloat16>, dim3(fb::grid_for(n, 8, 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
        static_cast<__nv_bfloat16*>(dx), n, tanh_approx);
  else
    fb::launch_pdl(fb::gelu_bwd_kernel<float>, dim3(fb::grid_for(n, 4, 256)), dim3(256), 0, st, static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<float*>(dx), n, tanh_approx);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_dropout(const void* x, void* y, long long n, float p, unsigned long long seed,
                          const unsigned long long* seed_dev, int is_bf16, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::launch_pdl(fb::dropout_kernel<__nv_bfloat16>, dim3(fb::grid_for(n, 8, 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, p, seed, seed_dev);
  else
    fb::launch_pdl(fb::dropout_kernel<float>, dim3(fb::grid_for(n, 4, 256)), dim3(256), 0, st, static_cast<const float*>(x),
                                                                       static_cast<float*>(y), n, p, seed, seed_dev);
  return static_cast<int>(cudaGetLastError());
}

// `out` (fp32, `cols` long) is added to: zero it first for a plain column sum.
extern "C" int fb_colsum(const void* x, float* out, int rows, int cols, long long ld, int is_bf16, void* stream) {
  return fb_colsum_dyn(x, out, rows, cols, ld, is_bf16, nullptr, stream);
}

extern "C" int fb_colsum_dyn(const void* x, float* out, int rows, int cols, long long ld, int is_bf16, const int* rows_dyn,
                             void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vec = is_bf16 ? 8 : 4;
  if (ld % vec == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int rpbv = 64;
    dim3 gridv((cols + 32 * vec - 1) / (32 * vec), (rows + rpbv - 1) / rpbv);
    if (is_bf16)
      fb::launch_pdl(fb::colsum_vec_kernel<__nv_bfloat16>, dim3(gridv), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), out, rows, cols, ld, rpbv, rows_dyn);
    else
      fb::launch_pdl(fb::colsum_vec_kernel<float>, dim3(gridv), dim3(256), 0, st, static_cast<const float*>(x), out, rows, cols, ld, rpbv, rows_dyn);
    return static_cast<int>(cudaGetLastError());
  }
  int rpb = 256;
  dim3 grid((cols + 31) / 32, (rows + rpb - 1) / rpb);
  dim3 block(32, 32);
  if (is_bf16)
    fb::launch_pdl(fb::colsum_kernel<__nv_bfloat16>, dim3(grid), dim3(block), 0, st, static_cast<const __nv_bfloat16*>(x), out, rows, cols, ld, rpb, rows_dyn);
  else
    fb::launch_pdl(fb::colsum_kernel<float>, dim3(grid), dim3(block), 0, st, static_cast<const float*>(x), out, rows, cols, ld, rpb, rows_dyn);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_cast(const void* x, void* y, long long n, float scale, int in_bf16, int out_bf16, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = fb::grid_for(n, 4, 256);
  if (in_bf16 && !out_bf16)
    fb::launch_pdl(fb::cast_kernel<__nv_bfloat16, float>, dim3(g), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<float*>(y), n, scale);
  else if (!in_bf16 && out_bf16)
    fb::launch_pdl(fb::cast_kernel<float, __nv_bfloat16>, dim3(g), dim3(256), 0, st, static_cast<const float*>(x), static_cast<__nv_bfloat16*>(y), n, scale);
  else if (in_bf16)
    fb::launch_pdl(fb::cast_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(g), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, scale);
  else
    fb::launch_pdl(fb::cast_kernel<float, float>, dim3(g), dim3(256), 0, st, static_cast<const float*>(x), static_cast<float*>(y), n, scale);
  return static_cast<int>(cudaGetLastError());
}

// dw (fp32 [vocab, dim]) += scatter of dy ([tokens, dim]) by ids; padding_idx < 0 disables the skip.
extern "C" int fb_embedding_bwd(const void* dy, const long long* ids, float* dw, long long tokens, int dim, long long vocab,
                                long long padding_idx, int is_bf16, void* stream) {
  if (tokens <= 0 || dim <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int warps = 8;
  const long long grid = (tokens + warps - 1) / warps;
  if (is_bf16)
    fb::launch_pdl(fb::embedding_bwd_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), 0, st, static_cast<const __nv_bfloat16*>(dy), ids, dw, tokens, dim, vocab, padding_idx);
  else
    fb::launch_pdl(fb::embedding_bwd_kernel<float>, dim3(static_cast<unsigned>(grid)), dim3(warps * 32), 0, st, static_cast<const float*>(dy), ids, dw,
                                                                                        tokens, dim, vocab, padding_idx);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_compact_targets(const long long* targets, int rows, long long ignore_index, int* idx, long long* targets_c,
                                  int* counts, void* stream) {
  if (rows <= 0) return 0;
  fb::launch_pdl(fb::compact_targets_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), targets, rows, ignore_index, idx, targets_c, counts);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gather_rows(const void* x, long long ld, const int* idx, const int* counts, void* xc, long long ldc, int rows,
                              int cols, int is_bf16, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::launch_pdl(fb::gather_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(x), ld, idx, counts,
                                                                static_cast<__nv_bfloat16*>(xc), ldc, cols);
  else
    fb::launch_pdl(fb::gather_rows_kernel<float>, dim3(rows), dim3(128), 0, st, static_cast<const float*>(x), ld, idx, counts, static_cast<float*>(xc), ldc, cols);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_scatter_rows(const void* dxc, long long ldc, const int* idx, const int* counts, void* dx, long long ld, int rows,
                               int cols, int is_bf16, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::launch_pdl(fb::scatter_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(dxc), ldc, idx, counts,
                                                                 static_cast<__nv_bfloat16*>(dx), ld, cols);
  else
    fb::launch_pdl(fb::scatter_rows_kernel<float>, dim3(rows), dim3(128), 0, st, static_cast<const float*>(dxc), ldc, idx, counts, static_cast<float*>(dx), ld, cols);
  return static_cast<int>(cudaGetLastError());
}

FB_BOUNDS_ATTACH(elementwise)
