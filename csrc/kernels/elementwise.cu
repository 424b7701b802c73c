// Vectorised elementwise kernels: GELU (erf / tanh) forward and backward, dropout, bias-gradient
// column sums and dtype casts.
//
// GELU replaces `torch::gelu` (flodl-sys/ops_tensor.cpp:329-345) where it is not already folded
// into a GEMM epilogue; the column sum replaces the bias-gradient reduction libtorch's autograd
// runs for `torch::linear`.
#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

__device__ __forceinline__ float gelu_fwd_f(float x, int tanh_approx) {
  if (tanh_approx) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
  }
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}
__device__ __forceinline__ float gelu_bwd_f(float x, int tanh_approx) {
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
  constexpr int V = VecIO<T>::kVec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * V;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    if (i + V <= n) {
      float v[V];
      VecIO<T>::load(x + i, v);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = gelu_fwd_f(v[j], tanh_approx);
      VecIO<T>::store(y + i, v);
    } else {
      for (long long k = i; k < n; ++k) VecIO<T>::put(y + k, gelu_fwd_f(VecIO<T>::get(x + k), tanh_approx));
    }
  }
}

template <typename T>
__global__ void gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                                long long n, int tanh_approx) {
  constexpr int V = VecIO<T>::kVec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * V;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    if (i + V <= n) {
      float a[V], b[V];
      VecIO<T>::load(dy + i, a);
      VecIO<T>::load(x + i, b);
#pragma unroll
      for (int j = 0; j < V; ++j) a[j] *= gelu_bwd_f(b[j], tanh_approx);
      VecIO<T>::store(dx + i, a);
    } else {
      for (long long k = i; k < n; ++k)
        VecIO<T>::put(dx + k, VecIO<T>::get(dy + k) * gelu_bwd_f(VecIO<T>::get(x + k), tanh_approx));
    }
  }
}

// y = x * mask(seed, idx) / (1 - p); used for forward and (with dy as x) for backward.
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p,
                               unsigned long long seed_in, const unsigned long long* __restrict__ seed_dev) {
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
                              long long ld, int rows_per_block) {
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

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y, long long n, float scale) {
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
    fb::gelu_fwd_kernel<__nv_bfloat16><<<fb::grid_for(n, 8, 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, tanh_approx);
  else
    fb::gelu_fwd_kernel<float><<<fb::grid_for(n, 4, 256), 256, 0, st>>>(static_cast<const float*>(x),
                                                                        static_cast<float*>(y), n, tanh_approx);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int tanh_approx, int is_bf16,
                           void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::gelu_bwd_kernel<__nv_bfloat16><<<fb::grid_for(n, 8, 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
        static_cast<__nv_bfloat16*>(dx), n, tanh_approx);
  else
    fb::gelu_bwd_kernel<float><<<fb::grid_for(n, 4, 256), 256, 0, st>>>(
        static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<float*>(dx), n, tanh_approx);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_dropout(const void* x, void* y, long long n, float p, unsigned long long seed,
                          const unsigned long long* seed_dev, int is_bf16, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::dropout_kernel<__nv_bfloat16><<<fb::grid_for(n, 8, 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, p, seed, seed_dev);
  else
    fb::dropout_kernel<float><<<fb::grid_for(n, 4, 256), 256, 0, st>>>(static_cast<const float*>(x),
                                                                       static_cast<float*>(y), n, p, seed, seed_dev);
  return static_cast<int>(cudaGetLastError());
}

// `out` (fp32, `cols` long) is added to: zero it first for a plain column sum.
extern "C" int fb_colsum(const void* x, float* out, int rows, int cols, long long ld, int is_bf16, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rpb = 256;
  dim3 grid((cols + 31) / 32, (rows + rpb - 1) / rpb);
  dim3 block(32, 32);
  if (is_bf16)
    fb::colsum_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(x), out, rows, cols, ld, rpb);
  else
    fb::colsum_kernel<float><<<grid, block, 0, st>>>(static_cast<const float*>(x), out, rows, cols, ld, rpb);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_cast(const void* x, void* y, long long n, float scale, int in_bf16, int out_bf16, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = fb::grid_for(n, 4, 256);
  if (in_bf16 && !out_bf16)
    fb::cast_kernel<__nv_bfloat16, float><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<float*>(y), n, scale);
  else if (!in_bf16 && out_bf16)
    fb::cast_kernel<float, __nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const float*>(x), static_cast<__nv_bfloat16*>(y), n, scale);
  else if (in_bf16)
    fb::cast_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, scale);
  else
    fb::cast_kernel<float, float><<<g, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), n, scale);
  return static_cast<int>(cudaGetLastError());
}
