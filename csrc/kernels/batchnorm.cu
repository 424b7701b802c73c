// BatchNorm over dim 1 of an NC(HW) tensor with fused residual add and ReLU.
//
// Replaces `torch::batch_norm` (flodl-sys/ops_training.cpp:1025-1046, cuDNN) plus the separate
// add and ReLU nodes of a residual block (ddp-bench/src/models/resnet.rs:209-301):
//     y = relu( (x - mean_c) * rstd_c * gamma_c + beta_c + residual )      (residual, relu optional)
// Training mode: batch statistics, biased variance for normalisation, unbiased for the running
// estimate (momentum update in place), as libtorch does. Eval mode uses the running statistics.
//
// Forward = one partial-statistics pass + one normalise pass; backward = one partial-reduction pass
// (sum dy', sum dy'*xhat with dy' = dy masked by the ReLU) + one pass writing dx and d(residual).
// Per-channel partials go to a scratch buffer of C * kSplits * 2 floats and are folded by every
// block that needs them (kSplits is small), which avoids a third launch and any atomics.
#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

constexpr int kBnSplits = 16;
constexpr int kBnThreads = 256;

// grid (C, kBnSplits): block (c, s) reduces samples n = s, s + kBnSplits, ... of channel c
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_stats_kernel(const T* __restrict__ x, float* __restrict__ partial, int N, int C, int HW) {
  __shared__ float scratch[32];
  const int c = blockIdx.x, s = blockIdx.y;
  float sum = 0.f, sq = 0.f;
  for (int n = s; n < N; n += kBnSplits) {
    const T* p = x + (static_cast<long long>(n) * C + c) * HW;
    for (int i = threadIdx.x; i < HW; i += kBnThreads) {
      const float v = VecIO<T>::get(p + i);
      sum += v;
      sq += v * v;
    }
  }
  sum = block_sum(sum, scratch);
  sq = block_sum(sq, scratch);
  if (threadIdx.x == 0) {
    partial[(c * kBnSplits + s) * 2] = sum;
    partial[(c * kBnSplits + s) * 2 + 1] = sq;
  }
}

// grid (C, kBnSplits)
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ residual, const float* __restrict__ gamma,
                const float* __restrict__ beta, const float* __restrict__ partial, float* __restrict__ running_mean,
                float* __restrict__ running_var, float* __restrict__ save_mean, float* __restrict__ save_rstd,
                T* __restrict__ y, int N, int C, int HW, float eps, float momentum, int relu, int training) {
  const int c = blockIdx.x, s = blockIdx.y;
  float mean, rstd;
  if (training) {
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < kBnSplits; ++i) {
      sum += partial[(c * kBnSplits + i) * 2];
      sq += partial[(c * kBnSplits + i) * 2 + 1];
    }
    const float cnt = static_cast<float>(N) * HW;
    mean = sum / cnt;
    const float var = fmaxf(sq / cnt - mean * mean, 0.f);
    rstd = rsqrtf(var + eps);
    if (s == 0 && threadIdx.x == 0) {
      save_mean[c] = mean;
      save_rstd[c] = rstd;
      if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean;
      if (running_var) running_var[c] = (1.f - momentum) * running_var[c] + momentum * var * (cnt / fmaxf(cnt - 1.f, 1.f));
    }
  } else {
    mean = running_mean[c];
    rstd = rsqrtf(running_var[c] + eps);
  }
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  const float scale = rstd * g, shift = b - mean * scale;
  for (int n = s; n < N; n += kBnSplits) {
    const long long off = (static_cast<long long>(n) * C + c) * HW;
    for (int i = threadIdx.x; i < HW; i += kBnThreads) {
      float v = VecIO<T>::get(x + off + i) * scale + shift;
      if (residual) v += VecIO<T>::get(residual + off + i);
      if (relu) v = fmaxf(v, 0.f);
      VecIO<T>::put(y + off + i, v);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_reduce_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y,
                     const float* __restrict__ save_mean, const float* __restrict__ save_rstd, float* __restrict__ partial,
                     int N, int C, int HW, int relu) {
  __shared__ float scratch[32];
  const int c = blockIdx.x, s = blockIdx.y;
  const float mean = save_mean[c], rstd = save_rstd[c];
  float s1 = 0.f, s2 = 0.f;
  for (int n = s; n < N; n += kBnSplits) {
    const long long off = (static_cast<long long>(n) * C + c) * HW;
    for (int i = threadIdx.x; i < HW; i += kBnThreads) {
      float g = VecIO<T>::get(dy + off + i);
      if (relu && VecIO<T>::get(y + off + i) <= 0.f) g = 0.f;
      const float xh = (VecIO<T>::get(x + off + i) - mean) * rstd;
      s1 += g;
      s2 += g * xh;
    }
  }
  s1 = block_sum(s1, scratch);
  s2 = block_sum(s2, scratch);
  if (threadIdx.x == 0) {
    partial[(c * kBnSplits + s) * 2] = s1;
    partial[(c * kBnSplits + s) * 2 + 1] = s2;
  }
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y, const float* __restrict__ gamma,
                    const float* __restrict__ save_mean, const float* __restrict__ save_rstd, const float* __restrict__ partial,
                    T* __restrict__ dx, T* __restrict__ dres, float* __restrict__ dgamma, float* __restrict__ dbeta,
                    int accumulate, int N, int C, int HW, int relu) {
  const int c = blockIdx.x, s = blockIdx.y;
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < kBnSplits; ++i) {
    s1 += partial[(c * kBnSplits + i) * 2];
    s2 += partial[(c * kBnSplits + i) * 2 + 1];
  }
  if (s == 0 && threadIdx.x == 0) {
    if (dgamma) dgamma[c] = accumulate ? dgamma[c] + s2 : s2;
    if (dbeta) dbeta[c] = accumulate ? dbeta[c] + s1 : s1;
  }
  const float cnt = static_cast<float>(N) * HW;
  const float mean = save_mean[c], rstd = save_rstd[c];
  const float g = gamma ? gamma[c] : 1.f;
  const float m1 = s1 / cnt, m2 = s2 / cnt;
  for (int n = s; n < N; n += kBnSplits) {
    const long long off = (static_cast<long long>(n) * C + c) * HW;
    for (int i = threadIdx.x; i < HW; i += kBnThreads) {
      float gy = VecIO<T>::get(dy + off + i);
      if (relu && VecIO<T>::get(y + off + i) <= 0.f) gy = 0.f;
      const float xh = (VecIO<T>::get(x + off + i) - mean) * rstd;
      VecIO<T>::put(dx + off + i, g * rstd * (gy - m1 - xh * m2));
      if (dres) VecIO<T>::put(dres + off + i, gy);
    }
  }
}

}  // namespace fb

extern "C" int fb_bn_scratch_floats(int C) { return C * fb::kBnSplits * 2; }

// scratch: fb_bn_scratch_floats(C) floats.
extern "C" int fb_bn_fwd(const void* x, const void* residual, const float* gamma, const float* beta, float* running_mean,
                         float* running_var, void* y, float* save_mean, float* save_rstd, float* scratch, int N, int C,
                         int HW, float eps, float momentum, int relu, int training, int is_bf16, void* stream) {
  using namespace fb;
  if (N <= 0 || C <= 0 || HW <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(C, kBnSplits);
  if (is_bf16) {
    using T = __nv_bfloat16;
    if (training) bn_stats_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(x), scratch, N, C, HW);
    bn_apply_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(residual), gamma, beta, scratch,
                                                    running_mean, running_var, save_mean, save_rstd, static_cast<T*>(y), N, C, HW,
                                                    eps, momentum, relu, training);
  } else {
    using T = float;
    if (training) bn_stats_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(x), scratch, N, C, HW);
    bn_apply_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(residual), gamma, beta, scratch,
                                                    running_mean, running_var, save_mean, save_rstd, static_cast<T*>(y), N, C, HW,
                                                    eps, momentum, relu, training);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_bn_bwd(const void* dy, const void* x, const void* y, const float* gamma, const float* save_mean,
                         const float* save_rstd, void* dx, void* dresidual, float* dgamma, float* dbeta, int accumulate,
                         float* scratch, int N, int C, int HW, int relu, int is_bf16, void* stream) {
  using namespace fb;
  if (N <= 0 || C <= 0 || HW <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(C, kBnSplits);
  if (is_bf16) {
    using T = __nv_bfloat16;
    bn_bwd_reduce_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(y),
                                                         save_mean, save_rstd, scratch, N, C, HW, relu);
    bn_bwd_apply_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(y),
                                                        gamma, save_mean, save_rstd, scratch, static_cast<T*>(dx),
                                                        static_cast<T*>(dresidual), dgamma, dbeta, accumulate, N, C, HW, relu);
  } else {
    using T = float;
    bn_bwd_reduce_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(y),
                                                         save_mean, save_rstd, scratch, N, C, HW, relu);
    bn_bwd_apply_kernel<T><<<grid, kBnThreads, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(y),
                                                        gamma, save_mean, save_rstd, scratch, static_cast<T*>(dx),
                                                        static_cast<T*>(dresidual), dgamma, dbeta, accumulate, N, C, HW, relu);
  }
  return static_cast<int>(cudaGetLastError());
}
