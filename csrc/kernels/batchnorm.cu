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
//
// Work split: block (c, s) owns the samples n = s, s + kSplits, ... of channel c. Their HW-element
// rows are walked as ONE flattened index space in 16-byte vectors, so all 256 threads stay busy
// for 8x8 feature maps as well as 32x32 ones (a per-row loop leaves 3/4 of the block idle at HW = 64).
#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

constexpr int kBnSplits = 16;
constexpr int kBnThreads = 256;

// Calls f(offset, count) for this block's elements: `count` consecutive elements (V when the
// vector path applies, else 1) starting at `offset` from the tensor base.
template <int V, typename F>
__device__ __forceinline__ void bn_for_each(int N, int C, int HW, int c, int s, F f) {
  const int rows = (N - s + kBnSplits - 1) / kBnSplits;     // samples owned by this block
  if (rows <= 0) return;
  if (HW % V == 0) {
    const int per_row = HW / V;
    const int total = rows * per_row;
    for (int q = threadIdx.x; q < total; q += kBnThreads) {
      const int r = q / per_row;
      const int i = (q - r * per_row) * V;
      const long long off = (static_cast<long long>(s + r * kBnSplits) * C + c) * HW + i;
      f(off, true);
    }
  } else {
    const long long total = static_cast<long long>(rows) * HW;
    for (long long q = threadIdx.x; q < total; q += kBnThreads) {
      const int r = static_cast<int>(q / HW);
      const int i = static_cast<int>(q - static_cast<long long>(r) * HW);
      const long long off = (static_cast<long long>(s + r * kBnSplits) * C + c) * HW + i;
      f(off, false);
    }
  }
}

template <typename T>
__device__ __forceinline__ bool bn_aligned(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// grid (C, kBnSplits)
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_stats_kernel(const T* __restrict__ x, float* __restrict__ partial, int N, int C, int HW) {
  constexpr int V = VecIO<T>::kVec;
  __shared__ float scratch[32];
  const int c = blockIdx.x, s = blockIdx.y;
  float sum = 0.f, sq = 0.f;
  const bool vec_ok = bn_aligned<T>(x);
  if (vec_ok) {
    bn_for_each<V>(N, C, HW, c, s, [&](long long off, bool vec) {
      if (vec) {
        float v[V];
        VecIO<T>::load(x + off, v);
#pragma unroll
        for (int j = 0; j < V; ++j) { sum += v[j]; sq += v[j] * v[j]; }
      } else {
        const float v = VecIO<T>::get(x + off);
        sum += v; sq += v * v;
      }
    });
  } else {
    bn_for_each<1>(N, C, HW, c, s, [&](long long off, bool) {
      const float v = VecIO<T>::get(x + off);
      sum += v; sq += v * v;
    });
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
  constexpr int V = VecIO<T>::kVec;
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
  const bool vec_ok = bn_aligned<T>(x) && bn_aligned<T>(y) && (!residual || bn_aligned<T>(residual));
  auto one = [&](long long off) {
    float v = VecIO<T>::get(x + off) * scale + shift;
    if (residual) v += VecIO<T>::get(residual + off);
    if (relu) v = fmaxf(v, 0.f);
    VecIO<T>::put(y + off, v);
  };
  if (vec_ok) {
    bn_for_each<V>(N, C, HW, c, s, [&](long long off, bool vec) {
      if (!vec) { one(off); return; }
      float v[V], r[V];
      VecIO<T>::load(x + off, v);
      if (residual) VecIO<T>::load(residual + off, r);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float o = fmaf(v[j], scale, shift);
        if (residual) o += r[j];
        v[j] = relu ? fmaxf(o, 0.f) : o;
      }
      VecIO<T>::store(y + off, v);
    });
  } else {
    bn_for_each<1>(N, C, HW, c, s, [&](long long off, bool) { one(off); });
  }
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_reduce_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y,
                     const float* __restrict__ save_mean, const float* __restrict__ save_rstd, float* __restrict__ partial,
                     int N, int C, int HW, int relu) {
  constexpr int V = VecIO<T>::kVec;
  __shared__ float scratch[32];
  const int c = blockIdx.x, s = blockIdx.y;
  const float mean = save_mean[c], rstd = save_rstd[c];
  float s1 = 0.f, s2 = 0.f;
  const bool vec_ok = bn_aligned<T>(dy) && bn_aligned<T>(x) && bn_aligned<T>(y);
  auto one = [&](long long off) {
    float g = VecIO<T>::get(dy + off);
    if (relu && VecIO<T>::get(y + off) <= 0.f) g = 0.f;
    s1 += g;
    s2 += g * (VecIO<T>::get(x + off) - mean) * rstd;
  };
  if (vec_ok) {
    bn_for_each<V>(N, C, HW, c, s, [&](long long off, bool vec) {
      if (!vec) { one(off); return; }
      float g[V], xv[V], yv[V];
      VecIO<T>::load(dy + off, g);
      VecIO<T>::load(x + off, xv);
      if (relu) VecIO<T>::load(y + off, yv);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float gj = (relu && yv[j] <= 0.f) ? 0.f : g[j];
        s1 += gj;
        s2 += gj * (xv[j] - mean) * rstd;
      }
    });
  } else {
    bn_for_each<1>(N, C, HW, c, s, [&](long long off, bool) { one(off); });
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
  constexpr int V = VecIO<T>::kVec;
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
  const float k = g * rstd;
  const bool vec_ok = bn_aligned<T>(dy) && bn_aligned<T>(x) && bn_aligned<T>(y) && bn_aligned<T>(dx) && (!dres || bn_aligned<T>(dres));
  auto one = [&](long long off) {
    float gy = VecIO<T>::get(dy + off);
    if (relu && VecIO<T>::get(y + off) <= 0.f) gy = 0.f;
    const float xh = (VecIO<T>::get(x + off) - mean) * rstd;
    VecIO<T>::put(dx + off, k * (gy - m1 - xh * m2));
    if (dres) VecIO<T>::put(dres + off, gy);
  };
  if (vec_ok) {
    bn_for_each<V>(N, C, HW, c, s, [&](long long off, bool vec) {
      if (!vec) { one(off); return; }
      float gy[V], xv[V], yv[V];
      VecIO<T>::load(dy + off, gy);
      VecIO<T>::load(x + off, xv);
      if (relu) VecIO<T>::load(y + off, yv);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        if (relu && yv[j] <= 0.f) gy[j] = 0.f;
        xv[j] = k * (gy[j] - m1 - (xv[j] - mean) * rstd * m2);
      }
      VecIO<T>::store(dx + off, xv);
      if (dres) VecIO<T>::store(dres + off, gy);
    });
  } else {
    bn_for_each<1>(N, C, HW, c, s, [&](long long off, bool) { one(off); });
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
