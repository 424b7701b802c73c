// Fused LayerNorm forward / backward, one warp per row, the row held in registers.
//
// Replaces `at::native_layer_norm` (flodl-sys/ops_tensor.cpp:442-460) and, for the encoder
// blocks, the separate dropout + residual add that precede it
// (flodl-hf/src/models/transformer_layer.rs:224-263):
//     pre = residual + dropout(x)        (both optional)
//     y   = (pre - mean) * rstd * gamma + beta
// The dropout mask is a pure function of (seed, element index), so the backward pass
// regenerates it and nothing but `pre`, mean and rstd is saved.
//
// Backward produces d(pre) (which is also the residual-branch gradient), optionally
// d(x) = d(pre) * mask, and per-block partial sums of dgamma / dbeta in a scratch buffer that
// a second tiny kernel folds.
#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

constexpr int kLnWarps = 4;

// N consecutive fp32 values p[off .. off+N) as 16-byte loads (N is 4 or 8, off a multiple of N, the
// array 16-byte aligned as every parameter slot is); `fill` when p is null.
template <int N>
__device__ __forceinline__ void load_f32_vec(const float* __restrict__ p, int off, float fill, float (&out)[N]) {
  if (!p) {
#pragma unroll
    for (int j = 0; j < N; ++j) out[j] = fill;
    return;
  }
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(p + off + j));
      out[j] = q.x; out[j + 1] = q.y; out[j + 2] = q.z; out[j + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) out[j] = __ldg(p + off + j);
  }
}

template <typename T, int VPL>
__global__ void __launch_bounds__(kLnWarps * 32)
ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual, const float* __restrict__ gamma,
              const float* __restrict__ beta, T* __restrict__ y, T* __restrict__ pre_out,
              float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int cols, float eps,
              float p_drop, uint64_t seed_in, const unsigned long long* __restrict__ seed_dev) {
  pdl_entry();
  constexpr int V = VecIO<T>::kVec;
  const uint64_t seed = seed_in + (seed_dev ? *seed_dev : 0ull);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kLnWarps + warp;
  if (row >= rows) return;
  const int nvec = cols / V;
  const float inv_keep = p_drop > 0.f ? 1.f / (1.f - p_drop) : 1.f;
  const T* xr = x + static_cast<long long>(row) * cols;
  const T* rr = residual ? residual + static_cast<long long>(row) * cols : nullptr;

  float v[VPL][V];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      VecIO<T>::load(xr + vi * V, v[i]);
      if (p_drop > 0.f) {
        const uint64_t base = static_cast<uint64_t>(row) * cols + static_cast<uint64_t>(vi) * V;
#pragma unroll
        for (int j = 0; j < V; j += 4) {
          float s[4];
          dropout_scale4(seed, base + j, p_drop, inv_keep, s);
#pragma unroll
          for (int k = 0; k < 4; ++k) v[i][j + k] *= s[k];
        }
      }
      if (rr) {
        float r[V];
        VecIO<T>::load(rr + vi * V, r);
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] += r[j];
      }
      if (pre_out) {
        // keep what the backward pass will see: the value rounded to the storage type
        VecIO<T>::store(pre_out + static_cast<long long>(row) * cols + vi * V, v[i]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) sum += v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) v[i][j] = 0.f;
    }
  }
  const float mean = warp_sum(sum) / cols;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    if (lane + i * 32 < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float d = v[i][j] - mean;
        sq += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / cols + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float o[V], g[V], b[V];
      load_f32_vec<V>(gamma, vi * V, 1.f, g);
      load_f32_vec<V>(beta, vi * V, 0.f, b);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = fmaf((v[i][j] - mean) * rstd, g[j], b[j]);
      VecIO<T>::store(y + static_cast<long long>(row) * cols + vi * V, o);
    }
  }
}

template <typename T, int VPL>
__global__ void __launch_bounds__(kLnWarps * 32)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ pre, const float* __restrict__ mean,
              const float* __restrict__ rstd, const float* __restrict__ gamma, T* __restrict__ dpre,
              T* __restrict__ dx_drop, float* __restrict__ partial, int rows, int cols, float p_drop,
              uint64_t seed_in, const unsigned long long* __restrict__ seed_dev) {
  pdl_entry();
  constexpr int V = VecIO<T>::kVec;
  const uint64_t seed = seed_in + (seed_dev ? *seed_dev : 0ull);
  __shared__ float red[kLnWarps][32 * VPL * V + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = cols / V;
  const float inv_keep = p_drop > 0.f ? 1.f / (1.f - p_drop) : 1.f;
  float dg[VPL][V], db[VPL][V];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) dg[i][j] = db[i][j] = 0.f;

  // gamma does not change from row to row: one set of 16-byte loads per thread, kept in registers
  float gm[VPL][V];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      load_f32_vec<V>(gamma, vi * V, 1.f, gm[i]);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) gm[i][j] = 1.f;
    }
  }

  for (int row = blockIdx.x * kLnWarps + warp; row < rows; row += gridDim.x * kLnWarps) {
    const float mu = mean[row], rs = rstd[row];
    float g_dy[VPL][V], xh[VPL][V];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float a[V], b[V];
        VecIO<T>::load(dy + static_cast<long long>(row) * cols + vi * V, a);
        VecIO<T>::load(pre + static_cast<long long>(row) * cols + vi * V, b);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float g = gm[i][j];
          xh[i][j] = (b[j] - mu) * rs;
          dg[i][j] += a[j] * xh[i][j];
          db[i][j] += a[j];
          g_dy[i][j] = a[j] * g;
          s1 += g_dy[i][j];
          s2 += g_dy[i][j] * xh[i][j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) g_dy[i][j] = xh[i][j] = 0.f;
      }
    }
    s1 = warp_sum(s1) / cols;
    s2 = warp_sum(s2) / cols;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = rs * (g_dy[i][j] - s1 - xh[i][j] * s2);
        VecIO<T>::store(dpre + static_cast<long long>(row) * cols + vi * V, o);
        if (dx_drop) {
          const uint64_t base = static_cast<uint64_t>(row) * cols + static_cast<uint64_t>(vi) * V;
#pragma unroll
          for (int j = 0; j < V; j += 4) {
            float s[4];
            dropout_scale4(seed, base + j, p_drop, inv_keep, s);
#pragma unroll
            for (int k = 0; k < 4; ++k) o[j + k] *= s[k];
          }
          VecIO<T>::store(dx_drop + static_cast<long long>(row) * cols + vi * V, o);
        }
      }
    }
  }
  if (!partial) return;
  // fold the 4 warps of the block, then one partial row per block: [dgamma | dbeta]
  for (int pass = 0; pass < 2; ++pass) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int j = 0; j < V; ++j) red[warp][(lane + i * 32) * V + j] = pass == 0 ? dg[i][j] : db[i][j];
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kLnWarps; ++w) s += red[w][c];
      partial[(static_cast<long long>(blockIdx.x) * 2 + pass) * cols + c] = s;
    }
  }
}

__global__ void __launch_bounds__(256)
ln_bwd_finalize_kernel(const float* __restrict__ partial, float* __restrict__ dgamma, float* __restrict__ dbeta, int nblocks,
                       int cols, int accumulate) {
  pdl_entry();
  // block = 32 columns x 8 row-groups; each row-group strides over the partial rows
  __shared__ float rg[8][33], rb[8][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float g = 0.f, b = 0.f;
  // gridDim.y slices of the partial rows run in parallel (only used with accumulate, where the
  // slices can add into the destination atomically); 4 rows in flight per thread
  if (c < cols) {
    const int step = 8 * gridDim.y;
    int i = blockIdx.y * 8 + grp;
    for (; i + 3 * step < nblocks; i += 4 * step) {
      float gg[4], bb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        gg[u] = partial[(static_cast<long long>(i + u * step) * 2) * cols + c];
        bb[u] = partial[(static_cast<long long>(i + u * step) * 2 + 1) * cols + c];
      }
      g += (gg[0] + gg[1]) + (gg[2] + gg[3]);
      b += (bb[0] + bb[1]) + (bb[2] + bb[3]);
    }
    for (; i < nblocks; i += step) {
      g += partial[(static_cast<long long>(i) * 2) * cols + c];
      b += partial[(static_cast<long long>(i) * 2 + 1) * cols + c];
    }
  }
  rg[grp][lane] = g;
  rb[grp][lane] = b;
  __syncthreads();
  if (grp == 0 && c < cols) {
#pragma unroll
    for (int w = 1; w < 8; ++w) { g += rg[w][lane]; b += rb[w][lane]; }
    if (gridDim.y > 1) {
      if (dgamma) atomicAdd(dgamma + c, g);
      if (dbeta) atomicAdd(dbeta + c, b);
    } else {
      if (dgamma) dgamma[c] = accumulate ? dgamma[c] + g : g;
      if (dbeta) dbeta[c] = accumulate ? dbeta[c] + b : b;
    }
  }
}

template <typename T, int VPL>
static int ln_fwd_launch(const void* x, const void* res, const float* gamma, const float* beta, void* y,
                         void* pre, float* mean, float* rstd, int rows, int cols, float eps, float p,
                         uint64_t seed, const unsigned long long* seed_dev, cudaStream_t st) {
  const int grid = (rows + kLnWarps - 1) / kLnWarps;
  launch_pdl(ln_fwd_kernel<T, VPL>, dim3(grid), dim3(kLnWarps * 32), 0, st, static_cast<const T*>(x), static_cast<const T*>(res), gamma, beta, static_cast<T*>(y),
      static_cast<T*>(pre), mean, rstd, rows, cols, eps, p, seed, seed_dev);
  return static_cast<int>(cudaGetLastError());
}

template <typename T, int VPL>
static int ln_bwd_launch(const void* dy, const void* pre, const float* mean, const float* rstd,
                         const float* gamma, void* dpre, void* dxd, float* partial, int grid, int rows,
                         int cols, float p, uint64_t seed, const unsigned long long* seed_dev, cudaStream_t st) {
  launch_pdl(ln_bwd_kernel<T, VPL>, dim3(grid), dim3(kLnWarps * 32), 0, st, static_cast<const T*>(dy), static_cast<const T*>(pre), mean, rstd, gamma, static_cast<T*>(dpre),
      static_cast<T*>(dxd), partial, rows, cols, p, seed, seed_dev);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fb

#define FB_LN_DISPATCH(FN, ...)                                                     \
  do {                                                                              \
    const int vec = is_bf16 ? 8 : 4;                                                \
    const int vpl = (cols / vec + 31) / 32;                                         \
    if (is_bf16) {                                                                  \
      switch (vpl) {                                                                \
        case 1: return fb::FN<__nv_bfloat16, 1>(__VA_ARGS__);                       \
        case 2: return fb::FN<__nv_bfloat16, 2>(__VA_ARGS__);                       \
        case 3: return fb::FN<__nv_bfloat16, 3>(__VA_ARGS__);                       \
        case 4: return fb::FN<__nv_bfloat16, 4>(__VA_ARGS__);                       \
        default: return -4;                                                         \
      }                                                                             \
    } else {                                                                        \
      switch (vpl) {                                                                \
        case 1: return fb::FN<float, 1>(__VA_ARGS__);                               \
        case 2: return fb::FN<float, 2>(__VA_ARGS__);                               \
        case 3: return fb::FN<float, 3>(__VA_ARGS__);                               \
        case 4: return fb::FN<float, 4>(__VA_ARGS__);                               \
        case 5: case 6: return fb::FN<float, 6>(__VA_ARGS__);                       \
        case 7: case 8: return fb::FN<float, 8>(__VA_ARGS__);                       \
        default: return -4;                                                         \
      }                                                                             \
    }                                                                               \
  } while (0)

extern "C" int fb_layernorm_max_cols(int is_bf16) { return 1024; }

extern "C" int fb_layernorm_fwd(const void* x, const void* residual, const float* gamma, const float* beta,
                                void* y, void* pre_out, float* mean, float* rstd, int rows, int cols,
                                float eps, float p_drop, unsigned long long seed, const unsigned long long* seed_dev, int is_bf16, void* stream) {
  if (rows <= 0) return 0;
  if (cols % (is_bf16 ? 8 : 4) || cols > 1024) return -4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FB_LN_DISPATCH(ln_fwd_launch, x, residual, gamma, beta, y, pre_out, mean, rstd, rows, cols, eps, p_drop, seed, seed_dev, st);
}

// One resident wave: the backward kernel keeps its dgamma / dbeta partial sums in registers (about
// 160 per thread), so three 128-thread blocks fit on an SM; more blocks than that would run as a
// second, mostly empty wave.
extern "C" int fb_layernorm_bwd_grid(int rows) {
  static int cap = 0;
  if (!cap) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cap = 3 * (sms > 0 ? sms : 148);
  }
  int g = (rows + fb::kLnWarps - 1) / fb::kLnWarps;
  return g < cap ? g : cap;
}

// `partial` must hold fb_layernorm_bwd_grid(rows) * 2 * cols floats.
extern "C" int fb_layernorm_bwd(const void* dy, const void* pre, const float* mean, const float* rstd,
                                const float* gamma, void* dpre, void* dx_drop, float* partial, float* dgamma,
                                float* dbeta, int accumulate, int rows, int cols, float p_drop,
                                unsigned long long seed, const unsigned long long* seed_dev, int is_bf16, void* stream) {
  if (rows <= 0) return 0;
  if (cols % (is_bf16 ? 8 : 4) || cols > 1024) return -4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = fb_layernorm_bwd_grid(rows);
  auto run = [&]() -> int {
    FB_LN_DISPATCH(ln_bwd_launch, dy, pre, mean, rstd, gamma, dpre, dx_drop, partial, grid, rows, cols, p_drop, seed, seed_dev, st);
  };
  int r = run();
  if (r) return r;
  if (partial && (dgamma || dbeta)) {
    const dim3 fgrid((cols + 31) / 32, accumulate ? 8 : 1);
    fb::launch_pdl(fb::ln_bwd_finalize_kernel, dim3(fgrid), dim3(256), 0, st, partial, dgamma, dbeta, grid, cols, accumulate);
    return static_cast<int>(cudaGetLastError());
  }
  return 0;
}
