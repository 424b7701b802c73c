// Fused softmax cross-entropy: one pass for the row statistics, one pass that writes the gradient.
//
// Replaces `at::cross_entropy_loss` (flodl-sys/ops_training.cpp:926-937; mean reduction,
// ignore_index) and the log_softmax / nll backward kernels libtorch runs for it. Logits may be
// bf16 or fp32; all math is fp32. The gradient (softmax - onehot) / n_valid is produced in the
// forward launch (it may overwrite the logits), so the backward pass is a scalar multiply that the
// consumer GEMMs take as their `alpha`.
#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

__global__ void ce_count_kernel(const long long* __restrict__ targets, int rows, long long ignore_index,
                                float* __restrict__ count_inv /* [0]=count, [1]=1/max(count,1) */) {
  __shared__ float scratch[32];
  float c = 0.f;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) c += (targets[i] != ignore_index) ? 1.f : 0.f;
  c = block_sum(c, scratch);
  if (threadIdx.x == 0) {
    count_inv[0] = c;
    count_inv[1] = 1.f / fmaxf(c, 1.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
ce_fwd_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ targets, int rows,
              int V, long long ignore_index, T* __restrict__ dlogits, long long ldd,
              const float* __restrict__ count_inv, float* __restrict__ row_loss, const int* __restrict__ counts) {
  pdl_entry();
  constexpr int VEC = VecIO<T>::kVec;
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  if (counts && row >= counts[1]) {      // compacted input: nothing lives past the padded count
    if (row_loss && threadIdx.x == 0) row_loss[row] = 0.f;
    return;
  }
  const long long t = targets[row];
  const T* lr = logits + static_cast<long long>(row) * ld;
  T* dr = dlogits ? dlogits + static_cast<long long>(row) * ldd : nullptr;
  const int nvec = V / VEC;
  const bool aligned = ((reinterpret_cast<uintptr_t>(lr) & 15) == 0) && (!dr || (reinterpret_cast<uintptr_t>(dr) & 15) == 0);

  if (t != ignore_index) (void)FB_INDEX_OK(t, V, 201);        // a label outside the vocabulary is recorded (and treated as ignored)
  if (counts) (void)FB_INDEX_OK(counts[0], static_cast<long long>(rows) + 1, 202);
  if (t == ignore_index || t < 0 || t >= V) {
    if (row_loss && threadIdx.x == 0) row_loss[row] = 0.f;
    if (dr) {
      if (aligned) {
        float z[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) z[j] = 0.f;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) VecIO<T>::store(dr + i * VEC, z);
        for (int k = nvec * VEC + threadIdx.x; k < V; k += blockDim.x) VecIO<T>::put(dr + k, 0.f);
      } else {
        for (int k = threadIdx.x; k < V; k += blockDim.x) VecIO<T>::put(dr + k, 0.f);
      }
    }
    return;
  }

  // online max / sum-exp per thread
  float m = -INFINITY, s = 0.f;
  auto visit = [&](float x) {
    if (x > m) {
      s = s * __expf(m - x) + 1.f;
      m = x;
    } else {
      s += __expf(x - m);
    }
  };
  if (aligned) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float v[VEC];
      VecIO<T>::load(lr + i * VEC, v);
#pragma unroll
      for (int j = 0; j < VEC; ++j) visit(v[j]);
    }
    for (int k = nvec * VEC + threadIdx.x; k < V; k += blockDim.x) visit(VecIO<T>::get(lr + k));
  } else {
    for (int k = threadIdx.x; k < V; k += blockDim.x) visit(VecIO<T>::get(lr + k));
  }
  const float gmax = block_max(m, scratch);
  const float mine = (m == -INFINITY) ? 0.f : s * __expf(m - gmax);
  const float gsum = block_sum(mine, scratch);
  const float lse = __logf(gsum) + gmax;
  if (row_loss && threadIdx.x == 0) row_loss[row] = lse - VecIO<T>::get(lr + t);
  if (!dr) return;

  const float inv_n = count_inv ? count_inv[1] : 1.f;
  const float inv_sum = 1.f / gsum;
  if (aligned) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float v[VEC];
      VecIO<T>::load(lr + i * VEC, v);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float pr = __expf(v[j] - gmax) * inv_sum;
        v[j] = (pr - ((i * VEC + j) == t ? 1.f : 0.f)) * inv_n;
      }
      VecIO<T>::store(dr + i * VEC, v);
    }
    for (int k = nvec * VEC + threadIdx.x; k < V; k += blockDim.x) {
      const float pr = __expf(VecIO<T>::get(lr + k) - gmax) * inv_sum;
      VecIO<T>::put(dr + k, (pr - (k == t ? 1.f : 0.f)) * inv_n);
    }
  } else {
    for (int k = threadIdx.x; k < V; k += blockDim.x) {
      const float pr = __expf(VecIO<T>::get(lr + k) - gmax) * inv_sum;
      VecIO<T>::put(dr + k, (pr - (k == t ? 1.f : 0.f)) * inv_n);
    }
  }
}

// loss = sum(row_loss) / max(count, 1), in a fixed order (deterministic).
__global__ void ce_finalize_kernel(const float* __restrict__ row_loss, int rows, const float* __restrict__ count_inv,
                                   float* __restrict__ loss) {
  pdl_entry();
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) s += row_loss[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) loss[0] = s * count_inv[1];
}

// x[r][c] *= *scalar (device scalar); rows of length `cols` with leading dimension `ld`.
template <typename T>
__global__ void scale_rows_kernel(T* __restrict__ x, long long ld, int rows, int cols, const float* __restrict__ scalar) {
  pdl_entry();
  const float a = *scalar;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    T* xr = x + static_cast<long long>(r) * ld;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) VecIO<T>::put(xr + c, VecIO<T>::get(xr + c) * a);
  }
}

}  // namespace fb

// count_inv: 2 floats, row_loss: `rows` floats, loss: 1 float (all device memory, caller-owned).
extern "C" int fb_softmax_ce_dyn(const void* logits, long long ld, const long long* targets, int rows, int V,
                                 long long ignore_index, void* dlogits, long long ldd, float* count_inv,
                                 float* row_loss, float* loss, int is_bf16, const int* counts, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  fb::launch_pdl(fb::ce_count_kernel, dim3(1), dim3(1024), 0, st, targets, rows, ignore_index, count_inv);
  if (is_bf16)
    fb::launch_pdl(fb::ce_fwd_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(logits), ld, targets, rows,
                                                           V, ignore_index, static_cast<__nv_bfloat16*>(dlogits), ldd,
                                                           count_inv, row_loss, counts);
  else
    fb::launch_pdl(fb::ce_fwd_kernel<float>, dim3(rows), dim3(256), 0, st, static_cast<const float*>(logits), ld, targets, rows, V,
                                                   ignore_index, static_cast<float*>(dlogits), ldd, count_inv, row_loss, counts);
  if (loss) fb::launch_pdl(fb::ce_finalize_kernel, dim3(1), dim3(1024), 0, st, row_loss, rows, count_inv, loss);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_softmax_ce(const void* logits, long long ld, const long long* targets, int rows, int V,
                             long long ignore_index, void* dlogits, long long ldd, float* count_inv,
                             float* row_loss, float* loss, int is_bf16, void* stream) {
  return fb_softmax_ce_dyn(logits, ld, targets, rows, V, ignore_index, dlogits, ldd, count_inv, row_loss, loss, is_bf16, nullptr, stream);
}

extern "C" int fb_scale_rows(void* x, long long ld, int rows, int cols, const float* scalar, int is_bf16, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (is_bf16)
    fb::launch_pdl(fb::scale_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, static_cast<__nv_bfloat16*>(x), ld, rows, cols, scalar);
  else
    fb::launch_pdl(fb::scale_rows_kernel<float>, dim3(grid), dim3(256), 0, st, static_cast<float*>(x), ld, rows, cols, scalar);
  return static_cast<int>(cudaGetLastError());
}

FB_BOUNDS_ATTACH(softmax_ce)
