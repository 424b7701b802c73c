// Optimizer and gradient-norm kernels over flat buffers.
//
//  * fused Adam / AdamW: replaces `at::_fused_adamw_` (flodl-sys/ops_training.cpp:653-725); same
//    update as the decomposed form at ops_training.cpp:576-613:
//        p *= 1 - lr*wd;  m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;
//        p -= (lr / (1-b1^t)) * m / (sqrt(v / (1-b2^t)) + eps)
//    One launch covers every parameter of the group because parameters, gradients and moments
//    live in flat buffers; the kernel also refreshes the bf16 shadow copy the GEMMs read.
//  * fused SGD-momentum: replaces the per-parameter op chain of flodl/src/nn/optim/sgd.rs:132-172
//    (g += wd*p; v = mu*v + g (v = g on the first step); p -= lr*v).
//  * sum of squares + clip coefficient: replaces `_foreach_norm` + stack + norm + `.item()` of
//    ops_training.cpp:769-800 without the host sync: the coefficient min(1, max/(norm+1e-6))
//    stays on the device and the optimizer kernel multiplies the gradient by it.
//
// Hyper-parameters that change every step (lr, bias corrections) are read from device memory so a
// captured CUDA graph can replay the step with new values.
#include <atomic>

#include "../include/flodl_b200.h"
#include "common.cuh"

namespace fb {

// hyper = {lr, 1-b1^t, 1-b2^t, weight_decay}
template <typename TG>
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, const TG* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
            __nv_bfloat16* __restrict__ p16, long long n, const float* __restrict__ hyper, float b1, float b2,
            float eps, const float* __restrict__ grad_scale, const int* __restrict__ skip, float4 hv) {
  pdl_entry();
  // `skip`: a device-visible word that a collective sets when it gave up; the update is then left out
  // and the parameters stay as they were, so the host can raise before anything diverged.
  if (skip && __ldg(skip) != 0) return;
  // hyper-parameters from device memory (a captured graph replays with fresh values) or, when `hyper` is null, by value
  const float lr = hyper ? hyper[0] : hv.x, bc1 = hyper ? hyper[1] : hv.y, bc2 = hyper ? hyper[2] : hv.z, wd = hyper ? hyper[3] : hv.w;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 pp = *reinterpret_cast<float4*>(p + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float gg[4];
      if constexpr (sizeof(TG) == 4) {
        float4 t = *reinterpret_cast<const float4*>(g + i);
        gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
      } else {
        uint2 raw = *reinterpret_cast<const uint2*>(g + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
      }
      float* pa = reinterpret_cast<float*>(&pp);
      float* ma = reinterpret_cast<float*>(&mm);
      float* va = reinterpret_cast<float*>(&vv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gg[j] * gs;
        pa[j] *= decay;
        ma[j] = b1 * ma[j] + (1.f - b1) * gj;
        va[j] = b2 * va[j] + (1.f - b2) * gj * gj;
        pa[j] -= step_size * ma[j] / (sqrtf(va[j]) * inv_sqrt_bc2 + eps);
      }
      *reinterpret_cast<float4*>(p + i) = pp;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (p16) {
        __nv_bfloat162 o[2] = {__floats2bfloat162_rn(pa[0], pa[1]), __floats2bfloat162_rn(pa[2], pa[3])};
        *reinterpret_cast<uint2*>(p16 + i) = *reinterpret_cast<uint2*>(o);
      }
    } else {
      for (long long k = i; k < n; ++k) {
        const float gj = VecIO<TG>::get(g + k) * gs;
        float pk = p[k] * decay;
        const float mk = b1 * m[k] + (1.f - b1) * gj;
        const float vk = b2 * v[k] + (1.f - b2) * gj * gj;
        pk -= step_size * mk / (sqrtf(vk) * inv_sqrt_bc2 + eps);
        p[k] = pk; m[k] = mk; v[k] = vk;
        if (p16) p16[k] = __float2bfloat16(pk);
      }
    }
  }
}

// hyper = {lr, momentum, weight_decay, first_step (0/1)}
template <typename TG>
__global__ void __launch_bounds__(256)
sgd_kernel(float* __restrict__ p, const TG* __restrict__ g, float* __restrict__ buf, __nv_bfloat16* __restrict__ p16,
           long long n, const float* __restrict__ hyper, const float* __restrict__ grad_scale, const int* __restrict__ skip) {
  pdl_entry();
  if (skip && __ldg(skip) != 0) return;
  const float lr = hyper[0], mu = hyper[1], wd = hyper[2];
  const bool first = hyper[3] != 0.f;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float pk = p[i];
    float gk = VecIO<TG>::get(g + i) * gs + wd * pk;
    if (buf) {
      const float b = first ? gk : mu * buf[i] + gk;
      buf[i] = b;
      gk = b;
    }
    pk -= lr * gk;
    p[i] = pk;
    if (p16) p16[i] = __float2bfloat16(pk);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  pdl_entry();
  __shared__ float scratch[32];
  constexpr int V = VecIO<T>::kVec;
  float s = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * V;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
    if (i + V <= n) {
      float v[V];
      VecIO<T>::load(x + i, v);
#pragma unroll
      for (int j = 0; j < V; ++j) s += v[j] * v[j];
    } else {
      for (long long k = i; k < n; ++k) {
        const float t = VecIO<T>::get(x + k);
        s += t * t;
      }
    }
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// out = {norm, clip coefficient = min(1, max_norm / (norm + 1e-6)) or 1 when max_norm <= 0}
__global__ void sumsq_finalize_kernel(const float* __restrict__ partial, int nparts, float max_norm,
                                      float extra_scale, float* __restrict__ out) {
  pdl_entry();
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) {
    const float norm = sqrtf(s) * extra_scale;
    out[0] = norm;
    float coef = 1.f;
    if (max_norm > 0.f && norm > max_norm) coef = max_norm / (norm + 1e-6f);
    out[1] = coef * extra_scale;
  }
}

}  // namespace fb

extern "C" int fb_adam_step(float* p, const void* g, float* m, float* v, void* p16, long long n,
                            const float* hyper, float b1, float b2, float eps, const float* grad_scale,
                            int g_bf16, const int* skip, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (g_bf16)
    fb::launch_pdl(fb::adam_kernel<__nv_bfloat16>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, p, static_cast<const __nv_bfloat16*>(g), m, v, static_cast<__nv_bfloat16*>(p16), n, hyper, b1, b2, eps, grad_scale, skip, make_float4(0.f, 0.f, 0.f, 0.f));
  else
    fb::launch_pdl(fb::adam_kernel<float>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, p, static_cast<const float*>(g), m, v,
                                                                     static_cast<__nv_bfloat16*>(p16), n, hyper, b1, b2,
                                                                     eps, grad_scale, skip, make_float4(0.f, 0.f, 0.f, 0.f));
  return static_cast<int>(cudaGetLastError());
}

// The same update with the hyper-parameters {lr, 1-b1^t, 1-b2^t, weight_decay} passed from the host (eager callers
// that have them at hand and do not replay the launch from a graph).
extern "C" int fb_adam_step_host(float* p, const void* g, float* m, float* v, long long n, const float* hyper_host, float b1, float b2,
                                 float eps, int g_bf16, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  const float4 hv = make_float4(hyper_host[0], hyper_host[1], hyper_host[2], hyper_host[3]);
  if (g_bf16)
    fb::launch_pdl(fb::adam_kernel<__nv_bfloat16>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, p, static_cast<const __nv_bfloat16*>(g), m, v,
                   static_cast<__nv_bfloat16*>(nullptr), n, static_cast<const float*>(nullptr), b1, b2, eps, static_cast<const float*>(nullptr),
                   static_cast<const int*>(nullptr), hv);
  else
    fb::launch_pdl(fb::adam_kernel<float>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, p, static_cast<const float*>(g), m, v,
                   static_cast<__nv_bfloat16*>(nullptr), n, static_cast<const float*>(nullptr), b1, b2, eps, static_cast<const float*>(nullptr),
                   static_cast<const int*>(nullptr), hv);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_sgd_step(float* p, const void* g, float* buf, void* p16, long long n, const float* hyper,
                           const float* grad_scale, int g_bf16, const int* skip, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (g_bf16)
    fb::launch_pdl(fb::sgd_kernel<__nv_bfloat16>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, p, static_cast<const __nv_bfloat16*>(g), buf, static_cast<__nv_bfloat16*>(p16), n, hyper, grad_scale, skip);
  else
    fb::launch_pdl(fb::sgd_kernel<float>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, p, static_cast<const float*>(g), buf,
                                                                    static_cast<__nv_bfloat16*>(p16), n, hyper, grad_scale, skip);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_grad_norm_parts(long long n) {
  long long b = (n / 8 + 255) / 256;
  if (b > 1024) b = 1024;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

// partial: fb_grad_norm_parts(n) floats of scratch; out: 2 floats {norm, clip coefficient}.
// `extra_scale` multiplies the norm (e.g. 1/loss_scale) and is folded into the coefficient.
extern "C" int fb_grad_norm(const void* g, long long n, float* partial, float max_norm, float extra_scale,
                            float* out, int is_bf16, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int parts = fb_grad_norm_parts(n);
  if (is_bf16)
    fb::launch_pdl(fb::sumsq_partial_kernel<__nv_bfloat16>, dim3(parts), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(g), n, partial);
  else
    fb::launch_pdl(fb::sumsq_partial_kernel<float>, dim3(parts), dim3(256), 0, st, static_cast<const float*>(g), n, partial);
  fb::launch_pdl(fb::sumsq_finalize_kernel, dim3(1), dim3(256), 0, st, partial, parts, max_norm, extra_scale, out);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of fb_grad_norm (no counterpart in the reference).
//
// Who needs it: code that computes a gradient norm from a place where device memory must not be
// requested - inside a region that is being captured into a CUDA graph by a caller who owns no
// memory pool, from a host thread that is forbidden to touch the allocator while a collective is
// pending on another stream, or from a foreign runtime that links this library through the C ABI
// and has no allocator to hand us. Such callers still own the gradient buffer and the two-float
// result; the only thing fb_grad_norm additionally needs is room for one partial sum per block,
// and here that room is a fixed array inside the library.
//
// The array costs 4 KB on every GPU that loads the library, for the life of the process. All calls
// share it: each launch overwrites every slot it later reads, so nothing has to be cleared between
// calls, but two calls that overlap on the GPU (different streams, no ordering) would corrupt
// each other's partial sums - serialise them. The first call on a device looks the array's device
// address up (with that device current) and remembers it; make that first call outside any
// stream capture.
constexpr int kNormScratchFloats = 1024;
static __device__ __align__(256) float g_norm_scratch[kNormScratchFloats];

extern "C" int fb_grad_norm_noalloc(const void* g, long long n, float max_norm, float extra_scale, float* out,
                                    int is_bf16, void* stream) {
  if (n < 0 || n > FB_GRAD_NORM_NOALLOC_MAX_ELEMS) return -4;   // see fb_grad_norm_noalloc_max()
  constexpr int kMaxDevices = 64;
  // Two host threads may make the first call on one device at the same time; both resolve the same
  // address, so a relaxed atomic slot is all the cache needs.
  static std::atomic<float*> scratch_of[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -4;
  float* partial = scratch_of[dev].load(std::memory_order_relaxed);
  if (!partial) {
    // In host code `g_norm_scratch` is only a handle for the symbol; the kernel needs the address
    // the array has on THIS device.
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_norm_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    scratch_of[dev].store(ptr, std::memory_order_relaxed);
    partial = ptr;
  }
  const int parts = fb_grad_norm_parts(n);
  if (parts > kNormScratchFloats) return -4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    fb::launch_pdl(fb::sumsq_partial_kernel<__nv_bfloat16>, dim3(parts), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(g), n, partial);
  else
    fb::launch_pdl(fb::sumsq_partial_kernel<float>, dim3(parts), dim3(256), 0, st, static_cast<const float*>(g), n, partial);
  fb::launch_pdl(fb::sumsq_finalize_kernel, dim3(1), dim3(256), 0, st, partial, parts, max_norm, extra_scale, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" long long fb_grad_norm_noalloc_max(void) { return FB_GRAD_NORM_NOALLOC_MAX_ELEMS; }
