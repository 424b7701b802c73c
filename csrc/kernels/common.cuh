// Shared device helpers for the bandwidth-bound kernels: 16-byte vector access, bf16<->fp32
// packing, warp/block reductions and a counter-based RNG (Philox-4x32-10) for dropout masks that
// the backward pass regenerates instead of storing.
#pragma once
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

template <typename T>
struct VecIO;

template <>
struct VecIO<float> {
  static constexpr int kVec = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  __device__ static float get(const float* p) { return *p; }
  __device__ static void put(float* p, float v) { *p = v; }
};

template <>
struct VecIO<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
  }
  __device__ static float get(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void put(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds >= 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// Philox-4x32-10: 4 uniform 32-bit words per (key, counter).
__device__ __forceinline__ uint4 philox4x32(uint2 key, uint4 ctr) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// Keep-mask for element `idx` of a dropout site: deterministic in (seed, idx), so forward and
// backward agree without storing the mask. Returns 1/(1-p) for kept elements, 0 for dropped.
__device__ __forceinline__ float dropout_scale(uint64_t seed, uint64_t idx, float p, float inv_keep) {
  uint4 r = philox4x32(make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)),
                       make_uint4(static_cast<uint32_t>(idx >> 2), static_cast<uint32_t>(idx >> 34), 0u, 0u));
  const uint32_t w = (idx & 3) == 0 ? r.x : (idx & 3) == 1 ? r.y : (idx & 3) == 2 ? r.z : r.w;
  const float u = (w >> 8) * (1.0f / 16777216.0f);
  return u >= p ? inv_keep : 0.f;
}
// Four consecutive elements starting at a multiple of 4.
__device__ __forceinline__ void dropout_scale4(uint64_t seed, uint64_t idx4, float p, float inv_keep, float (&s)[4]) {
  uint4 r = philox4x32(make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)),
                       make_uint4(static_cast<uint32_t>(idx4 >> 2), static_cast<uint32_t>(idx4 >> 34), 0u, 0u));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = ((w[i] >> 8) * (1.0f / 16777216.0f)) >= p ? inv_keep : 0.f;
}


// ---- fast GELU for bf16 outputs ---------------------------------------------------------------------
// One hardware tanh (tanh.approx.f32, relative error 2^-11) per value. For the erf form,
// erf(x / sqrt(2)) is written as tanh(g(x)) with g an odd degree-5 polynomial fitted (minimax over
// [0, 6]) so that |tanh(g(x)) - erf(x / sqrt(2))| < 3.7e-5, i.e. |GELU error| < 6e-5: below half a
// bf16 ulp wherever |GELU(x)| > 0.03. x is clamped to +-8 before the polynomial (its quartic term is
// negative, and tanh has long saturated there).
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float erf_tanh_arg(float x) {
  const float u = fminf(fmaxf(x, -8.0f), 8.0f);
  const float u2 = u * u;
  return u * fmaf(u2, fmaf(u2, -0.00031580707f, 0.03679825612f), 0.7977178338f);
}
__device__ __forceinline__ float gelu_erf_fast(float x) {
  const float hx = 0.5f * x;
  return fmaf(hx, tanh_approx(erf_tanh_arg(x)), hx);
}
__device__ __forceinline__ float dgelu_erf_fast(float x) {
  const float cdf = fmaf(0.5f, tanh_approx(erf_tanh_arg(x)), 0.5f);
  const float pdf = 0.3989422804f * ex2_approx(-0.7213475204f * x * x);   // exp(-x^2/2) / sqrt(2 pi)
  return fmaf(x, pdf, cdf);
}
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float hx = 0.5f * x;
  const float u = x * fmaf(x * x, 0.0356774081f, 0.7978845608f);
  return fmaf(hx, tanh_approx(u), hx);
}
__device__ __forceinline__ float dgelu_tanh_fast(float x) {
  const float x2 = x * x;
  const float t = tanh_approx(x * fmaf(x2, 0.0356774081f, 0.7978845608f));
  const float du = fmaf(x2, 0.1070322243f, 0.7978845608f);
  return fmaf(0.5f * x * (1.0f - t * t), du, fmaf(0.5f, t, 0.5f));
}


// ---- bounds-checked debug build -------------------------------------------------------------------
// With -DFLODL_BOUNDS_CHECK=1 (FLODL_B200_BOUNDS_CHECK=1 at build time) every index that a kernel
// takes from device memory (token ids, compaction tables, targets, row counts) is range-checked
// before it is used. A violation never traps: the first one is recorded as {site, index, limit} in
// a host-visible word that `fb_bounds_report` reads, and the access is skipped. This is the
// stand-in for a memory checker on machines where none may be run. A regular build compiles the
// checks away.
#ifndef FLODL_BOUNDS_CHECK
#define FLODL_BOUNDS_CHECK 0
#endif
#if FLODL_BOUNDS_CHECK
static __device__ int* g_fb_bounds_word = nullptr;     // one per translation unit, all attached to the same record
__device__ __forceinline__ bool fb_index_ok(long long i, long long n, int site) {
  if (i >= 0 && i < n) return true;
  int* w = g_fb_bounds_word;
  if (w && atomicCAS(w, 0, site) == 0) {
    w[1] = static_cast<int>(i < -2147483647LL ? -2147483647LL : (i > 2147483647LL ? 2147483647LL : i));
    w[2] = static_cast<int>(n > 2147483647LL ? 2147483647LL : n);
  }
  return false;
}
#define FB_INDEX_OK(i, n, site) (::fb::fb_index_ok((i), (n), (site)))
#define FB_BOUNDS_ATTACH(name)                                                                  \
  extern "C" int fb_bounds_attach_##name(int* dev_word) {                                       \
    return static_cast<int>(cudaMemcpyToSymbol(::fb::g_fb_bounds_word, &dev_word, sizeof(dev_word))); \
  }
#else
#define FB_INDEX_OK(i, n, site) (true)
#define FB_BOUNDS_ATTACH(name) \
  extern "C" int fb_bounds_attach_##name(int*) { return 0; }
#endif

// ---- programmatic dependent launch -----------------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its predecessor
// in the stream is still running. `pdl_wait()` blocks until the predecessor grid has completed and
// its writes are visible; it must precede the first access to anything the predecessor produced
// (and any write the predecessor might still read). `pdl_launch_dependents()` tells the scheduler
// that the successor may begin its own preamble. Both are no-ops for ordinary launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// First statements of every kernel launched through `launch_pdl`: wait for the predecessor, then let the
// successor's blocks be scheduled as this grid's blocks retire.
__device__ __forceinline__ void pdl_entry() {
  pdl_wait();
  pdl_launch_dependents();
}

// Host switch: FLODL_B200_PDL=0 turns the launch attribute off everywhere.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("FLODL_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}


// `kern<<<grid, block, smem, stream>>>(args...)` with the programmatic-serialization attribute: the
// launch latency and block ramp-up of this kernel overlap the tail of the one before it in the stream
// (which matters when a training step is hundreds of kernels of a few microseconds each). The kernel
// must start with `pdl_entry()`.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace fb
