// Collectives over peer-mapped ("symmetric") buffers: every rank holds a pointer to the same
// buffer on every other GPU of the NVSwitch domain and the kernels below load from / store to
// those peers directly. Two data paths, no TMA in either:
//   * NVLS: when the buffers are bound to an NVLink-switch multicast object (csrc/runtime/vmm.cpp),
//     `multimem.ld_reduce` lets the switch read one offset on every GPU and return the sum, and
//     `multimem.st` lets it write every GPU's copy. An all-reduce then moves each byte over a
//     GPU's links once per direction instead of twice, and costs one load + one store per vector
//     instead of W + W.
//   * plain P2P ld/st over NVLink (any world size, per-rank weights, and every test in which a
//     rank leaves or a wait runs out).
//
//  * fb_allreduce       - replaces the per-tensor `ncclAllReduce` group the reference issues after
//                         backward (flodl-sys/ops_cuda.cpp:326-369, flodl/src/distributed/ddp.rs:133-147,
//                         weighted form ddp.rs:206-225). One launch per flat bucket; the average
//                         (or per-rank weight) and the bf16<->fp32 cast are fused.
//                           two-shot, in place: rank r reduces shard r from all peers and pushes
//                                               the result into every peer's buffer;
//                           one-shot          : every rank reads all peers and writes a local
//                                               output (for small buckets, latency bound).
//  * fb_param_average   - replaces scratch copy + `ncclAllReduce(Avg)` over the parameters +
//                         foreach sub/norm of Local-SGD averaging
//                         (flodl/src/distributed/ddp_run/worker.rs:515-584): peer reduce into a
//                         staging buffer, then w = lerp(w, mean, alpha) in place, the bf16 shadow
//                         refresh and the partial sums of |post-pre|^2 and |post|^2, one launch.
//  * fb_broadcast       - replaces the per-tensor `ncclBroadcast` group (ops_cuda.cpp:371-413,
//                         ddp.rs:150-167): every non-root rank pulls the root's flat buffer.
//
// Synchronisation: per-block flags in a peer-mapped signal pad, written with st.release.sys and
// polled with ld.acquire.sys. Block b of rank r only ever waits for block b of the other ranks, so
// no grid-wide barrier is needed and the kernels are safe under partial residency. Every poll
// loop is bounded; on give-up (or when the host raises `abort`) the kernel records a status code
// and returns with the context intact. Flag values are per-block epochs kept in device memory,
// so a captured CUDA graph replays correctly.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/flodl_b200.h"
#include "../kernels/common.cuh"
#include "../kernels/ptx_sm100.cuh"

namespace fb {

struct SymmCtx {
  void* data[FB_MAX_RANKS];      // peer pointers to the payload buffer, indexed by rank
  uint32_t* sig[FB_MAX_RANKS];   // peer pointers to the signal pads
  uint32_t* epochs;              // local: one epoch counter per block
  const int* abort;              // optional host-mapped abort word
  int* status;                   // status word (host-mapped when the host wants to poll it without a sync)
  int* status_dev;               // the same word in device memory (read by kernels, e.g. the optimizers' skip check)
  long long timeout_ns;          // bound of every wait
  char* mc;                      // multicast address of the payload buffer (nullptr: no NVLS)
  int rank, world;
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The status word may live in host-mapped memory (the host polls it without a sync), where device
// atomics are not dependable: first writer wins by a plain check-then-store, made visible system-wide.
__device__ __forceinline__ void set_status_sys(int* status, int* status_dev, int code) {
  if (status_dev) atomicCAS(status_dev, 0, code);
  if (!status) return;
  volatile int* s = status;
  if (*s == 0) {
    *s = code;
    __threadfence_system();
  }
}

// All threads of the block call this. Returns false after a bounded wait ran out.
//
// Failure spreads through the fabric: a rank whose wait runs out writes a "poison" word into every
// peer's signal pad, and every barrier looks at its own poison word while it waits. So once one
// rank has given up, the collectives of all ranks return at their next barrier with a status the
// host reads, instead of pairing flags of different launches. The pad, the epochs and the poison
// word are cleared together by the host (`SymmetricBuffer.recover`, between two host barriers).
constexpr int kStatusPeerGaveUp = 7;

__device__ __forceinline__ bool symm_block_barrier(const SymmCtx& c, uint32_t& epoch, int* sh_fail) {
  __syncthreads();
  epoch += 1;
  const int t = threadIdx.x;
  if (t < c.world) {
    __threadfence_system();
    st_release_sys(c.sig[t] + blockIdx.x * FB_MAX_RANKS + c.rank, epoch);
    const uint32_t* mine = c.sig[c.rank] + blockIdx.x * FB_MAX_RANKS + t;
    const uint32_t* poison = c.sig[c.rank] + FB_SIGNAL_POISON_INDEX;
    int fail = 0;
    const unsigned long long t0 = global_ns();
    // The wait ends when the peer's flag arrives, when a peer has given up, when the host raises
    // `abort`, or when `timeout_ns` has passed on the global timer. The iteration bound is a second
    // line of defence derived from the same timeout (a poll with its back-off takes well over 16 ns).
    const unsigned long long max_it = static_cast<unsigned long long>(c.timeout_ns) / 16ull + 4096ull;
    if (ld_acquire_sys(poison) != 0) fail = kStatusPeerGaveUp;
    if (!fail) {
      fail = kStatusWaitPeer;
      for (unsigned long long it = 0; it < max_it; ++it) {
        if (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) >= 0) { fail = 0; break; }
        if ((it & 63) == 63) {
          if (ld_acquire_sys(poison) != 0) { fail = kStatusPeerGaveUp; break; }
          if (c.abort && *reinterpret_cast<const volatile int*>(c.abort)) break;
          if (global_ns() - t0 > static_cast<unsigned long long>(c.timeout_ns)) break;
        }
        if (it > 32) __nanosleep(64);
      }
    }
    if (fail) {
      *sh_fail = 1;
      set_status_sys(c.status, c.status_dev, fail);
      st_release_sys(c.sig[t] + FB_SIGNAL_POISON_INDEX, 1u);   // tell peer t (and this rank's own later launches)
    }
  }
  __syncthreads();
  return *reinterpret_cast<volatile int*>(sh_fail) == 0;
}

template <typename T>
struct Pack;  // 16-byte packet helpers
template <>
struct Pack<float> {
  static constexpr int N = 4;
  __device__ static void to_f(const uint4& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
  }
  __device__ static uint4 from_f(const float (&v)[4]) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
  }
};
template <>
struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void to_f(const uint4& r, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ static uint4 from_f(const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return r;
  }
};

__device__ __forceinline__ uint4 ld_peer(const void* p) {
  // peer data is written by other GPUs between launches: bypass L1, keep it volatile
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
__device__ __forceinline__ void st_peer(void* p, const uint4& r) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
}

struct Weights {
  float w[FB_MAX_RANKS];
};

// ---------------------------------------------------------------------------------------------
// two-shot all-reduce, in place on the symmetric buffer
// ---------------------------------------------------------------------------------------------
template <typename T, int W>
__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(SymmCtx c, long long byte_off, long long n, Weights wts) {
  __shared__ int sh_fail;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  constexpr int E = Pack<T>::N;
  const long long nvec = n / E;                       // caller guarantees n % E == 0
  const long long per = (nvec + W - 1) / W;           // vectors per shard
  const long long v0 = per * c.rank;
  const long long v1 = (v0 + per < nvec) ? v0 + per : nvec;

  if (symm_block_barrier(c, epoch, &sh_fail)) {
    // U vectors per thread per trip: U*W independent 16-byte peer loads are in flight per thread,
    // which is what it takes to cover the NVLink round trip at full rate.
    constexpr int U = (W <= 2) ? 8 : (W <= 4 ? 4 : 2);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = v0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < v1; i0 += stride * U) {
      uint4 raw[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < v1) {
#pragma unroll
          for (int p = 0; p < W; ++p) {
            const int src = (c.rank + p) % W;  // stagger so peers are not all hit in the same order
            raw[u][p] = ld_peer(static_cast<const char*>(c.data[src]) + byte_off + i * 16);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < v1) {
          float acc[E];
#pragma unroll
          for (int j = 0; j < E; ++j) acc[j] = 0.f;
#pragma unroll
          for (int p = 0; p < W; ++p) {
            const int src = (c.rank + p) % W;
            float v[E];
            Pack<T>::to_f(raw[u][p], v);
            const float w = wts.w[src];
#pragma unroll
            for (int j = 0; j < E; ++j) acc[j] += v[j] * w;
          }
          const uint4 out = Pack<T>::from_f(acc);
#pragma unroll
          for (int p = 0; p < W; ++p) {
            const int dst = (c.rank + p) % W;
            st_peer(static_cast<char*>(c.data[dst]) + byte_off + i * 16, out);
          }
        }
      }
    }
    symm_block_barrier(c, epoch, &sh_fail);
  }
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}


// ---------------------------------------------------------------------------------------------
// NVLS (multimem) primitives and kernels
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Multimem;
template <>
struct Multimem<float> {
  __device__ static uint4 ld_reduce(const void* mc) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    return r;
  }
};
template <>
struct Multimem<__nv_bfloat16> {
  __device__ static uint4 ld_reduce(const void* mc) {   // eight bf16 values, accumulated in fp32 by the switch
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    return r;
  }
};
__device__ __forceinline__ void multimem_st(void* mc, const uint4& r) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
}

// In-place all-reduce: rank r owns shard r, asks the switch for the sum of that shard over all
// GPUs, scales it and multicasts the result into every GPU's buffer.
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_nvls_kernel(SymmCtx c, long long byte_off, long long n, float scale) {
  __shared__ int sh_fail;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  constexpr int E = Pack<T>::N;
  const long long nvec = n / E;
  const long long per = (nvec + c.world - 1) / c.world;
  const long long v0 = per * c.rank;
  const long long v1 = (v0 + per < nvec) ? v0 + per : nvec;
  if (symm_block_barrier(c, epoch, &sh_fail)) {
    constexpr int U = 8;      // independent switch reductions in flight per thread
    char* base = c.mc + byte_off;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = v0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < v1; i0 += stride * U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < v1) raw[u] = Multimem<T>::ld_reduce(base + (i0 + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * stride < v1) {
          float v[E];
          Pack<T>::to_f(raw[u], v);
#pragma unroll
          for (int j = 0; j < E; ++j) v[j] *= scale;
          multimem_st(base + (i0 + u * stride) * 16, Pack<T>::from_f(v));
        }
      }
    }
    symm_block_barrier(c, epoch, &sh_fail);
  }
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}

// Broadcast from `root`: the root reads its own bytes and multicasts them; each byte leaves the
// root once and the switch replicates it.
__global__ void __launch_bounds__(512)
broadcast_nvls_kernel(SymmCtx c, long long byte_off, long long nbytes, int root) {
  __shared__ int sh_fail;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  if (symm_block_barrier(c, epoch, &sh_fail)) {
    if (c.rank == root) {
      constexpr int U = 8;
      const long long nvec = nbytes / 16;
      const char* src = static_cast<const char*>(c.data[root]) + byte_off;
      char* dst = c.mc + byte_off;
      const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
      for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * stride < nvec) raw[u] = *reinterpret_cast<const uint4*>(src + (i0 + u * stride) * 16);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * stride < nvec) multimem_st(dst + (i0 + u * stride) * 16, raw[u]);
      }
    }
    symm_block_barrier(c, epoch, &sh_fail);
  }
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}

// ---------------------------------------------------------------------------------------------
// one-shot all-reduce: out (local, any dtype) = sum_p w_p * in_p
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TO, int W>
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(SymmCtx c, long long byte_off, long long n, TO* __restrict__ out, Weights wts) {
  __shared__ int sh_fail;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  constexpr int E = Pack<TI>::N;
  const long long nvec = n / E;
  if (symm_block_barrier(c, epoch, &sh_fail)) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
      // canonical rank order: every rank must produce bit-identical sums
      uint4 raw[W];
#pragma unroll
      for (int p = 0; p < W; ++p) raw[p] = ld_peer(static_cast<const char*>(c.data[p]) + byte_off + i * 16);
      float acc[E];
#pragma unroll
      for (int j = 0; j < E; ++j) acc[j] = 0.f;
#pragma unroll
      for (int p = 0; p < W; ++p) {
        float v[E];
        Pack<TI>::to_f(raw[p], v);
        const float w = wts.w[p];
#pragma unroll
        for (int j = 0; j < E; ++j) acc[j] += v[j] * w;
      }
#pragma unroll
      for (int j = 0; j < E; ++j) VecIO<TO>::put(out + i * E + j, acc[j]);
    }
    // peers may overwrite their inputs once everybody has finished reading
    symm_block_barrier(c, epoch, &sh_fail);
  }
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}

// ---------------------------------------------------------------------------------------------
// parameter averaging + lerp + divergence partials (fp32 master weights)
// ---------------------------------------------------------------------------------------------
// c.data[]  : peer pointers to the fp32 parameter buffers
// stage[]   : peer pointers to fp32 staging buffers of the same size
// partial   : 2 * gridDim.x floats (local scratch); out2 = {sum (post-pre)^2, sum post^2}
template <int W, bool NVLS>
__global__ void __launch_bounds__(512)
param_average_kernel(SymmCtx c, SymmCtx stage, long long n, Weights wts, float alpha,
                     __nv_bfloat16* __restrict__ p16, float* __restrict__ partial, unsigned int* __restrict__ done_counter,
                     float* __restrict__ out2) {
  __shared__ int sh_fail;
  __shared__ float scratch[32];
  __shared__ bool is_last;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  const long long nvec = n / 4;
  const int world = NVLS ? c.world : W;
  const long long per = (nvec + world - 1) / world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  float d2 = 0.f, n2 = 0.f;

  if (symm_block_barrier(c, epoch, &sh_fail)) {
    if constexpr (NVLS) {
      // the switch sums shard `rank` of every GPU's parameters; the mean goes to every staging buffer
      const long long v0 = per * c.rank;
      const long long v1 = (v0 + per < nvec) ? v0 + per : nvec;
      constexpr int U = 8;
      const float inv = wts.w[0];
      for (long long i0 = v0 + tid; i0 < v1; i0 += stride * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * stride < v1) raw[u] = Multimem<float>::ld_reduce(c.mc + (i0 + u * stride) * 16);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * stride < v1) {
            float v[4];
            Pack<float>::to_f(raw[u], v);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] *= inv;
            multimem_st(stage.mc + (i0 + u * stride) * 16, Pack<float>::from_f(v));
          }
        }
      }
    } else {
      const long long v0 = per * c.rank;
      const long long v1 = (v0 + per < nvec) ? v0 + per : nvec;
      // U * W independent 16-byte peer loads in flight per thread (see the all-reduce kernel)
      constexpr int U = (W <= 2) ? 8 : (W <= 4 ? 4 : 2);
      for (long long i0 = v0 + tid; i0 < v1; i0 += stride * U) {
        uint4 raw[U][W];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < v1) {
#pragma unroll
            for (int p = 0; p < W; ++p) raw[u][p] = ld_peer(static_cast<const char*>(c.data[(c.rank + p) % W]) + i * 16);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < v1) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int p = 0; p < W; ++p) {
              float v[4];
              Pack<float>::to_f(raw[u][p], v);
              const float w = wts.w[(c.rank + p) % W];
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[j] += v[j] * w;
            }
            const uint4 o = Pack<float>::from_f(acc);
#pragma unroll
            for (int p = 0; p < W; ++p) st_peer(static_cast<char*>(stage.data[(c.rank + p) % W]) + i * 16, o);
          }
        }
      }
    }
    if (symm_block_barrier(c, epoch, &sh_fail)) {
      // block b of every rank wrote the vectors {v0(s) + b*blockDim + t + k*stride} of shard s:
      // exactly those are complete in my staging buffer now, and only those are touched below.
      const char* st_local = static_cast<const char*>(stage.data[c.rank]);
      float* w_local = static_cast<float*>(c.data[c.rank]);
      for (int s = 0; s < world; ++s) {
        const long long v0 = per * s;
        const long long v1 = (v0 + per < nvec) ? v0 + per : nvec;
        constexpr int U2 = 4;
        for (long long i0 = v0 + tid; i0 < v1; i0 += stride * U2) {
          uint4 ra[U2], ro[U2];
#pragma unroll
          for (int u = 0; u < U2; ++u) {
            const long long i = i0 + u * stride;
            if (i < v1) {
              ra[u] = ld_peer(st_local + i * 16);
              ro[u] = *reinterpret_cast<const uint4*>(w_local + i * 4);
            }
          }
#pragma unroll
          for (int u = 0; u < U2; ++u) {
            const long long i = i0 + u * stride;
            if (i < v1) {
              float avg[4], old[4], nw[4];
              Pack<float>::to_f(ra[u], avg);
              Pack<float>::to_f(ro[u], old);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                nw[j] = old[j] + alpha * (avg[j] - old[j]);
                const float d = nw[j] - old[j];
                d2 += d * d;
                n2 += nw[j] * nw[j];
              }
              *reinterpret_cast<uint4*>(w_local + i * 4) = Pack<float>::from_f(nw);
              if (p16) {
                __nv_bfloat162 h[2] = {__floats2bfloat162_rn(nw[0], nw[1]), __floats2bfloat162_rn(nw[2], nw[3])};
                *reinterpret_cast<uint2*>(p16 + i * 4) = *reinterpret_cast<uint2*>(h);
              }
            }
          }
        }
      }
    }
  }
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
  // fold the divergence partials; the last block to finish writes the two totals
  d2 = block_sum(d2, scratch);
  n2 = block_sum(n2, scratch);
  if (threadIdx.x == 0) {
    partial[2 * blockIdx.x] = d2;
    partial[2 * blockIdx.x + 1] = n2;
    __threadfence();
    const unsigned int prev = atomicAdd(done_counter, 1u);
    is_last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    float a = 0.f, b = 0.f;
    for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += blockDim.x) {
      a += reinterpret_cast<volatile float*>(partial)[2 * i];
      b += reinterpret_cast<volatile float*>(partial)[2 * i + 1];
    }
    a = block_sum(a, scratch);
    b = block_sum(b, scratch);
    if (threadIdx.x == 0) {
      out2[0] = a;
      out2[1] = b;
      *done_counter = 0;  // ready for the next launch / graph replay
    }
  }
}

// ---------------------------------------------------------------------------------------------
// broadcast from `root`
// ---------------------------------------------------------------------------------------------
// Two ranks (or a message too small to matter): every other rank pulls the root's bytes. More ranks:
// the root's NVLink egress would be shared by W-1 pullers, so the message is cut in W shards; rank r
// first pulls shard r from the root (the root sends each byte once), then every rank pulls the other
// shards from their owners, which spreads that traffic over all links (scatter + all-gather).
// Block b of every rank copies the same element set of a shard, so the per-block barrier between the
// phases is enough.
__device__ __forceinline__ void pull_range(const char* src, char* dst, long long v0, long long v1, long long tid, long long stride) {
  constexpr int U = 8;      // independent peer loads in flight per thread
  for (long long i0 = v0 + tid; i0 < v1; i0 += stride * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < v1) raw[u] = ld_peer(src + (i0 + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < v1) *reinterpret_cast<uint4*>(dst + (i0 + u * stride) * 16) = raw[u];
  }
}

__global__ void __launch_bounds__(512)
broadcast_kernel(SymmCtx c, long long byte_off, long long nbytes, int root) {
  __shared__ int sh_fail;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  const long long nvec = nbytes / 16;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  char* dst = static_cast<char*>(c.data[c.rank]) + byte_off;
  const bool sharded = c.world > 2 && nbytes >= (1 << 20);
  if (symm_block_barrier(c, epoch, &sh_fail)) {
    if (!sharded) {
      if (c.rank != root) pull_range(static_cast<const char*>(c.data[root]) + byte_off, dst, 0, nvec, tid, stride);
      symm_block_barrier(c, epoch, &sh_fail);
    } else {
      const long long per = (nvec + c.world - 1) / c.world;
      if (c.rank != root) {
        const long long v0 = per * c.rank, v1 = (v0 + per < nvec) ? v0 + per : nvec;
        pull_range(static_cast<const char*>(c.data[root]) + byte_off, dst, v0, v1, tid, stride);
      }
      if (symm_block_barrier(c, epoch, &sh_fail)) {
        if (c.rank != root) {
          for (int k = 1; k < c.world; ++k) {
            const int s = (c.rank + k) % c.world;       // staggered so the owners are not all hit in the same order
            const long long v0 = per * s, v1 = (v0 + per < nvec) ? v0 + per : nvec;
            pull_range(static_cast<const char*>(c.data[s]) + byte_off, dst, v0, v1, tid, stride);
          }
        }
        symm_block_barrier(c, epoch, &sh_fail);
      }
    }
  }
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}

// Barrier only (used to fence host-driven phases, and by the tests to exercise the timeout path).
__global__ void barrier_kernel(SymmCtx c) {
  __shared__ int sh_fail;
  if (threadIdx.x == 0) sh_fail = 0;
  uint32_t epoch = c.epochs[blockIdx.x];
  symm_block_barrier(c, epoch, &sh_fail);
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}

static SymmCtx make_ctx(const fb_symm_ctx* h) {
  SymmCtx c;
  for (int i = 0; i < FB_MAX_RANKS; ++i) {
    c.data[i] = i < h->world ? h->data[i] : nullptr;
    c.sig[i] = i < h->world ? static_cast<uint32_t*>(h->sig[i]) : nullptr;
  }
  c.epochs = static_cast<uint32_t*>(h->epochs);
  c.abort = static_cast<const int*>(h->abort);
  c.status = static_cast<int*>(h->status);
  c.status_dev = static_cast<int*>(h->status_dev);
  c.timeout_ns = h->timeout_ns > 0 ? h->timeout_ns : 2000000000LL;
  c.mc = static_cast<char*>(h->mc);
  c.rank = h->rank;
  c.world = h->world;
  return c;
}

static Weights make_weights(const fb_symm_ctx* h, const float* weights) {
  Weights w;
  for (int i = 0; i < FB_MAX_RANKS; ++i) w.w[i] = (i < h->world) ? (weights ? weights[i] : 1.0f / h->world) : 0.f;
  return w;
}

static int clamp_blocks(int blocks) {
  if (blocks < 1) blocks = 1;
  if (blocks > FB_MAX_BLOCKS) blocks = FB_MAX_BLOCKS;
  return blocks;
}

}  // namespace fb

#define FB_DISPATCH_WORLD(W, ...) \
  switch (W) {                    \
    case 1: { constexpr int kW = 1; __VA_ARGS__; break; } \
    case 2: { constexpr int kW = 2; __VA_ARGS__; break; } \
    case 3: { constexpr int kW = 3; __VA_ARGS__; break; } \
    case 4: { constexpr int kW = 4; __VA_ARGS__; break; } \
    case 5: { constexpr int kW = 5; __VA_ARGS__; break; } \
    case 6: { constexpr int kW = 6; __VA_ARGS__; break; } \
    case 7: { constexpr int kW = 7; __VA_ARGS__; break; } \
    case 8: { constexpr int kW = 8; __VA_ARGS__; break; } \
    default: return -5;           \
  }

// weights: host array of `world` floats (nullptr = 1/world each). n = element count, multiple of 16 bytes.
extern "C" int fb_allreduce(const fb_symm_ctx* h, long long byte_off, long long n, int is_bf16, const float* weights,
                            int blocks, void* stream) {
  using namespace fb;
  if (n <= 0) return 0;
  if ((n * (is_bf16 ? 2 : 4)) % 16 || byte_off % 16) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SymmCtx c = make_ctx(h);
  Weights w = make_weights(h, weights);
  blocks = clamp_blocks(blocks);
  // 512-thread blocks on few SMs: measured on 2 x B200 under a BERT-base step, spreading the same threads over
  // 96..222 blocks of 128 threads slowed the overlapped GEMMs more (7.29..7.85 ms per step against 7.22).
  const int threads = 512;
  if (h->mc && !weights && h->world > 1) {
    // equal weights: the switch does the sum (fp32 accumulate), the kernel applies 1/world
    const float scale = 1.0f / static_cast<float>(h->world);
    if (is_bf16) allreduce_nvls_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(c, byte_off, n, scale);
    else allreduce_nvls_kernel<float><<<blocks, threads, 0, st>>>(c, byte_off, n, scale);
    return static_cast<int>(cudaGetLastError());
  }
  FB_DISPATCH_WORLD(h->world,
    if (is_bf16) allreduce_twoshot_kernel<__nv_bfloat16, kW><<<blocks, threads, 0, st>>>(c, byte_off, n, w);
    else allreduce_twoshot_kernel<float, kW><<<blocks, threads, 0, st>>>(c, byte_off, n, w));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_allreduce_oneshot(const fb_symm_ctx* h, long long byte_off, long long n, int in_bf16, void* out,
                                    int out_bf16, const float* weights, int blocks, void* stream) {
  using namespace fb;
  if (n <= 0) return 0;
  if ((n * (in_bf16 ? 2 : 4)) % 16 || byte_off % 16) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SymmCtx c = make_ctx(h);
  Weights w = make_weights(h, weights);
  blocks = clamp_blocks(blocks);
  FB_DISPATCH_WORLD(h->world,
    if (in_bf16 && out_bf16) allreduce_oneshot_kernel<__nv_bfloat16, __nv_bfloat16, kW><<<blocks, 512, 0, st>>>(c, byte_off, n, static_cast<__nv_bfloat16*>(out), w);
    else if (in_bf16) allreduce_oneshot_kernel<__nv_bfloat16, float, kW><<<blocks, 512, 0, st>>>(c, byte_off, n, static_cast<float*>(out), w);
    else if (out_bf16) allreduce_oneshot_kernel<float, __nv_bfloat16, kW><<<blocks, 512, 0, st>>>(c, byte_off, n, static_cast<__nv_bfloat16*>(out), w);
    else allreduce_oneshot_kernel<float, float, kW><<<blocks, 512, 0, st>>>(c, byte_off, n, static_cast<float*>(out), w));
  return static_cast<int>(cudaGetLastError());
}

// params / staging are fp32, n % 4 == 0. partial: 2*blocks floats; counter: one zeroed uint; out2: 2 floats.
extern "C" int fb_param_average(const fb_symm_ctx* params, const fb_symm_ctx* staging, long long n, const float* weights,
                                float alpha, void* p16, float* partial, unsigned int* counter, float* out2, int blocks,
                                void* stream) {
  using namespace fb;
  if (n <= 0) return 0;
  if (n % 4) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SymmCtx c = make_ctx(params);
  SymmCtx s = make_ctx(staging);
  Weights w = make_weights(params, weights);
  blocks = clamp_blocks(blocks);
  if (params->mc && staging->mc && !weights && params->world > 1) {
    param_average_kernel<1, true><<<blocks, 512, 0, st>>>(c, s, n, w, alpha, static_cast<__nv_bfloat16*>(p16), partial, counter, out2);
    return static_cast<int>(cudaGetLastError());
  }
  FB_DISPATCH_WORLD(params->world,
    param_average_kernel<kW, false><<<blocks, 512, 0, st>>>(c, s, n, w, alpha, static_cast<__nv_bfloat16*>(p16), partial, counter, out2));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_broadcast(const fb_symm_ctx* h, long long byte_off, long long nbytes, int root, int blocks, void* stream) {
  using namespace fb;
  if (nbytes <= 0) return 0;
  if (nbytes % 16 || byte_off % 16) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SymmCtx c = make_ctx(h);
  blocks = clamp_blocks(blocks);
  if (h->mc && h->world > 1 && nbytes >= (1 << 16)) {
    broadcast_nvls_kernel<<<blocks, 512, 0, st>>>(c, byte_off, nbytes, root);
    return static_cast<int>(cudaGetLastError());
  }
  broadcast_kernel<<<blocks, 512, 0, st>>>(c, byte_off, nbytes, root);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fb_symm_barrier(const fb_symm_ctx* h, int blocks, void* stream) {
  using namespace fb;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SymmCtx c = make_ctx(h);
  barrier_kernel<<<clamp_blocks(blocks), 32, 0, st>>>(c);
  return static_cast<int>(cudaGetLastError());
}
