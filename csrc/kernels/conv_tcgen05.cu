// Convolution filter gradient on the tensor cores, for channels-last (N-H-W-C) bf16 tensors.
//
// Replaces the filter-gradient half of `torch::conv2d`'s backward (flodl-sys/ops_nn.cpp:17-60, cuDNN)
// for the CIFAR-ResNet shapes: 3x3 / 1x1 filters, stride 1 or 2, 16..64 channels, where the library
// kernels spend 15-20 us per layer on problems whose data fits in L2 many times over.
//
//   dW[co][r][s][ci] += sum over output pixels p of  dY[p][co] * X[p*stride + (r,s) - pad][ci]
//
// As a GEMM per filter tap: M = Co, N = Ci, K = pixels. Both operands are "MN-major" for the MMA
// (the reduction index, the pixel, is the slow index of both N-H-W-C tensors), which is what the
// 128-byte-swizzled K-by-64 panels of this file's shared-memory tiles hold:
//   * A tile  = 64 output pixels x 64 channels of dY (channels beyond Co are zero-filled by TMA's
//     out-of-bounds rule), presented to the MMA as M = 128 with a second, permanently zero panel, so
//     accumulator row i sits in TMEM lane i exactly as in the GEMM kernel;
//   * B tiles = for every tap, the same 64 pixels of X shifted by the tap's offset: a 4-D TMA box
//     whose start coordinate may be negative (zero fill = the convolution's padding) and whose
//     traversal stride is the convolution stride; 64 channels wide, channels beyond Ci zero-filled.
// One CTA walks a strided subset of the 64-pixel patches, accumulating all taps side by side in
// TMEM (tap t in columns [t*Ci, (t+1)*Ci)); at the end the 4 epilogue warps move the accumulators to
// shared memory and add them to the fp32 gradient with bulk reduce-add copies, so any number of CTAs
// can share one layer. Filters whose taps do not fit 512 TMEM columns (Ci = 64) take two passes.
//
// Every wait is bounded (ptx_sm100.cuh); on expiry the kernel records a status and leaves.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>

#include "../include/flodl_b200.h"
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fb {

void ensure_thread_context();   // gemm_tcgen05.cu

namespace {

constexpr int kPix = 64;                  // pixels per K chunk
constexpr int kPanel = kPix * 128;        // bytes of one 64-pixel x 64-channel bf16 panel
constexpr int kConvThreads = 32 * 6;      // TMA warp, MMA warp, 4 epilogue warps
constexpr int kMaxStages = 8;
constexpr int kMaxTapsPerPass = 9;
constexpr int kPipeBytes = 168 * 1024;    // shared memory given to the stage ring

struct WgradParams {
  int N, Ho, Wo, Ci, Co;
  int kh, kw, stride, pad;
  int hbox, wbox;          // the 64-pixel patch of the OUTPUT grid: hbox * wbox == 64
  int taps_per_pass, passes;
  int chunks;              // N * (Ho / hbox) * (Wo / wbox)
  // B tiles hold exactly Ci channels per pixel: 32-, 64- or 128-byte rows with the matching swizzle
  int b_bytes, b_layout, b_sbo, b_kstep;
  int stages, stage_bytes, zero_off, bars_off;
  float* dw;               // [Co][kh][kw][Ci] fp32, accumulated into
  int* status;
};

// Division by a run-time constant as multiply-high + shifts (Granlund-Montgomery round-up form,
// exact for every 32-bit dividend when the divisor is at least 2). The loader threads decode a pixel
// index per 16-byte copy; with hardware division those chains of ~100 dependent instructions were
// what bounded the kernels below.
struct FastDiv {
  uint32_t m, sh;
  __device__ __forceinline__ uint32_t div(uint32_t n) const {
    const uint32_t t = __umulhi(m, n);
    return (t + ((n - t) >> 1)) >> sh;
  }
};
inline FastDiv make_fastdiv(uint32_t d) {   // d >= 2
  uint32_t l = 0;
  while ((1ull << l) < d) ++l;
  FastDiv f;
  f.m = static_cast<uint32_t>(((1ull << 32) * ((1ull << l) - d)) / d + 1);
  f.sh = l - 1;
  return f;
}

// UMMA layout code of the swizzle whose span is one `channels`-wide bf16 row (128, 64 or 32 bytes)
inline int swizzle_code(int channels) { return channels == 64 ? 2 : channels == 32 ? 4 : 6; }

__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}

// UMMA shared-memory descriptor with an explicit swizzle mode (2 = 128 B, 4 = 64 B, 6 = 32 B).
__device__ __forceinline__ uint64_t conv_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout) << 61;
  return d;
}

// Column sums of a 32-lane x 16-value tile by recursive halving: each exchange step halves the columns
// a lane still carries, and after the last one lane l returns the total of column stat_column(l)
// (both lanes of a pair return the same column). 16 shuffles instead of the 80 of a per-column butterfly.
__device__ __forceinline__ float colsum16(float (&v)[16], int lane) {
#pragma unroll
  for (int half = 8, off = 16; half >= 1; half >>= 1, off >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = up ? v[i] : v[i + half];
      const float keep = up ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}
// the column whose total colsum16 leaves in lane `lane`
__device__ __forceinline__ int stat_column(int lane) {
  return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
}

__device__ __forceinline__ void tma4(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
                   smem_u32(dst)),
               "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

__global__ void __launch_bounds__(kConvThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmDy, const __grid_constant__ CUtensorMap tmX, const WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = p.stage_bytes;                            // A panel (8 KB) + one B tile per tap
  const int kConvStages = p.stages;
  uint8_t* bars_mem = smem + p.bars_off;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bars_mem);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_bar = empty_bar + kMaxStages;                       // accumulators of a pass complete
  uint64_t* drained_bar = acc_bar + 1;                              // epilogue has read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drained_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.kh * p.kw;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kConvStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    mbar_init(drained_bar, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmDy);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  // Rows 64..127 of A come from one zero panel shared by all stages (each stage's descriptor reaches
  // it through its own leading-dimension offset). Whatever it holds only ever reaches accumulator
  // rows 64..127, which nobody reads.
  {
    uint4* z = reinterpret_cast<uint4*>(smem + p.zero_off);
    for (int i = threadIdx.x; i < kPanel / 16; i += kConvThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  const int per_row = p.Wo / p.wbox, per_img = (p.Ho / p.hbox) * per_row;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int pass = 0; pass < p.passes && ok; ++pass) {
        const int t0 = pass * p.taps_per_pass;
        const int nt = min(p.taps_per_pass, taps - t0);
        if (pass > 0) {   // the epilogue stages its results in the pipeline buffers: wait until it is done with them
          ok = mbar_wait(drained_bar, (pass - 1) & 1, abort_flag, p.status, kStatusWaitEpi);
          if (!ok) break;
        }
        for (int c = blockIdx.x; c < p.chunks && ok; c += gridDim.x) {
          ok = mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kStatusWaitEmpty);
          if (!ok) break;
          const int n = c / per_img, r = c - n * per_img;
          const int ho0 = (r / per_row) * p.hbox, wo0 = (r % per_row) * p.wbox;
          uint8_t* sa = smem + s * stage_bytes;
          mbar_expect_tx(&full_bar[s], kPanel + nt * p.b_bytes);
          tma4(sa, &tmDy, &full_bar[s], 0, wo0, ho0, n);
          for (int t = 0; t < nt; ++t) {
            const int tap = t0 + t, dy = tap / p.kw, dx = tap - dy * p.kw;
            tma4(sa + kPanel + t * p.b_bytes, &tmX, &full_bar[s], 0, wo0 * p.stride + dx - p.pad, ho0 * p.stride + dy - p.pad, n);
          }
          if (++s == kConvStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, p.Ci, 1, 1);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int pass = 0; pass < p.passes && ok; ++pass) {
        const int t0 = pass * p.taps_per_pass;
        const int nt = min(p.taps_per_pass, taps - t0);
        if (pass > 0) {   // the epilogue must have emptied the accumulators of the previous pass
          ok = mbar_wait(drained_bar, (pass - 1) & 1, abort_flag, p.status, kStatusWaitEpi);
          if (!ok) break;
          tc_fence_after_sync();
        }
        bool first = true;
        for (int c = blockIdx.x; c < p.chunks && ok; c += gridDim.x) {
          ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, kStatusWaitFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * stage_bytes);
          const uint32_t a_lbo = smem_u32(smem + p.zero_off) - sa;      // panel 0 -> the shared zero panel
          for (int t = 0; t < nt; ++t) {
            const uint32_t sb = sa + kPanel + t * p.b_bytes;
#pragma unroll
            for (int k4 = 0; k4 < kPix / 16; ++k4) {
              const uint64_t da = conv_desc(sa + k4 * 2048, a_lbo, 1024, 2);
              const uint64_t db = conv_desc(sb + k4 * p.b_kstep, p.b_bytes, p.b_sbo, p.b_layout);
              umma_bf16<1>(tmem_base + t * p.Ci, da, db, idesc, (first && k4 == 0) ? 0u : 1u);
            }
          }
          first = false;
          umma_commit(&empty_bar[s]);
          if (++s == kConvStages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(acc_bar);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int q = warp & 3;                       // TMEM lane quarter of this warp
    const int co = q * 32 + lane;
    float* stage = reinterpret_cast<float*>(smem);  // pipeline buffers are idle by the time a pass completes
    bool ok = true;
    for (int pass = 0; pass < p.passes && ok; ++pass) {
      const int t0 = pass * p.taps_per_pass;
      const int nt = min(p.taps_per_pass, taps - t0);
      ok = mbar_wait(acc_bar, pass & 1, abort_flag, p.status, kStatusWaitAccum);
      if (!ok) break;
      tc_fence_after_sync();
      const int row_floats = nt * p.Ci;            // one output channel's slice for this pass
      if (q * 32 < p.Co) {
        for (int col = 0; col < row_floats; col += 16) {
          uint32_t v[16];
          tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + col, v);
          tmem_ld_wait();
          if (co < p.Co) {
            float4* dst = reinterpret_cast<float4*>(stage + static_cast<size_t>(co) * row_floats + col);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                   __uint_as_float(v[4 * j + 3]));
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (co < p.Co) {
          bulk_reduce_add_f32(p.dw + (static_cast<size_t>(co) * taps + t0) * p.Ci, stage + static_cast<size_t>(co) * row_floats,
                              static_cast<uint32_t>(row_floats * 4));
          tma_store_commit();
        }
      }
      tc_fence_before_sync();
      if (p.passes > 1) {
        // the staging area doubles as pipeline memory: the copies must have read it before the
        // producer of the next pass may overwrite it
        tma_store_wait_read();
        __syncwarp();
      }
      if (lane == 0) mbar_arrive(drained_bar);
    }
    tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// Forward convolution and data gradient: out[p][n] = sum over taps t and channels k of
//     in[p * stride + sign * ((r,s)_t - pad)][k] * Wt[k][n]
// with (in, K, N, sign) = (X, Ci, Co, +1) for the forward pass and (dY, Co, Ci, -1) for the stride-1
// data gradient. M = 128 output pixels per tile (one or two TMA boxes, each inside one image), one
// MMA group per tap accumulating into the same TMEM columns; the filter stays in shared memory for
// the CTA's lifetime ([Co][Ci] per tap: K-major B for the forward pass, the same bytes read as
// MN-major B for the data gradient). Persistent CTAs, two accumulator buffers so the epilogue of a
// tile overlaps the next tile's loads and MMAs. Output rows leave as bf16 straight from registers:
// a tile of full-width image rows is one contiguous block of N-H-W-C memory.
struct FwdParams {
  int Kc, Nout, Ci, taps, kw, stride, pad, sign;
  int wbox, hbox, nbox;        // nbox boxes of wbox x hbox output pixels make one 128-pixel tile
  int per_img;                 // boxes per image
  int images;
  long long pixels;            // N * Ho * Wo
  int tiles;
  int a_bytes, a_layout, a_sbo;             // one tap's A tile: 128 rows of Kc channels
  int w_bytes, w_layout, w_sbo, w_kstep, b_mn;
  int stages, ring_off, bars_off;
  __nv_bfloat16* out;
  float* stats;                // optional [2][Nout]: per-channel sum and sum of squares, added to
  int* status;
};

constexpr int kFwdMaxStages = 12;

__global__ void __launch_bounds__(kConvThreads, 1)
conv_fwd_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem + p.ring_off;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.bars_off);
  uint64_t* empty_bar = full_bar + kFwdMaxStages;
  uint64_t* acc_full = empty_bar + kFwdMaxStages;     // [2]
  uint64_t* acc_empty = acc_full + 2;                 // [2]
  uint64_t* w_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat_smem = reinterpret_cast<float*>(smem + p.bars_off + 512);   // [4 warps][2][Nout]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int acc_cols = p.Nout <= 32 ? 32 : p.Nout <= 64 ? 64 : p.Nout <= 128 ? 128 : 256;   // columns of one buffer

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    mbar_init(w_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmIn);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 2 * acc_cols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(w_bar, p.taps * p.w_bytes);
      for (int t = 0; t < p.taps; ++t) tma_load_2d(smem + t * p.w_bytes, &tmW, w_bar, t * p.Ci, 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const int box_bytes = p.a_bytes / p.nbox;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
        for (int t = 0; t < p.taps && ok; ++t) {
          ok = mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, kStatusWaitEmpty);
          if (!ok) break;
          const int dy = t / p.kw, dx = t - dy * p.kw;
          uint8_t* sa = ring + s * p.a_bytes;
          mbar_expect_tx(&full_bar[s], p.a_bytes);
          for (int b = 0; b < p.nbox; ++b) {
            const int c = tile * p.nbox + b;
            const int n = c / p.per_img, r = c - n * p.per_img;      // n may reach `images`: the box is then all zero fill
            const int ho0 = r * p.hbox;
            tma4(sa + b * box_bytes, &tmIn, &full_bar[s], 0, p.sign * (dx - p.pad), ho0 * p.stride + p.sign * (dy - p.pad), n);
          }
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, p.Nout, 0, p.b_mn);
      bool ok = mbar_wait(w_bar, 0, abort_flag, p.status, kStatusWaitFull);
      int s = 0, it = 0;
      uint32_t ph = 0;
      const uint32_t w0 = smem_u32(smem);
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        ok = mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, kStatusWaitEpi);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * acc_cols;
        for (int t = 0; t < p.taps && ok; ++t) {
          ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, kStatusWaitFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(ring + s * p.a_bytes);
          const uint32_t sw = w0 + t * p.w_bytes;
          for (int k = 0; k < p.Kc / 16; ++k) {
            const uint64_t da = conv_desc(sa + k * 32, 16, p.a_sbo, p.a_layout);
            const uint64_t db = conv_desc(sw + k * p.w_kstep, 16, p.w_sbo, p.w_layout);
            umma_bf16<1>(d, da, db, idesc, (t == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int q = warp & 3;
    const int row = q * 32 + lane;
    float* my_stats = stat_smem + q * 2 * p.Nout;
    float acc1[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};   // per 16-column group: this lane's column
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      ok = mbar_wait(&acc_full[buf], (it >> 1) & 1, abort_flag, p.status, kStatusWaitAccum);
      if (!ok) break;
      tc_fence_after_sync();
      const long long pix = static_cast<long long>(tile) * 128 + row;
      const bool live = pix < p.pixels;
      __nv_bfloat16* dst = p.out + pix * p.Nout;
      for (int col = 0; col < p.Nout; col += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * acc_cols + col, v);
        tmem_ld_wait();
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          pk[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        if (live) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + col);
          d4[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          d4[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        // statistics of the ROUNDED outputs (what the normalisation that follows will read);
        // rows past the end hold zeros (zero-filled loads), so they add nothing
        if (p.stats) {
          float f[16], f2[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const __nv_bfloat162 hh = *reinterpret_cast<const __nv_bfloat162*>(&pk[j >> 1]);
            f[j] = (j & 1) ? __high2float(hh) : __low2float(hh);
            f2[j] = f[j] * f[j];
          }
          const float t1 = colsum16(f, lane), t2 = colsum16(f2, lane);
#pragma unroll
          for (int g = 0; g < 4; ++g)
            if (col == 16 * g) { acc1[g] += t1; acc2[g] += t2; }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (p.stats && !(lane & 1)) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
        if (16 * g < p.Nout) {
          my_stats[16 * g + stat_column(lane)] = acc1[g];
          my_stats[p.Nout + 16 * g + stat_column(lane)] = acc2[g];
        }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (p.stats && warp > 1 && *abort_flag == 0) {
    // fold the four warps' sums: one atomic per channel and CTA
    for (int i = threadIdx.x - 2 * 32; i < 2 * p.Nout; i += 128)
      atomicAdd(p.stats + i, (stat_smem[i] + stat_smem[2 * p.Nout + i]) + (stat_smem[4 * p.Nout + i] + stat_smem[6 * p.Nout + i]));
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 2 * acc_cols);
  }
}

// ------------------------------------------------------------------------------------------------
// 3x3, stride-1, "same" convolution (forward and data gradient) with the input tile loaded ONCE.
//
// The TMA formulation above fetches every tap's 128-pixel window separately, and with 16 or 32
// channels a pixel is a 32- or 64-byte row: the copy engine's per-row cost dominates (measured
// here: about 0.5 us per 128-row box, 9 boxes per tile). This kernel instead works in a padded linear pixel
// space q = n * (H+1) * (W+1) + h * (W+1) + w, where column W and row H of every image are zero
// padding shared with the neighbouring row / image. In that space the input of tap (r, s) for output
// q is simply q + (r-1) * (W+1) + (s-1): a constant shift. A tile is 128 consecutive q; its input is
// the 128 + 2 * (W+2) pixels around it, brought in by four producer warps with 16-byte cp.async copies
// (zero-filled where q is padding) into per-8-channel planes [pixel][8 channels]. Such a plane is the
// tensor core's un-swizzled K-major operand layout (8-row x 16-byte core matrices, 128 bytes apart
// along M, one plane apart along K), and because rows are 16 bytes apart every tap's operand is the
// SAME buffer read from a start address shifted by 16 bytes x the tap's shift. Outputs at padding
// positions are computed and dropped (6 % extra rows for 32-wide images, 27 % for 8-wide).
struct HaloParams {
  const __nv_bfloat16* in;
  __nv_bfloat16* out;
  int N, H, W, Kc, Nout, Ci, sign, b_mn;
  int pitch, img;              // W + 1, (H + 1) * (W + 1)
  int q_total, tiles;
  int halo, span;              // W + 2, 128 + 2 * halo
  int nch, nch_log2, plane_bytes, a_bytes;
  int groups;                  // accumulators per tile (see the kernel)
  int w_bytes, w_layout, w_sbo, w_kstep;
  int stages, ring_off, bars_off;
  FastDiv div_img, div_pitch;
  float* stats;
  int* status;
  long long* ts;               // optional timeline of CTA 0 (nanoseconds): see conv_fprop's `ts` argument
};

constexpr int kHaloThreads = 32 * 9;     // 4 producer warps, MMA warp, 4 epilogue warps
constexpr int kHaloMaxStages = 8;

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

#ifndef FB_TIMELINE
#define FB_TIMELINE 0      // the timeline is a tuning aid, compiled in only with -DFB_TIMELINE=1
#endif
__device__ __forceinline__ void ts_mark(long long* ts, int slot) {
  if (FB_TIMELINE && ts && blockIdx.x == 0 && slot < 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    ts[slot] = static_cast<long long>(t);
  }
}

__global__ void __launch_bounds__(kHaloThreads, 1)
conv3x3_halo_kernel(const __grid_constant__ CUtensorMap tmW, const HaloParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem + p.ring_off;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.bars_off);
  uint64_t* empty_bar = full_bar + kHaloMaxStages;
  uint64_t* acc_full = empty_bar + kHaloMaxStages;    // [2]
  uint64_t* acc_empty = acc_full + 2;                 // [2]
  uint64_t* w_bar = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat_smem = reinterpret_cast<float*>(smem + p.bars_off + 512);   // [4 warps][2][Nout]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Consecutive MMAs into one accumulator wait for each other (about 0.1 us each, measured), so the
  // nine taps of a tile are spread round-robin over `groups` accumulators that the epilogue adds up.
  const int groups = p.groups;
  const int acc_cols = groups * p.Nout;            // columns of one buffer (two buffers)

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    mbar_init(w_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    if (lane == 0) tma_prefetch_desc(&tmW);
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) ts_mark(p.ts, 0);
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) ts_mark(p.ts, 1);

  if (warp < 4) {
    // ---------------------------------------------------------------- producers (cp.async)
    // Each warp loads whole tiles on its own (tile i of this CTA belongs to warp i % 4) and keeps two
    // of them in flight, so up to eight tiles are on their way at any time. A warp publishes a tile after
    // its own copies have landed and a proxy fence has made them visible to the tensor core's
    // (async-proxy) reads.
    const int items = ((p.span + 7) / 8) * 8 * p.nch;       // the plane has room for the rounded-up pixels
    bool ok = true;
    int pending = -1;                        // stage of the tile whose copies are still in flight
    // A parity wait can only tell "one phase behind" from "caught up", so a warp's successive tiles must
    // not skip a whole turn of the ring: no more producer warps than stages.
    const int nprod = p.stages < 4 ? p.stages : 4;
    int it = warp;
    for (int tile = blockIdx.x + warp * gridDim.x; warp < nprod && tile < p.tiles && ok; tile += nprod * gridDim.x, it += nprod) {
      const int s = it % p.stages;
      const uint32_t parity = ((it / p.stages) & 1) ^ 1;
      if (pending >= 0) {
        // Never hold back a finished tile while waiting for a stage: with a short ring the stage this
        // warp wants next may only be released after the MMA warp has consumed the tile it has not
        // published yet.
        const bool ready = __shfl_sync(0xffffffffu, lane == 0 ? static_cast<int>(mbar_test(&empty_bar[s], parity)) : 0, 0) != 0;
        if (!ready) {
          cp_async_wait_group<0>();
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[pending]);
          pending = -1;
        }
      }
      ok = mbar_wait(&empty_bar[s], parity, abort_flag, p.status, kStatusWaitEmpty);
      if (!ok) break;
      const uint32_t base = smem_u32(ring + s * p.a_bytes);
      const int q_first = tile * 128 - p.halo;
#pragma unroll 4
      for (int i = lane; i < items; i += 32) {
        // 8 consecutive lanes take 8 consecutive pixels of one channel plane; no branches, so the
        // unrolled iterations overlap their address arithmetic
        const int c = (i >> 3) & (p.nch - 1), pix = ((i >> (3 + p.nch_log2)) << 3) + (i & 7);
        const int q = q_first + pix;
        const uint32_t qc = static_cast<uint32_t>(min(max(q, 0), p.q_total - 1));
        const uint32_t n = p.div_img.div(qc), r = qc - n * p.img;
        const uint32_t h = p.div_pitch.div(r), w = r - h * p.pitch;
        const bool valid = q >= 0 && q < p.q_total && h < static_cast<uint32_t>(p.H) && w < static_cast<uint32_t>(p.W);
        const uint32_t off = valid ? ((n * p.H + h) * p.W + w) * p.Kc + c * 8 : 0u;
        cp_async16_zfill(base + c * p.plane_bytes + pix * 16, p.in + off, valid ? 16u : 0u);
      }
      cp_async_commit();
      if (lane == 0 && it < 10) ts_mark(p.ts, 2 + it);
      if (pending >= 0) {
        cp_async_wait_group<1>();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[pending]);
      }
      pending = s;
    }
    cp_async_wait_group<0>();
    if (pending >= 0 && ok) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[pending]);
    }
  } else if (warp == 4) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      mbar_expect_tx(w_bar, 9 * p.w_bytes);
      for (int tp = 0; tp < 9; ++tp) tma_load_2d(smem + tp * p.w_bytes, &tmW, w_bar, tp * p.Ci, 0);
      const uint32_t idesc = make_idesc_bf16(128, p.Nout, 0, p.b_mn);
      bool ok = mbar_wait(w_bar, 0, abort_flag, p.status, kStatusWaitFull);
      int s = 0, it = 0;
      uint32_t ph = 0;
      const uint64_t db0 = conv_desc(smem_u32(smem), 16, p.w_sbo, p.w_layout);
      const int ksteps = p.Kc / 16, a_kstep16 = (2 * p.plane_bytes) >> 4, w_kstep16 = p.w_kstep >> 4;
      // per-tap constants: start-address offsets of both operands (16-byte units) and the accumulator group
      uint64_t a_off[9], b_off[9];
      uint32_t dcol[9];
#pragma unroll
      for (int tp = 0; tp < 9; ++tp) {
        a_off[tp] = static_cast<uint64_t>(static_cast<int64_t>(p.sign * ((tp / 3 - 1) * p.pitch + (tp % 3 - 1))));
        b_off[tp] = static_cast<uint64_t>((tp * p.w_bytes) >> 4);
        dcol[tp] = static_cast<uint32_t>((tp % p.groups) * p.Nout);
      }
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        ok = mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, kStatusWaitEpi);
        if (!ok) break;
        ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, kStatusWaitFull);
        if (!ok) break;
        if (it < 10) ts_mark(p.ts, 12 + it);
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * acc_cols;
        // descriptors differ from one instruction to the next only in their 16-byte-granular start
        // address field (bits 0..13), which never carries out of the field for these offsets
        const uint64_t da0 = conv_desc(smem_u32(ring + s * p.a_bytes) + p.halo * 16, p.plane_bytes, 128, 0);
        for (int k = 0; k < ksteps; ++k) {
#pragma unroll
          for (int tp = 0; tp < 9; ++tp)
            umma_bf16<1>(d + dcol[tp], da0 + a_off[tp] + static_cast<uint64_t>(k * a_kstep16), db0 + b_off[tp] + static_cast<uint64_t>(k * w_kstep16), idesc,
                         (k == 0 && tp < groups) ? 0u : 1u);
        }
        umma_commit(&empty_bar[s]);
        umma_commit(&acc_full[buf]);
        if (it < 10) ts_mark(p.ts, 22 + it);
        if (++s == p.stages) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int q4 = warp & 3;                      // TMEM lane quarter this warp may read
    const int row = q4 * 32 + lane;
    float* my_stats = stat_smem + q4 * 2 * p.Nout;
    float acc1[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};   // per 16-column group: this lane's column
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      ok = mbar_wait(&acc_full[buf], (it >> 1) & 1, abort_flag, p.status, kStatusWaitAccum);
      if (!ok) break;
      tc_fence_after_sync();
      if (warp == 5 && lane == 0 && it < 10) ts_mark(p.ts, 32 + it);
      const int q = tile * 128 + row;
      bool live = false;
      __nv_bfloat16* dst = p.out;
      if (q < p.q_total) {
        const uint32_t n = p.div_img.div(q), r = q - n * p.img;
        const uint32_t h = p.div_pitch.div(r), w = r - h * p.pitch;
        live = h < static_cast<uint32_t>(p.H) && w < static_cast<uint32_t>(p.W);
        dst = p.out + (static_cast<size_t>(n * p.H + h) * p.W + w) * p.Nout;
      }
      for (int col = 0; col < p.Nout; col += 16) {
        float f32[16];
        {
          uint32_t v[16];
          tmem_ld16(tmem_base + (static_cast<uint32_t>(q4 * 32) << 16) + buf * acc_cols + col, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) f32[j] = __uint_as_float(v[j]);
        }
        for (int g = 1; g < groups; ++g) {
          uint32_t v[16];
          tmem_ld16(tmem_base + (static_cast<uint32_t>(q4 * 32) << 16) + buf * acc_cols + g * p.Nout + col, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) f32[j] += __uint_as_float(v[j]);
        }
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat162 hh = __floats2bfloat162_rn(f32[2 * j], f32[2 * j + 1]);
          pk[j] = live ? *reinterpret_cast<uint32_t*>(&hh) : 0u;
        }
        if (live) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + col);
          d4[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          d4[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        if (p.stats) {
          float f[16], f2[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const __nv_bfloat162 hh = *reinterpret_cast<const __nv_bfloat162*>(&pk[j >> 1]);
            f[j] = (j & 1) ? __high2float(hh) : __low2float(hh);
            f2[j] = f[j] * f[j];
          }
          const float t1 = colsum16(f, lane), t2 = colsum16(f2, lane);
#pragma unroll
          for (int g = 0; g < 4; ++g)
            if (col == 16 * g) { acc1[g] += t1; acc2[g] += t2; }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (warp == 5 && lane == 0 && it < 10) ts_mark(p.ts, 42 + it);
    }
    if (p.stats && !(lane & 1)) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
        if (16 * g < p.Nout) {
          my_stats[16 * g + stat_column(lane)] = acc1[g];
          my_stats[p.Nout + 16 * g + stat_column(lane)] = acc2[g];
        }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (p.stats && warp > 4 && *abort_flag == 0) {
    // fold the four warps' sums: one atomic per channel and CTA
    for (int i = threadIdx.x - 5 * 32; i < 2 * p.Nout; i += 128)
      atomicAdd(p.stats + i, (stat_smem[i] + stat_smem[2 * p.Nout + i]) + (stat_smem[4 * p.Nout + i] + stat_smem[6 * p.Nout + i]));
  }
  if (threadIdx.x == 0) ts_mark(p.ts, 52);
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// Filter gradient of the 3x3, stride-1, "same" convolution in the same padded linear pixel space:
//   dW[co][tap][ci] = sum over q of dYp[q][co] * Xp[q + shift(tap)][ci]
// (dYp and Xp are zero at padding positions, so padding outputs add nothing). The reduction index is the
// pixel, so both operands are "MN-major", and the per-8-channel planes [pixel][8 channels] are the
// un-swizzled MN-major layout (8 pixels x 16 bytes per core matrix, 128 bytes between pixel groups, one
// plane between channel groups).
//
// An MMA with M = 128 holds the tensor core for about 128 cycles whatever N is, so the kernel is bound by
// the NUMBER of instructions: with one instruction per tap (N = Ci) a 128-pixel chunk needs 72. Here the
// three horizontal taps are folded into N instead: the X tile is stored three times, shifted by -1, 0
// and +1 pixel (planes [dx][channel group], all at one stride), so one instruction with N = 3 * Ci covers
// a whole filter row and the row (dy) is picked by a start address shifted by +-(W+1) pixels: 24
// instructions per chunk. The copies are cheap next to that: each 16-byte piece of X is fetched once
// per plane through L1. M is 128 with Co real rows; planes Co/8 .. 15 of the A tile are zeros written
// once. Accumulators (tap t in columns [t*Ci, (t+1)*Ci)) and the epilogue follow conv_wgrad_kernel; Ci = 64
// (576 columns) stays with that kernel.
struct WgHaloParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* dy;
  float* dw;
  int N, H, W, Ci, Co;
  int pitch, img, q_total, chunks;
  int span;                                    // pixels per B plane: 128 + 2 * (W + 1)
  int a_planes, b_planes, a_log2, b_log2, b_plane_bytes, stage_bytes, stages, bars_off;
  FastDiv div_img, div_pitch;
  int* status;
};

constexpr int kWgAPlane = 128 * 16;          // bytes of one 8-channel plane of the 128-pixel dY chunk
constexpr int kWgABytes = 16 * kWgAPlane;    // M = 128 = 16 planes

__device__ __forceinline__ void cp_async16_ca_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// element offset of padded-linear pixel q (channel group c8) in an N-H-W-C tensor with C channels; *bytes
// is 16 when q is a real pixel and 0 (zero fill) when it is padding or out of range. Branch-free.
__device__ __forceinline__ uint32_t halo_off(int q, const WgHaloParams& p, int C, int c8, uint32_t* bytes) {
  const uint32_t qc = static_cast<uint32_t>(min(max(q, 0), p.q_total - 1));
  const uint32_t n = p.div_img.div(qc), r = qc - n * p.img;
  const uint32_t h = p.div_pitch.div(r), w = r - h * p.pitch;
  const bool valid = q >= 0 && q < p.q_total && h < static_cast<uint32_t>(p.H) && w < static_cast<uint32_t>(p.W);
  *bytes = valid ? 16u : 0u;
  return valid ? ((n * p.H + h) * p.W + w) * C + c8 * 8 : 0u;
}

__global__ void __launch_bounds__(kHaloThreads, 1)
conv3x3_wgrad_halo_kernel(const WgHaloParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.bars_off);
  uint64_t* empty_bar = full_bar + kHaloMaxStages;
  uint64_t* acc_bar = empty_bar + kHaloMaxStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  // planes Co/8 .. 15 of every stage's A tile stay zero for the kernel's lifetime
  for (int s = 0; s < p.stages; ++s) {
    uint4* z = reinterpret_cast<uint4*>(smem + s * p.stage_bytes + p.a_planes * kWgAPlane);
    const int n16 = (16 - p.a_planes) * kWgAPlane / 16;
    for (int i = threadIdx.x; i < n16; i += kHaloThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  const int per_pass = (p.chunks - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);

  if (warp < 4) {
    // ---------------------------------------------------------------- producers (cp.async)
    // as in conv3x3_halo_kernel: a warp per chunk, two chunks in flight per warp
    const int a_items = 128 * p.a_planes;
    const int span8 = (p.span + 7) / 8 * 8;
    const int b_items = (span8 + 8) * p.b_planes;        // pixels -1 .. span8 + 6 of the tile: every plane's share
    const uint32_t plane_set = static_cast<uint32_t>(p.b_planes * p.b_plane_bytes);   // the planes of one dx
    bool ok = true;
    {
      int pending = -1;
      // no more producer warps than stages (see conv3x3_halo_kernel)
      const int nprod = p.stages < 4 ? p.stages : 4;
      for (int j = warp; warp < nprod && j < per_pass && ok; j += nprod) {
        const int it = j;
        const int c = blockIdx.x + j * gridDim.x;
        const int s = it % p.stages;
        const uint32_t parity = ((it / p.stages) & 1) ^ 1;
        if (pending >= 0) {     // see conv3x3_halo_kernel: publish before a wait that may depend on it
          const bool ready = __shfl_sync(0xffffffffu, lane == 0 ? static_cast<int>(mbar_test(&empty_bar[s], parity)) : 0, 0) != 0;
          if (!ready) {
            cp_async_wait_group<0>();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[pending]);
            pending = -1;
          }
        }
        ok = mbar_wait(&empty_bar[s], parity, abort_flag, p.status, kStatusWaitEmpty);
        if (!ok) break;
        const uint32_t a_base = smem_u32(smem + s * p.stage_bytes), b_base = a_base + kWgABytes;
        const int q0 = c * 128;
#pragma unroll 4
        for (int i = lane; i < a_items; i += 32) {
          const int c8 = (i >> 3) & (p.a_planes - 1), pix = ((i >> (3 + p.a_log2)) << 3) + (i & 7);
          uint32_t bytes;
          const uint32_t off = halo_off(q0 + pix, p, p.Co, c8, &bytes);
          cp_async16_zfill(a_base + c8 * kWgAPlane + pix * 16, p.dy + off, bytes);
        }
        // plane set dx holds X shifted by dx - 1 pixels: index u of set dx is pixel q0 - pitch + u + dx - 1,
        // so the piece of pixel q0 - pitch - 1 + v goes to index v, v - 1, v - 2 of sets 0, 1, 2
#pragma unroll 2
        for (int i = lane; i < b_items; i += 32) {
          const int c8 = (i >> 3) & (p.b_planes - 1), v = ((i >> (3 + p.b_log2)) << 3) + (i & 7);
          uint32_t bytes;
          const uint32_t off = halo_off(q0 - p.pitch - 1 + v, p, p.Ci, c8, &bytes);
          const uint32_t dst = b_base + c8 * p.b_plane_bytes + v * 16;
          if (v < span8) cp_async16_ca_zfill(dst, p.x + off, bytes);
          if (v >= 1 && v - 1 < span8) cp_async16_ca_zfill(dst + plane_set - 16, p.x + off, bytes);
          if (v >= 2 && v - 2 < span8) cp_async16_ca_zfill(dst + 2 * plane_set - 32, p.x + off, bytes);
        }
        cp_async_commit();
        if (pending >= 0) {
          cp_async_wait_group<1>();
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[pending]);
        }
        pending = s;
      }
      cp_async_wait_group<0>();
      if (pending >= 0 && ok) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[pending]);
      }
    }
  } else if (warp == 4) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, 3 * p.Ci, 1, 1);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      {
        bool first = true;
        for (int j = 0; j < per_pass && ok; ++j) {
          ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, kStatusWaitFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * p.stage_bytes);
          const uint64_t da0 = conv_desc(a_base, 128, kWgAPlane, 0);
          // index u of a plane is pixel q0 - pitch + u (+ dx - 1): row dy of the filter starts at u = dy * pitch
          const uint64_t db0 = conv_desc(a_base + kWgABytes, 128, p.b_plane_bytes, 0);
          // pixel group outermost, filter row innermost: consecutive instructions go to different accumulators
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t acc = (first && ks == 0) ? 0u : 1u;
#pragma unroll
            for (int rr = 0; rr < 3; ++rr)
              umma_bf16<1>(tmem_base + rr * 3 * p.Ci, da0 + ks * 16, db0 + static_cast<uint64_t>(rr * p.pitch + ks * 16), idesc, acc);
          }
          first = false;
          umma_commit(&empty_bar[s]);
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(acc_bar);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int q4 = warp & 3;
    const int co = q4 * 32 + lane;
    float* stage = reinterpret_cast<float*>(smem);
    bool ok = mbar_wait(acc_bar, 0, abort_flag, p.status, kStatusWaitAccum);
    if (ok) {
      tc_fence_after_sync();
      const int t0 = 0, nt = 9;
      const int row_floats = nt * p.Ci;
      if (q4 * 32 < p.Co) {
        for (int col = 0; col < row_floats; col += 16) {
          uint32_t v[16];
          tmem_ld16(tmem_base + (static_cast<uint32_t>(q4 * 32) << 16) + col, v);
          tmem_ld_wait();
          if (co < p.Co) {
            float4* dst = reinterpret_cast<float4*>(stage + static_cast<size_t>(co) * row_floats + col);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                   __uint_as_float(v[4 * j + 3]));
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (co < p.Co) {
          bulk_reduce_add_f32(p.dw + (static_cast<size_t>(co) * 9 + t0) * p.Ci, stage + static_cast<size_t>(co) * row_floats,
                              static_cast<uint32_t>(row_floats * 4));
          tma_store_commit();
        }
      }
      tc_fence_before_sync();
    }
    tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// N-H-W-C bf16 tensor, box = `cbox` channels x wbox x hbox pixels of one image, optional traversal
// stride; the swizzle mode is the one whose span equals the row (cbox * 2 bytes: 32, 64 or 128).
int make_tmap_nhwc(CUtensorMap* out, const void* base, int N, int H, int W, int C, int cbox, int wbox, int hbox, int stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  ensure_thread_context();
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(N)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(C) * 2, static_cast<cuuint64_t>(W) * C * 2, static_cast<cuuint64_t>(H) * W * C * 2};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(cbox), static_cast<cuuint32_t>((wbox - 1) * stride + 1),
                       static_cast<cuuint32_t>((hbox - 1) * stride + 1), 1};
  cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(stride), static_cast<cuuint32_t>(stride), 1};
  const CUtensorMapSwizzle sw = cbox == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : cbox == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace
}  // namespace fb

namespace fb {
namespace {
int launch_wgrad_halo(const void* x, const void* dy, float* dw, int N, int H, int W, int Ci, int Co, int* status, void* stream) {
  WgHaloParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.dy = static_cast<const __nv_bfloat16*>(dy);
  p.dw = dw;
  p.N = N; p.H = H; p.W = W; p.Ci = Ci; p.Co = Co;
  p.pitch = W + 1;
  p.img = (H + 1) * (W + 1);
  const long long qt = static_cast<long long>(N) * p.img;
  if (qt > (1LL << 30)) return -4;
  if (static_cast<long long>(N) * H * W * (Ci > Co ? Ci : Co) >= (1LL << 31)) return -4;   // 32-bit element offsets
  p.q_total = static_cast<int>(qt);
  p.chunks = (p.q_total + 127) / 128;
  p.span = 128 + 2 * p.pitch;
  p.a_planes = Co / 8;
  p.b_planes = Ci / 8;
  p.a_log2 = p.a_planes == 1 ? 0 : p.a_planes == 2 ? 1 : p.a_planes == 4 ? 2 : 3;
  p.b_log2 = p.b_planes == 2 ? 1 : p.b_planes == 4 ? 2 : 3;
  p.div_img = make_fastdiv(p.img);
  p.div_pitch = make_fastdiv(p.pitch);
  p.b_plane_bytes = (p.span + 7) / 8 * 8 * 16;
  p.stage_bytes = (kWgABytes + 3 * p.b_planes * p.b_plane_bytes + 1023) / 1024 * 1024;
  p.stages = (196 * 1024) / p.stage_bytes;
  if (p.stages > kHaloMaxStages) p.stages = kHaloMaxStages;
  if (p.stages < 2) return -4;
  const int staging = Co * 9 * Ci * 4;
  int ring = p.stages * p.stage_bytes;
  if (ring < staging) ring = (staging + 1023) / 1024 * 1024;
  p.bars_off = ring;
  p.status = status;
  const int smem = p.bars_off + 512 + 1024;
  if (smem > 220 * 1024) return -4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv3x3_wgrad_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int grid = p.chunks / 2;       // at least two chunks per CTA amortise the epilogue's reduce-add
  if (grid > 148) grid = 148;
  if (grid < 1) grid = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kHaloThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
  }
  return static_cast<int>(cudaLaunchKernelEx(&cfg, conv3x3_wgrad_halo_kernel, p));
}
bool wgrad_halo_ok(int H, int W, int Ci, int Co, int k, int stride, int pad) {
  if (!(k == 3 && stride == 1 && pad == 1 && (Ci == 16 || Ci == 32) && (Co == 8 || Co == 16 || Co == 32 || Co == 64) && W >= 2 && H >= 1))
    return false;     // Ci = 64 would need 576 accumulator columns: conv_wgrad_kernel's two passes take it
  // two pipeline stages must fit (launch_wgrad_halo's layout)
  const int plane = (128 + 2 * (W + 1) + 7) / 8 * 8 * 16;
  return 2 * (kWgABytes + 3 * (Ci / 8) * plane + 1023) <= 196 * 1024;
}
}  // namespace
}  // namespace fb

// 1 when fb_conv_wgrad covers the problem, else 0 (the caller then uses the library convolution).
extern "C" int fb_conv_wgrad_supported(int N, int H, int W, int Ci, int Co, int kh, int kw, int stride, int pad) {
  if (N > 0 && kh == kw && fb::wgrad_halo_ok(H, W, Ci, Co, kh, stride, pad)) return 1;
  if (kh != kw || (kh != 1 && kh != 3) || (stride != 1 && stride != 2)) return 0;
  if (pad != (kh == 3 ? 1 : 0)) return 0;
  if ((Ci != 16 && Ci != 32 && Ci != 64) || Co % 8 || Co < 8 || Co > 64) return 0;
  const int Ho = (H + 2 * pad - kh) / stride + 1, Wo = (W + 2 * pad - kw) / stride + 1;
  if (Wo != 8 && Wo != 16 && Wo != 32 && Wo != 64) return 0;
  const int hbox = 64 / Wo;
  if (Ho % hbox) return 0;
  if (((hbox - 1) * stride + 1) > 256 || ((Wo - 1) * stride + 1) > 256) return 0;
  return N > 0;
}

// x: [N,H,W,Ci] bf16, dy: [N,Ho,Wo,Co] bf16, both channels-last contiguous and 16-byte aligned;
// dw: [Co][kh][kw][Ci] fp32, the gradient is ADDED to it.
extern "C" int fb_conv_wgrad(const void* x, const void* dy, float* dw, int N, int H, int W, int Ci, int Co, int kh, int kw,
                             int stride, int pad, int* status, void* stream) {
  using namespace fb;
  if (!fb_conv_wgrad_supported(N, H, W, Ci, Co, kh, kw, stride, pad)) return -4;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(dw) & 15)) return -3;
  if (kh == kw && wgrad_halo_ok(H, W, Ci, Co, kh, stride, pad)) return launch_wgrad_halo(x, dy, dw, N, H, W, Ci, Co, status, stream);
  WgradParams p;
  p.N = N; p.Ci = Ci; p.Co = Co; p.kh = kh; p.kw = kw; p.stride = stride; p.pad = pad;
  p.Ho = (H + 2 * pad - kh) / stride + 1;
  p.Wo = (W + 2 * pad - kw) / stride + 1;
  p.wbox = p.Wo >= 64 ? 64 : p.Wo;
  p.hbox = kPix / p.wbox;
  const int taps = kh * kw;
  p.taps_per_pass = taps < 512 / Ci ? taps : 512 / Ci;
  if (p.taps_per_pass > kMaxTapsPerPass) p.taps_per_pass = kMaxTapsPerPass;
  p.passes = (taps + p.taps_per_pass - 1) / p.taps_per_pass;
  p.chunks = N * (p.Ho / p.hbox) * (p.Wo / p.wbox);
  p.dw = dw;
  p.status = status;
  // B tiles are 64 channels wide whatever Ci is (missing channels zero-filled by the copy): measured
  // on B200, the copy engine spends about 4 cycles per pixel row on such a box and about 7 on an
  // exact 32- or 64-byte-wide one with the narrower swizzle, and the row rate is what bounds this kernel.
  const int cb = 64;
  p.b_bytes = kPix * cb * 2;
  p.b_layout = swizzle_code(cb);
  p.b_sbo = 8 * cb * 2;           // 8 pixel rows
  p.b_kstep = 16 * cb * 2;        // one MMA = 16 pixels
  p.stage_bytes = kPanel + p.taps_per_pass * p.b_bytes;
  p.stages = kPipeBytes / p.stage_bytes;
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages < 2) return -4;
  // the epilogue stages Co rows of (taps_per_pass * Ci) floats over the (then idle) ring
  int ring = p.stages * p.stage_bytes;
  const int staging = Co * p.taps_per_pass * Ci * 4;
  if (ring < staging) ring = (staging + 1023) / 1024 * 1024;
  p.zero_off = ring;
  p.bars_off = ring + kPanel;
  CUtensorMap tdy, tx;
  int r;
  if ((r = make_tmap_nhwc(&tdy, dy, N, p.Ho, p.Wo, Co, 64, p.wbox, p.hbox, 1))) return r;
  if ((r = make_tmap_nhwc(&tx, x, N, H, W, Ci, cb, p.wbox, p.hbox, stride))) return r;
  const int smem = p.bars_off + 512 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  if (smem > 200 * 1024) return -4;
  // one CTA per 64-pixel patch up to the machine size: the copy engine's row rate bounds a CTA, so more
  // CTAs win even though each adds its own reduce-add of the whole filter (ResNet-20 step, measured:
  // 4 patches per CTA 1.333 ms, 2 -> 1.309, 1 -> 1.306)
  static int per_cta = 0;
  if (!per_cta) {
    const char* e = getenv("FLODL_B200_WGRAD_CHUNKS_PER_CTA");
    per_cta = e ? atoi(e) : 1;
    if (per_cta < 1) per_cta = 1;
  }
  int grid = p.chunks / per_cta;
  if (grid > 148) grid = 148;
  if (grid < 1) grid = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kConvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
  }
  return static_cast<int>(cudaLaunchKernelEx(&cfg, conv_wgrad_kernel, tdy, tx, p));
}

namespace fb {
namespace {

// Filter as a 2-D bf16 matrix [Co][taps * Ci]; one box = one tap's [Co][Ci] block.
int make_tmap_filter(CUtensorMap* out, const void* base, int Co, int taps, int Ci) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  ensure_thread_context();
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(taps) * Ci, static_cast<cuuint64_t>(Co)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(taps) * Ci * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(Ci), static_cast<cuuint32_t>(Co)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = Ci == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : Ci == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}


// Shared launcher of the forward pass (dgrad == 0) and the stride-1 data gradient (dgrad == 1).
// (H, W) is the extent of `in`, (Ho, Wo) that of `out`.
int launch_conv_fwd(const void* in, const void* w, void* out, float* stats, int N, int H, int W, int Ho, int Wo, int Ci, int Co, int k, int stride,
                    int pad, int dgrad, int* status, void* stream) {
  FwdParams p;
  p.Kc = dgrad ? Co : Ci;
  p.Nout = dgrad ? Ci : Co;
  p.Ci = Ci;
  p.taps = k * k;
  p.kw = k;
  p.stride = stride;
  p.pad = pad;
  p.sign = dgrad ? -1 : 1;
  const int img = Ho * Wo;
  const int bp = img < 128 ? img : 128;          // pixels per box
  p.wbox = Wo;
  p.hbox = bp / Wo;
  p.nbox = 128 / bp;
  p.per_img = img / bp;
  p.images = N;
  p.pixels = static_cast<long long>(N) * img;
  p.tiles = static_cast<int>((p.pixels + 127) / 128);
  p.a_bytes = 128 * p.Kc * 2;
  p.a_layout = swizzle_code(p.Kc);
  p.a_sbo = 8 * p.Kc * 2;
  p.w_bytes = Co * Ci * 2;
  p.w_layout = swizzle_code(Ci);
  p.w_sbo = 8 * Ci * 2;
  p.w_kstep = dgrad ? 16 * Ci * 2 : 32;          // 16 filter rows (MN-major) or 16 channels inside a row (K-major)
  p.b_mn = dgrad;
  const int w_total = (p.taps * p.w_bytes + 1023) / 1024 * 1024;
  p.ring_off = w_total;
  p.stages = (200 * 1024 - w_total - 4096) / p.a_bytes;
  if (p.stages > kFwdMaxStages) p.stages = kFwdMaxStages;
  if (p.stages < 2) return -4;
  p.bars_off = w_total + p.stages * p.a_bytes;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.stats = stats;
  p.status = status;
  CUtensorMap tin, tw;
  int r;
  if ((r = make_tmap_nhwc(&tin, in, N, H, W, p.Kc, p.Kc, p.wbox, p.hbox, stride))) return r;
  if ((r = make_tmap_filter(&tw, w, Co, p.taps, Ci))) return r;
  const int smem = p.bars_off + 512 + 4 * 2 * p.Nout * 4 + 1024;
  if (smem > 220 * 1024) return -4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int grid = p.tiles < 148 ? p.tiles : 148;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kConvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
  }
  return static_cast<int>(cudaLaunchKernelEx(&cfg, conv_fwd_kernel, tin, tw, p));
}

int launch_conv_halo(const void* in, const void* w, void* out, float* stats, int N, int H, int W, int Ci, int Co, int dgrad, int* status,
                     void* stream, long long* ts = nullptr) {
  HaloParams p;
  p.in = static_cast<const __nv_bfloat16*>(in);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.N = N; p.H = H; p.W = W;
  p.Kc = dgrad ? Co : Ci;
  p.Nout = dgrad ? Ci : Co;
  p.Ci = Ci;
  p.sign = dgrad ? -1 : 1;
  p.b_mn = dgrad;
  p.pitch = W + 1;
  p.img = (H + 1) * (W + 1);
  const long long qt = static_cast<long long>(N) * p.img;
  if (qt > (1LL << 30)) return -4;
  p.q_total = static_cast<int>(qt);
  p.tiles = (p.q_total + 127) / 128;
  p.halo = W + 2;
  p.span = 128 + 2 * p.halo;
  p.groups = 256 / p.Nout > 9 ? 9 : 256 / p.Nout;
  if (static_cast<long long>(N) * H * W * (Ci > Co ? Ci : Co) >= (1LL << 31)) return -4;   // 32-bit element offsets
  p.nch = p.Kc / 8;
  p.nch_log2 = p.nch == 2 ? 1 : p.nch == 4 ? 2 : 3;
  p.div_img = make_fastdiv(p.img);
  p.div_pitch = make_fastdiv(p.pitch);
  p.plane_bytes = (p.span * 16 + 127) / 128 * 128;
  p.a_bytes = p.nch * p.plane_bytes;
  p.w_bytes = Co * Ci * 2;
  p.w_layout = swizzle_code(Ci);
  p.w_sbo = 8 * Ci * 2;
  p.w_kstep = dgrad ? 16 * Ci * 2 : 32;
  const int w_total = (9 * p.w_bytes + 1023) / 1024 * 1024;
  p.ring_off = w_total;
  p.stages = (200 * 1024 - w_total - 4096) / p.a_bytes;
  if (p.stages > kHaloMaxStages) p.stages = kHaloMaxStages;
  if (p.stages < 2) return -4;
  p.bars_off = w_total + p.stages * p.a_bytes;
  p.stats = stats;
  p.status = status;
  p.ts = ts;
  CUtensorMap tw;
  int r;
  if ((r = make_tmap_filter(&tw, w, Co, 9, Ci))) return r;
  const int smem = p.bars_off + 512 + 4 * 2 * p.Nout * 4 + 1024;
  if (smem > 220 * 1024) return -4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv3x3_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int grid = p.tiles < 148 ? p.tiles : 148;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kHaloThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
  }
  return static_cast<int>(cudaLaunchKernelEx(&cfg, conv3x3_halo_kernel, tw, p));
}

// shapes of the halo kernel: 3x3, stride 1, pad 1; image width up to 128 so that a stage stays small
bool halo_shape_ok(int H, int W, int Kc, int Nout, int Ci) {
  if (Kc != 16 && Kc != 32 && Kc != 64) return false;
  if (Ci != 16 && Ci != 32 && Ci != 64) return false;
  if (Nout % 16 || Nout < 16 || Nout > 64) return false;
  return H >= 1 && W >= 2 && W <= 128;
}

bool fwd_shape_ok(int Ho, int Wo, int Kc, int Nout, int k, int stride, int pad) {
  if ((k != 1 && k != 3) || (stride != 1 && stride != 2) || pad != k / 2) return false;
  if (Kc != 16 && Kc != 32 && Kc != 64) return false;
  if (Nout % 16 || Nout < 16 || Nout > 64) return false;
  if (Wo != 8 && Wo != 16 && Wo != 32 && Wo != 64 && Wo != 128) return false;
  const int img = Ho * Wo, bp = img < 128 ? img : 128;
  if (img < 64 || bp % Wo || img % bp) return false;
  const int hbox = bp / Wo;
  return (hbox - 1) * stride + 1 <= 256 && (Wo - 1) * stride + 1 <= 256;
}

}  // namespace
}  // namespace fb

// 1 when fb_conv_fprop covers the problem (x: [N,H,W,Ci], filter [Co][k][k][Ci]).
extern "C" int fb_conv_fprop_supported(int N, int H, int W, int Ci, int Co, int k, int stride, int pad) {
  if (N > 0 && k == 3 && stride == 1 && pad == 1 && fb::halo_shape_ok(H, W, Ci, Co, Ci)) return 1;
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  return N > 0 && fb::fwd_shape_ok(Ho, Wo, Ci, Co, k, stride, pad);
}

// y[N,Ho,Wo,Co] = conv(x[N,H,W,Ci], w[Co][k][k][Ci]), all bf16 and 16-byte aligned. `stats`, when given,
// is a zeroed-by-the-caller fp32 [2][Co] that receives the per-channel sum and sum of squares of y.
extern "C" int fb_conv_fprop_ts(const void* x, const void* w, void* y, float* stats, int N, int H, int W, int Ci, int Co, int k, int stride,
                                int pad, int* status, long long* ts, void* stream) {
  if (!(k == 3 && stride == 1 && pad == 1 && fb::halo_shape_ok(H, W, Ci, Co, Ci))) return -4;
  return fb::launch_conv_halo(x, w, y, stats, N, H, W, Ci, Co, 0, status, stream, ts);
}

extern "C" int fb_conv_fprop(const void* x, const void* w, void* y, float* stats, int N, int H, int W, int Ci, int Co, int k, int stride, int pad,
                             int* status, void* stream) {
  if (!fb_conv_fprop_supported(N, H, W, Ci, Co, k, stride, pad)) return -4;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return -3;
  if (k == 3 && stride == 1 && pad == 1 && fb::halo_shape_ok(H, W, Ci, Co, Ci))
    return fb::launch_conv_halo(x, w, y, stats, N, H, W, Ci, Co, 0, status, stream);
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  return fb::launch_conv_fwd(x, w, y, stats, N, H, W, Ho, Wo, Ci, Co, k, stride, pad, 0, status, stream);
}

// 1 when fb_conv_dgrad covers the problem: stride 1 only (the input and output grids coincide).
extern "C" int fb_conv_dgrad_supported(int N, int H, int W, int Ci, int Co, int k, int stride, int pad) {
  if (N > 0 && k == 3 && stride == 1 && pad == 1 && fb::halo_shape_ok(H, W, Co, Ci, Ci)) return 1;
  return N > 0 && stride == 1 && (Ci == 16 || Ci == 32 || Ci == 64) && fb::fwd_shape_ok(H, W, Co, Ci, k, 1, pad);
}

// dx[N,H,W,Ci] = conv_transpose(dy[N,H,W,Co], w[Co][k][k][Ci]) for stride 1, "same" padding.
extern "C" int fb_conv_dgrad(const void* dy, const void* w, void* dx, int N, int H, int W, int Ci, int Co, int k, int stride, int pad, int* status,
                             void* stream) {
  if (!fb_conv_dgrad_supported(N, H, W, Ci, Co, k, stride, pad)) return -4;
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(dx) & 15)) return -3;
  if (k == 3 && pad == 1 && fb::halo_shape_ok(H, W, Co, Ci, Ci)) return fb::launch_conv_halo(dy, w, dx, nullptr, N, H, W, Ci, Co, 1, status, stream);
  return fb::launch_conv_fwd(dy, w, dx, nullptr, N, H, W, H, W, Ci, Co, k, 1, pad, 1, status, stream);
}
