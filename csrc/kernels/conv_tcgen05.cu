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
//     traversal stride is the convolution stride.
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
constexpr int kConvStages = 2;
constexpr int kMaxTapsPerPass = 9;

struct WgradParams {
  int N, Ho, Wo, Ci, Co;
  int kh, kw, stride, pad;
  int hbox, wbox;          // the 64-pixel patch of the OUTPUT grid: hbox * wbox == 64
  int taps_per_pass, passes;
  int chunks;              // N * (Ho / hbox) * (Wo / wbox)
  float* dw;               // [Co][kh][kw][Ci] fp32, accumulated into
  int* status;
};

__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
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
  const int stage_bytes = (2 + p.taps_per_pass) * kPanel;          // A: 2 panels, B: one per tap
  uint8_t* bars_mem = smem + kConvStages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bars_mem);
  uint64_t* empty_bar = full_bar + kConvStages;
  uint64_t* acc_bar = empty_bar + kConvStages;                      // accumulators of a pass complete
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
  // The second A panel (rows 64..127 of M) starts as zeros. Its content only ever reaches
  // accumulator rows 64..127, which nobody reads, so it does not matter that a later pass finds the
  // epilogue's staging data there.
  for (int s = 0; s < kConvStages; ++s) {
    uint4* z = reinterpret_cast<uint4*>(smem + s * stage_bytes + kPanel);
    for (int i = threadIdx.x; i < kPanel / 16; i += kConvThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

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
          mbar_expect_tx(&full_bar[s], (1 + nt) * kPanel);
          tma4(sa, &tmDy, &full_bar[s], 0, wo0, ho0, n);
          for (int t = 0; t < nt; ++t) {
            const int tap = t0 + t, dy = tap / p.kw, dx = tap - dy * p.kw;
            tma4(sa + (2 + t) * kPanel, &tmX, &full_bar[s], 0, wo0 * p.stride + dx - p.pad, ho0 * p.stride + dy - p.pad, n);
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
          for (int t = 0; t < nt; ++t) {
            const uint32_t sb = sa + (2 + t) * kPanel;
#pragma unroll
            for (int k4 = 0; k4 < kPix / 16; ++k4) {
              const uint64_t da = make_smem_desc(sa + k4 * 2048, kPanel, 1024);
              const uint64_t db = make_smem_desc(sb + k4 * 2048, kPanel, 1024);
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

// N-H-W-C bf16 tensor, box = 64 channels x wbox x hbox pixels of one image, optional traversal stride
int make_tmap_nhwc(CUtensorMap* out, const void* base, int N, int H, int W, int C, int wbox, int hbox, int stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  ensure_thread_context();
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(N)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(C) * 2, static_cast<cuuint64_t>(W) * C * 2, static_cast<cuuint64_t>(H) * W * C * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>((wbox - 1) * stride + 1), static_cast<cuuint32_t>((hbox - 1) * stride + 1), 1};
  cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(stride), static_cast<cuuint32_t>(stride), 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace
}  // namespace fb

// 1 when fb_conv_wgrad covers the problem, else 0 (the caller then uses the library convolution).
extern "C" int fb_conv_wgrad_supported(int N, int H, int W, int Ci, int Co, int kh, int kw, int stride, int pad) {
  if (kh != kw || (kh != 1 && kh != 3) || (stride != 1 && stride != 2)) return 0;
  if (pad != (kh == 3 ? 1 : 0)) return 0;
  if (Ci % 16 || Ci < 16 || Ci > 64 || Co % 8 || Co < 8 || Co > 64) return 0;
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
  CUtensorMap tdy, tx;
  int r;
  if ((r = make_tmap_nhwc(&tdy, dy, N, p.Ho, p.Wo, Co, p.wbox, p.hbox, 1))) return r;
  if ((r = make_tmap_nhwc(&tx, x, N, H, W, Ci, p.wbox, p.hbox, stride))) return r;
  const int stage_bytes = (2 + p.taps_per_pass) * kPanel;
  const int smem = kConvStages * stage_bytes + 256 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kConvStages * (2 + kMaxTapsPerPass) * kPanel + 256 + 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  // enough CTAs to fill the machine, few enough that each one amortises its epilogue over >= 4 patches
  int grid = p.chunks / 4;
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
