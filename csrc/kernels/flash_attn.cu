// Flash-style attention forward / backward for head dim 64 on tcgen05 tensor cores.
//
// Replaces `at::scaled_dot_product_attention` (flodl-sys/ops_nn.cpp:367-388) behind the encoder
// layers (flodl-hf/src/models/transformer_layer.rs:243-251) and the decomposed
// matmul / masked_fill / softmax / matmul chain of `MultiheadAttention`
// (flodl/src/nn/attention.rs:108-151): additive key mask [B,S], causal masking, attention-prob
// dropout, O(S) memory (only the log-sum-exp per row is saved).
//
// Work split: one CTA per (query block of 128 rows, head, batch) in the forward pass, one CTA per
// (head, batch) in the backward pass. 4 warps (one TMEM lane = one query row per thread) do the
// softmax arithmetic; a fifth warp issues every TMA load and every `tcgen05.mma` from one thread.
// Q, K, V, dO tiles arrive by TMA with 128-byte swizzle in their natural [row][64] layout; the
// same tile serves as a K-major operand (QK^T, dO V^T) or an MN-major operand (P V, P^T dO,
// dS^T Q, dS K) by flipping the major bit of the instruction descriptor, so nothing is transposed.
// P and dS are written to shared memory by the softmax threads in the swizzled layout the MMA
// expects. All accumulators (S, dP, O, dQ, dK, dV) live in TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/flodl_b200.h"
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fb {

constexpr int kHD = 64;        // head dim
constexpr int kBlk = 128;      // rows per query / key block
constexpr int kAttnThreads = 160;
constexpr float kLog2e = 1.4426950408889634f;

// Per-CTA timeline of the single-block kernels (a tuning aid, compiled in only with -DFB_TIMELINE=1): 8 clock64
// stamps per CTA for the first 1024 CTAs of a launch (forward) / 16 per CTA (backward), read back with fb_attn_timeline.
#ifndef FB_TIMELINE
#define FB_TIMELINE 0
#endif
#if FB_TIMELINE
__device__ long long g_attn_ts[16 * 1024];
#define FB_ATTN_TS(slot) do { const int cta_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); if (cta_ < 1024) { \
    long long v_ = clock64(); if ((slot) >= 14) { unsigned long long g_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_)); v_ = static_cast<long long>(g_); } \
    g_attn_ts[cta_ * 16 + (slot)] = v_; } } while (0)
#else
#define FB_ATTN_TS(slot) do { } while (0)
#endif

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                      uint32_t box_inner, uint32_t box_outer);  // gemm_tcgen05.cu
void ensure_thread_context();                                    // gemm_tcgen05.cu

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static int make_tmap_bshd(CUtensorMap* out, const void* base, int B, int H, int S, long long sb, long long ss, long long sh) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  ensure_thread_context();
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHD), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh) * 2, static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {kHD, kBlk, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Address of the 16-byte chunk holding columns [8*chunk, 8*chunk+8) of `row` in a [128][64] bf16
// tile stored with the 128-byte swizzle (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t swz_chunk(uint32_t tile_base, int row, int chunk) {
  return tile_base + row * 128 + ((chunk ^ (row & 7)) << 4);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return r;
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// Row-per-thread data (the TMEM register layout: thread = row, 64 bf16 = 128 bytes per row) to and from global rows
// that are `row_stride` elements apart. A thread touching its own row would make every load / store instruction hit 32
// different 128-byte lines; instead each warp moves its 32 rows through a 4 KB staging area of shared memory
// (chunks XOR-swizzled by row, so both sides are free of bank conflicts) and eight lanes share one row in global
// memory. Only the warp's own rows are involved: __syncwarp is all the synchronisation needed.
//
// stage_half: thread `lane` deposits 32 consecutive columns [col0, col0 + 32) of its row.
__device__ __forceinline__ void stage_half(uint32_t stage, int lane, int col0, const float* v32) {
#pragma unroll
  for (int g = 0; g < 4; ++g) st_shared_v4(stage + lane * 128 + ((((col0 >> 3) + g) ^ (lane & 7)) << 4), pack8(v32 + 8 * g));
}
// flush_rows: after both halves were staged, writes rows [row0, row0 + 32) (those below `row_limit`) of a [*, 64] bf16 tensor.
__device__ __forceinline__ void flush_rows(uint32_t stage, int lane, __nv_bfloat16* base, long long row_stride, int row0, int row_limit) {
  __syncwarp();
  const int sub = lane >> 3, ch = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + sub;
    const uint4 val = ld_shared_v4(stage + r * 128 + ((ch ^ (r & 7)) << 4));
    if (row0 + r < row_limit) *reinterpret_cast<uint4*>(base + static_cast<long long>(row0 + r) * row_stride + ch * 8) = val;
  }
  __syncwarp();
}
// D[row] = sum_c a[row][c] * b[row][c] over 64 columns for the warp's 32 rows, eight lanes per row; lane l gets row l's sum.
__device__ __forceinline__ float row_dot64(const __nv_bfloat16* a, const __nv_bfloat16* b, long long row_stride, int row0, int row_limit, int lane) {
  const int sub = lane >> 3, ch = lane & 7;
  float mine = 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    // all loads of four iterations first (the shuffles below would otherwise serialise one memory latency per iteration)
    uint4 xa[4], xb[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int r = (half * 4 + k) * 4 + sub;
      xa[k] = xb[k] = make_uint4(0u, 0u, 0u, 0u);
      if (row0 + r < row_limit) {
        xa[k] = __ldg(reinterpret_cast<const uint4*>(a + static_cast<long long>(row0 + r) * row_stride + ch * 8));
        xb[k] = __ldg(reinterpret_cast<const uint4*>(b + static_cast<long long>(row0 + r) * row_stride + ch * 8));
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int it = half * 4 + k;
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&xa[k]);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&xb[k]);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = __bfloat1622float2(ha[e]), fb2 = __bfloat1622float2(hb[e]);
        d += fa.x * fb2.x + fa.y * fb2.y;
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      // row it*4 + g now sits in lanes 8g .. 8g+7; lane l wants row l = it*4 + g  <=>  it == l / 4, g == l % 4
      const float got = __shfl_sync(0xffffffffu, d, (lane & 3) * 8);
      if ((lane >> 2) == it) mine = got;
    }
  }
  return mine;
}

struct AttnParams {
  int B, H, S;
  long long sb, ss, sh;      // element strides of q/k/v
  long long osb, oss, osh;   // ... of o / dO
  long long gsb, gss, gsh;   // ... of dq / dk / dv
  const float* mask;         // [B, S] additive, may be null
  float scale;
  int causal;
  float p_drop;
  unsigned long long seed;
  const unsigned long long* seed_dev;
  int* status;
};

// ===================================================================================== forward
// Shared-memory layout of the forward kernel. Several key blocks: two K/V stages and P panels of their own
// (114 KB, two CTAs per SM). A single key block (S <= 128, the encoder shapes): Q and K are dead once S = Q K^T
// has completed, so the probabilities are written over them (49 KB); with the output accumulator taking over the
// TMEM columns of S as well (128 columns per CTA) and no running accumulator in registers, four CTAs share an
// SM and hide one another's load / MMA / softmax latencies, which is what bounds a 128 x 128 x 64 problem.
struct FwdSmem {
  int Q, K, V, P, MASK, BARS, TOTAL;
  __host__ __device__ explicit FwdSmem(bool single) {
    const int st = single ? 1 : 2;
    Q = 0;                       // 16 KB
    K = 16384;                   // st x 16 KB
    V = K + st * 16384;          // st x 16 KB
    P = single ? 0 : V + st * 16384;          // 2 panels x 16 KB
    MASK = single ? V + 16384 : P + 2 * 16384;        // 128 floats
    BARS = MASK + 512;
    TOTAL = BARS + 256;
  }
};

template <bool kSingle>
__global__ void __launch_bounds__(kAttnThreads, kSingle ? 4 : 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ o, float* __restrict__ lse,
                const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int n_kv_all = (p.S + kBlk - 1) / kBlk;
  constexpr int kv_stages = kSingle ? 1 : 2;
  constexpr int kTmemCols = kSingle ? 128 : 256;
  const FwdSmem L(kSingle);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.BARS);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* kv_empty = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* o_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* mask_s = reinterpret_cast<float*>(smem + L.MASK);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * kBlk;
  if (kSingle && threadIdx.x == 0) { FB_ATTN_TS(0); FB_ATTN_TS(14); }
  const int n_kv = p.causal ? min(n_kv_all, qb + 1) : n_kv_all;
  const unsigned long long seed = p.seed + (p.seed_dev ? *p.seed_dev : 0ull);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    mbar_init(o_done, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc<1>(tmem_slot, kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  pdl_entry();       // barriers, TMEM and descriptors are set up; everything below reads the predecessor's output
  if (kSingle && threadIdx.x == 0) FB_ATTN_TS(1);
  // single key block: every softmax thread has read its row of S before P V is issued (p_ready), so O reuses S's columns
  const uint32_t tmem_O = kSingle ? tmem_base : tmem_base + 128;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------- loads + MMA issue (one thread)
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, kHD, 0, 1);
      const uint32_t sQ = smem_u32(smem + L.Q);
      const uint32_t sP = smem_u32(smem + L.P);
      mbar_expect_tx(q_full, 16384);
      tma_load_4d(smem + L.Q, &tmQ, q_full, 0, q0, h, b);
      for (int j = 0; j < min(kv_stages, n_kv); ++j) {
        mbar_expect_tx(&kv_full[j], 32768);
        tma_load_4d(smem + L.K + j * 16384, &tmK, &kv_full[j], 0, j * kBlk, h, b);
        tma_load_4d(smem + L.V + j * 16384, &tmV, &kv_full[j], 0, j * kBlk, h, b);
      }
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusWaitFull);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % kv_stages;
        const int use = j / kv_stages;       // how many times this stage was used before
        const uint32_t sK = smem_u32(smem + L.K + st * 16384);
        const uint32_t sV = smem_u32(smem + L.V + st * 16384);
        ok = mbar_wait(&kv_full[st], use & 1, abort_flag, p.status, kStatusWaitFull);
        if (!ok) break;
        tc_fence_after_sync();
        if (kSingle) FB_ATTN_TS(2);
        // S = Q K^T (the softmax threads have drained S of block j-1: they arrived on p_ready)
#pragma unroll
        for (int k4 = 0; k4 < kHD / 16; ++k4)
          umma_bf16<1>(tmem_S, make_smem_desc(sQ + k4 * 32, 16, 1024), make_smem_desc(sK + k4 * 32, 16, 1024), idesc_s, k4 > 0);
        umma_commit(s_full);
        ok = mbar_wait(p_ready, j & 1, abort_flag, p.status, kStatusWaitEpi);
        if (!ok) break;
        if (j > 0) {
          ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, p.status, kStatusWaitEpi);
          if (!ok) break;
        }
        tc_fence_after_sync();
        // O_j = P V
#pragma unroll
        for (int k8 = 0; k8 < kBlk / 16; ++k8) {
          const uint32_t a = sP + (k8 >> 2) * 16384 + (k8 & 3) * 32;
          umma_bf16<1>(tmem_O, make_smem_desc(a, 16, 1024), make_smem_desc(sV + k8 * 2048, 8192, 1024), idesc_o, k8 > 0);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[st]);
        if (j + kv_stages < n_kv) {
          ok = mbar_wait(&kv_empty[st], use & 1, abort_flag, p.status, kStatusWaitEmpty);
          if (!ok) break;
          mbar_expect_tx(&kv_full[st], 32768);
          tma_load_4d(smem + L.K + st * 16384, &tmK, &kv_full[st], 0, (j + kv_stages) * kBlk, h, b);
          tma_load_4d(smem + L.V + st * 16384, &tmV, &kv_full[st], 0, (j + kv_stages) * kBlk, h, b);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax threads
    const int t = threadIdx.x;            // row within the block == TMEM lane
    const int q = q0 + t;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t sP = smem_u32(smem + L.P);
    const float sc = p.scale * kLog2e;
    const float inv_keep = p.p_drop > 0.f ? 1.f / (1.f - p.p_drop) : 1.f;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[kSingle ? 1 : kHD];      // running output row; not needed when there is one key block
#pragma unroll
    for (int i = 0; i < (kSingle ? 1 : kHD); ++i) acc[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int kv0 = j * kBlk;
      // stage the additive mask of this key block (mask * log2e; -inf beyond S)
      asm volatile("bar.sync 1, 128;");
      {
        const int kv = kv0 + t;
        float mv = (kv < p.S) ? (p.mask ? p.mask[static_cast<long long>(b) * p.S + kv] * kLog2e : 0.f) : -INFINITY;
        mask_s[t] = mv;
      }
      asm volatile("bar.sync 1, 128;");
      ok = mbar_wait(s_full, j & 1, abort_flag, p.status, kStatusWaitAccum);
      if (!ok) break;
      tc_fence_after_sync();
      if (kSingle && t == 0) FB_ATTN_TS(3);
      // pass 1: row maximum
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kBlk; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_S + lane_base + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i4 = 0; i4 < 32; i4 += 4) {
          const float4 mk = *reinterpret_cast<const float4*>(mask_s + c + i4);     // one 16-byte shared load per 4 keys
          const float mk4[4] = {mk.x, mk.y, mk.z, mk.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = i4 + k;
            float s = __uint_as_float(v[i]) * sc + mk4[k];
            if (p.causal && kv0 + c + i > q) s = -INFINITY;
            m_blk = fmaxf(m_blk, s);
          }
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);   // m_run = -inf on the first block -> 0
      float l_blk = 0.f;
      // pass 2: probabilities -> shared memory (bf16, swizzled), row sum
#pragma unroll 1
      for (int c = 0; c < kBlk; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_S + lane_base + c, v);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int i4 = 0; i4 < 32; i4 += 4) {
          const float4 mk = *reinterpret_cast<const float4*>(mask_s + c + i4);
          const float mk4[4] = {mk.x - m_use, mk.y - m_use, mk.z - m_use, mk.w - m_use};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = i4 + k;
            float s = __uint_as_float(v[i]) * sc + mk4[k];      // score - row maximum in one FMA
            if (p.causal && kv0 + c + i > q) s = -INFINITY;
            pr[i] = exp2f(s);
            l_blk += pr[i];
          }
        }
        if (p.p_drop > 0.f) {
          const unsigned long long base = ((static_cast<unsigned long long>(b) * p.H + h) * p.S + q) * p.S + kv0 + c;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float s4[4];
            dropout_scale4(seed, base + i, p.p_drop, inv_keep, s4);
#pragma unroll
            for (int k = 0; k < 4; ++k) pr[i + k] *= s4[k];
          }
        }
        const uint32_t panel = sP + (c >> 6) * 16384;
#pragma unroll
        for (int g = 0; g < 4; ++g) st_shared_v4(swz_chunk(panel, t, ((c & 63) >> 3) + g), pack8(pr + 8 * g));
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      if (kSingle && t == 0) FB_ATTN_TS(4);
      mbar_arrive(p_ready);
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      ok = __all_sync(0xffffffffu, mbar_wait(o_full, j & 1, abort_flag, p.status, kStatusWaitAccum));   // warp-uniform: the staged stores below use __syncwarp
      if (!ok) break;
      tc_fence_after_sync();
      if (kSingle && t == 0) FB_ATTN_TS(5);
      if constexpr (kSingle) {
        // the only block: normalise, then out through the warp's staging area (P is dead: P V has completed)
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        const uint32_t stage = smem_u32(smem + L.P) + warp * 4096;
#pragma unroll
        for (int c = 0; c < kHD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_O + lane_base + c, v);
          tmem_ld_wait();
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]) * inv_l;
          stage_half(stage, lane, c, f);
        }
        flush_rows(stage, lane, o + static_cast<long long>(b) * p.osb + static_cast<long long>(h) * p.osh, p.oss, q0 + warp * 32, p.S);
      } else {
#pragma unroll
        for (int c = 0; c < kHD; c += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_O + lane_base + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c + i] = acc[c + i] * alpha + __uint_as_float(v[i]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(o_done);
    }
    if constexpr (!kSingle) {
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {      // every MMA has completed: the P panels serve as staging area
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        const uint32_t stage = smem_u32(smem + L.P) + warp * 4096;
#pragma unroll
        for (int c = 0; c < kHD; c += 32) {
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = acc[c + i] * inv_l;
          stage_half(stage, lane, c, f);
        }
        flush_rows(stage, lane, o + static_cast<long long>(b) * p.osb + static_cast<long long>(h) * p.osh, p.oss, q0 + warp * 32, p.S);
      }
    }
    if (ok && q < p.S) {
      // natural-log LSE of the scaled, masked scores
      lse[(static_cast<long long>(b) * p.H + h) * p.S + q] = (l_run > 0.f) ? (m_run + log2f(l_run)) / kLog2e : -INFINITY;
    }
  }
  if (kSingle && threadIdx.x == 0) FB_ATTN_TS(6);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
  if (kSingle && threadIdx.x == 0) { FB_ATTN_TS(7); FB_ATTN_TS(15); }
}

// ==================================================================================== backward
// Several key blocks: every tile has a buffer of its own and every accumulator its own TMEM columns (129 KB, 512
// columns: one CTA per SM). A single key block (S <= 128): V is dead once dP = dO V^T has completed, so the first
// dS panel takes its place (112.75 KB), and dV / dK / dQ accumulate in the columns S and dP occupied until the
// softmax threads had read them (256 columns): two CTAs share an SM.
struct BwdSmem {
  int Q, DO, K, V, P, DS, MASK, BARS, TOTAL;
  __host__ __device__ explicit BwdSmem(bool single) {
    Q = 0;
    DO = 16384;
    K = 2 * 16384;
    if (single) {
      P = 3 * 16384;           // 2 panels
      V = 5 * 16384;
      DS = 5 * 16384;          // 2 panels, the first one over V
      MASK = 7 * 16384;
    } else {
      V = 3 * 16384;
      P = 4 * 16384;           // 2 panels
      DS = 6 * 16384;          // 2 panels
      MASK = 8 * 16384;
    }
    BARS = MASK + 512;
    TOTAL = BARS + 256;
  }
};

template <bool kSingle>
__global__ void __launch_bounds__(kAttnThreads, kSingle ? 2 : 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                const float* __restrict__ lse, __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk,
                __nv_bfloat16* __restrict__ dv, float* __restrict__ dq_accum, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // The single-block layout leaves no room for alignment slack (two CTAs must fit in one SM): it relies on the
  // 1024-byte alignment of the dynamic shared-memory window and reports instead of computing if that does not hold.
  uint8_t* smem = kSingle ? smem_raw : reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (kSingle && (smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, static_cast<int>(kStatusBadArg));
    return;
  }
  const BwdSmem L(kSingle);
  constexpr int kTmemCols = kSingle ? 256 : 512;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.BARS);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;
  uint64_t* sdp_full = bars + 2;
  uint64_t* pds_ready = bars + 3;
  uint64_t* grads_full = bars + 4;
  uint64_t* tile_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* mask_s = reinterpret_cast<float*>(smem + L.MASK);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;
  const int nblk = (p.S + kBlk - 1) / kBlk;
  if (kSingle && threadIdx.x == 0) FB_ATTN_TS(8);
  const unsigned long long seed = p.seed + (p.seed_dev ? *p.seed_dev : 0ull);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(q_full, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 128);
    mbar_init(grads_full, 1);
    mbar_init(tile_done, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc<1>(tmem_slot, kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128;
  pdl_entry();
  if (kSingle && threadIdx.x == 0) FB_ATTN_TS(7);
  // single key block: S and dP have been read by every softmax thread (pds_ready) before the gradient MMAs are issued
  const uint32_t tDV = tmem_base + (kSingle ? 0 : 256), tDK = tmem_base + (kSingle ? 64 : 320), tDQ = tmem_base + (kSingle ? 128 : 384);

  if (warp == 4) {
    if (lane == 0) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);      // S, dP: both operands K-major
      const uint32_t idesc_mn = make_idesc_bf16(128, kHD, 1, 1);      // dV, dK: A^T (MN-major) x MN-major
      const uint32_t idesc_kn = make_idesc_bf16(128, kHD, 0, 1);      // dQ: K-major x MN-major
      const uint32_t sQ = smem_u32(smem + L.Q), sDO = smem_u32(smem + L.DO);
      const uint32_t sK = smem_u32(smem + L.K), sV = smem_u32(smem + L.V);
      const uint32_t sP = smem_u32(smem + L.P), sDS = smem_u32(smem + L.DS);
      int it = 0;
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int i0 = p.causal ? j : 0;
        if (j > 0) {  // the previous key block's tiles (and their dK/dV drain) are finished
          ok = mbar_wait(tile_done, (it - 1) & 1, abort_flag, p.status, kStatusWaitEpi);
          if (!ok) break;
        }
        mbar_expect_tx(kv_full, 32768);
        tma_load_4d(smem + L.K, &tmK, kv_full, 0, j * kBlk, h, b);
        tma_load_4d(smem + L.V, &tmV, kv_full, 0, j * kBlk, h, b);
        for (int i = i0; i < nblk && ok; ++i, ++it) {
          if (i > i0) {
            ok = mbar_wait(tile_done, (it - 1) & 1, abort_flag, p.status, kStatusWaitEpi);
            if (!ok) break;
          }
          mbar_expect_tx(q_full, 32768);
          tma_load_4d(smem + L.Q, &tmQ, q_full, 0, i * kBlk, h, b);
          tma_load_4d(smem + L.DO, &tmDO, q_full, 0, i * kBlk, h, b);
          if (i == i0) {
            ok = mbar_wait(kv_full, j & 1, abort_flag, p.status, kStatusWaitFull);
            if (!ok) break;
          }
          ok = mbar_wait(q_full, it & 1, abort_flag, p.status, kStatusWaitFull);
          if (!ok) break;
          tc_fence_after_sync();
          if (kSingle) FB_ATTN_TS(5);
#pragma unroll
          for (int k4 = 0; k4 < kHD / 16; ++k4) {
            umma_bf16<1>(tS, make_smem_desc(sQ + k4 * 32, 16, 1024), make_smem_desc(sK + k4 * 32, 16, 1024), idesc_kk, k4 > 0);
          }
#pragma unroll
          for (int k4 = 0; k4 < kHD / 16; ++k4) {
            umma_bf16<1>(tDP, make_smem_desc(sDO + k4 * 32, 16, 1024), make_smem_desc(sV + k4 * 32, 16, 1024), idesc_kk, k4 > 0);
          }
          umma_commit(sdp_full);
          ok = mbar_wait(pds_ready, it & 1, abort_flag, p.status, kStatusWaitEpi);
          if (!ok) break;
          tc_fence_after_sync();
          // dV += P^T dO ; dK += dS^T Q   (M = key index, K = query index: 8 steps of 16 rows)
#pragma unroll
          for (int k8 = 0; k8 < kBlk / 16; ++k8) {
            umma_bf16<1>(tDV, make_smem_desc(sP + k8 * 2048, 16384, 1024), make_smem_desc(sDO + k8 * 2048, 8192, 1024), idesc_mn,
                         (i > i0 || k8 > 0));
          }
#pragma unroll
          for (int k8 = 0; k8 < kBlk / 16; ++k8) {
            umma_bf16<1>(tDK, make_smem_desc(sDS + k8 * 2048, 16384, 1024), make_smem_desc(sQ + k8 * 2048, 8192, 1024), idesc_mn,
                         (i > i0 || k8 > 0));
          }
          // dQ_tile = dS K   (M = query, K = key index)
#pragma unroll
          for (int k8 = 0; k8 < kBlk / 16; ++k8) {
            const uint32_t a = sDS + (k8 >> 2) * 16384 + (k8 & 3) * 32;
            umma_bf16<1>(tDQ, make_smem_desc(a, 16, 1024), make_smem_desc(sK + k8 * 2048, 8192, 1024), idesc_kn, k8 > 0);
          }
          umma_commit(grads_full);
        }
      }
    }
  } else {
    const int t = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t sP = smem_u32(smem + L.P), sDS = smem_u32(smem + L.DS);
    const float sc = p.scale * kLog2e;
    const float inv_keep = p.p_drop > 0.f ? 1.f / (1.f - p.p_drop) : 1.f;
    int it = 0;
    bool ok = true;
    // D = rowsum(dO * O) (eight lanes per row, coalesced) and the LSE of a query row
    auto load_row_stats = [&](int i, float& Dq, float& lse_q) {
      const int q = i * kBlk + t;
      lse_q = q < p.S ? __ldg(lse + (static_cast<long long>(b) * p.H + h) * p.S + q) * kLog2e : 0.f;
      Dq = row_dot64(o + static_cast<long long>(b) * p.osb + static_cast<long long>(h) * p.osh,
                     d_o + static_cast<long long>(b) * p.osb + static_cast<long long>(h) * p.osh, p.oss, i * kBlk + warp * 32, p.S, lane);
    };
    float D_first = 0.f, lse_first = 0.f;
    for (int j = 0; j < nblk && ok; ++j) {
      const int kv0 = j * kBlk;
      const int i0 = p.causal ? j : 0;
      asm volatile("bar.sync 1, 128;");
      {
        const int kv = kv0 + t;
        // the mask load, and with a single key block the row statistics too, are in flight together
        const float mraw = (kv < p.S && p.mask) ? __ldg(p.mask + static_cast<long long>(b) * p.S + kv) : 0.f;
        if constexpr (kSingle) load_row_stats(0, D_first, lse_first);
        mask_s[t] = (kv < p.S) ? mraw * kLog2e : -INFINITY;
      }
      asm volatile("bar.sync 1, 128;");
      if (kSingle && t == 0) FB_ATTN_TS(6);
      for (int i = i0; i < nblk && ok; ++i, ++it) {
        const int q = i * kBlk + t;
        const bool q_ok = q < p.S;
        float Dq = D_first, lse_q = lse_first;
        if constexpr (!kSingle) load_row_stats(i, Dq, lse_q);
        if (kSingle && t == 0) FB_ATTN_TS(9);
        ok = mbar_wait(sdp_full, it & 1, abort_flag, p.status, kStatusWaitAccum);
        if (!ok) break;
        tc_fence_after_sync();
        if (kSingle && t == 0) FB_ATTN_TS(10);
#pragma unroll 1
        for (int c = 0; c < kBlk; c += 32) {
          uint32_t sv[32], dpv[32];
          tmem_ld32(tS + lane_base + c, sv);
          tmem_ld32(tDP + lane_base + c, dpv);
          tmem_ld_wait();
          float pr[32], ds[32];
          float z[32];
          if (p.p_drop > 0.f) {
            const unsigned long long base = ((static_cast<unsigned long long>(b) * p.H + h) * p.S + q) * p.S + kv0 + c;
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              float s4[4];
              dropout_scale4(seed, base + e, p.p_drop, inv_keep, s4);
#pragma unroll
              for (int k = 0; k < 4; ++k) z[e + k] = s4[k];
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) z[e] = 1.f;
          }
          const bool row_live = q_ok && lse_q != -INFINITY;
#pragma unroll
          for (int e4 = 0; e4 < 32; e4 += 4) {
            const float4 mk = *reinterpret_cast<const float4*>(mask_s + c + e4);
            const float mk4[4] = {mk.x - lse_q, mk.y - lse_q, mk.z - lse_q, mk.w - lse_q};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int e = e4 + k;
              float s = __uint_as_float(sv[e]) * sc + mk4[k];   // score - log-sum-exp in one FMA
              if (p.causal && kv0 + c + e > q) s = -INFINITY;
              const float pe = row_live ? exp2f(s) : 0.f;
              const float dpe = __uint_as_float(dpv[e]) * z[e];
              pr[e] = pe * z[e];
              ds[e] = pe * (dpe - Dq) * p.scale;
            }
          }
          const uint32_t pp = sP + (c >> 6) * 16384, dp = sDS + (c >> 6) * 16384;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            st_shared_v4(swz_chunk(pp, t, ((c & 63) >> 3) + g), pack8(pr + 8 * g));
            st_shared_v4(swz_chunk(dp, t, ((c & 63) >> 3) + g), pack8(ds + 8 * g));
          }
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        if (kSingle && t == 0) FB_ATTN_TS(11);
        mbar_arrive(pds_ready);
        ok = __all_sync(0xffffffffu, mbar_wait(grads_full, it & 1, abort_flag, p.status, kStatusWaitAccum));   // warp-uniform: staged stores below
        if (!ok) break;
        tc_fence_after_sync();
        if (kSingle && t == 0) FB_ATTN_TS(12);
        // ---- dQ tile: last key block of this query block -> bf16 rows through the staging area (the P panels are dead:
        //      every MMA of this tile has completed); otherwise accumulate in the fp32 scratch
        const uint32_t stage = sP + warp * 4096;
        {
          const int j_first = 0;
          const int j_last = p.causal ? min(i, nblk - 1) : nblk - 1;
          float* acc_row = dq_accum ? dq_accum + ((static_cast<long long>(b) * p.H + h) * p.S + q) * kHD : nullptr;
#pragma unroll
          for (int c = 0; c < kHD; c += 32) {
            uint32_t v[32];
            tmem_ld32(tDQ + lane_base + c, v);
            tmem_ld_wait();
            float f[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
            if (q_ok && j != j_first) {
#pragma unroll
              for (int e = 0; e < 32; e += 4) {
                float4 old = *reinterpret_cast<const float4*>(acc_row + c + e);
                f[e] += old.x; f[e + 1] += old.y; f[e + 2] += old.z; f[e + 3] += old.w;
              }
            }
            if (j == j_last) {
              stage_half(stage, lane, c, f);
            } else if (q_ok) {
#pragma unroll
              for (int e = 0; e < 32; e += 4)
                *reinterpret_cast<float4*>(acc_row + c + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
            }
          }
          if (j == j_last)
            flush_rows(stage, lane, dq + static_cast<long long>(b) * p.gsb + static_cast<long long>(h) * p.gsh, p.gss, i * kBlk + warp * 32, p.S);
        }
        // ---- last query block of this key block: drain dK, dV the same way
        if (i == nblk - 1) {
          __nv_bfloat16* const bases[2] = {dk + static_cast<long long>(b) * p.gsb + static_cast<long long>(h) * p.gsh,
                                            dv + static_cast<long long>(b) * p.gsb + static_cast<long long>(h) * p.gsh};
#pragma unroll
          for (int which = 0; which < 2; ++which) {
#pragma unroll
            for (int c = 0; c < kHD; c += 32) {
              uint32_t v[32];
              tmem_ld32((which == 0 ? tDK : tDV) + lane_base + c, v);
              tmem_ld_wait();
              float f[32];
#pragma unroll
              for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
              stage_half(stage, lane, c, f);
            }
            flush_rows(stage, lane, bases[which], p.gss, kv0 + warp * 32, p.S);
          }
        }
        tc_fence_before_sync();
        mbar_arrive(tile_done);
      }
    }
  }
  if (kSingle && threadIdx.x == 0) FB_ATTN_TS(13);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

static AttnParams make_params(int B, int H, int S, const long long* qs, const long long* os, const long long* gs, const float* mask,
                              float scale, int causal, float p_drop, unsigned long long seed,
                              const unsigned long long* seed_dev, int* status) {
  AttnParams p;
  p.B = B; p.H = H; p.S = S; p.sb = qs[0]; p.ss = qs[1]; p.sh = qs[2]; p.mask = mask;
  p.osb = os[0]; p.oss = os[1]; p.osh = os[2];
  p.gsb = gs[0]; p.gss = gs[1]; p.gsh = gs[2]; p.scale = scale; p.causal = causal;
  p.p_drop = p_drop; p.seed = seed; p.seed_dev = seed_dev; p.status = status;
  return p;
}

static bool strides_ok(const void* ptr, long long sb, long long ss, long long sh) {
  return (reinterpret_cast<uintptr_t>(ptr) % 16 == 0) && sb % 8 == 0 && ss % 8 == 0 && sh % 8 == 0;
}

}  // namespace fb

#if FB_TIMELINE
extern "C" int fb_attn_timeline(long long* host_out, int count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host_out, fb::g_attn_ts, sizeof(long long) * static_cast<size_t>(count)));
}
#endif

extern "C" int fb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const float* mask, int B, int H,
                           int S, const long long* qkv_strides, const long long* o_strides, float scale, int causal,
                           float p_drop, unsigned long long seed, const unsigned long long* seed_dev, int* status,
                           void* stream) {
  using namespace fb;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  const long long sb = qkv_strides[0], ss = qkv_strides[1], sh = qkv_strides[2];
  if (!strides_ok(q, sb, ss, sh) || !strides_ok(k, sb, ss, sh) || !strides_ok(v, sb, ss, sh) ||
      !strides_ok(o, o_strides[0], o_strides[1], o_strides[2]))
    return -3;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_bshd(&tq, q, B, H, S, sb, ss, sh))) return r;
  if ((r = make_tmap_bshd(&tk, k, B, H, S, sb, ss, sh))) return r;
  if ((r = make_tmap_bshd(&tv, v, B, H, S, sb, ss, sh))) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem(false).TOTAL + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem(true).TOTAL + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const bool single = S <= kBlk;
  const int smem_bytes = FwdSmem(single).TOTAL + 1024;
  AttnParams p = make_params(B, H, S, qkv_strides, o_strides, o_strides, mask, scale, causal, p_drop, seed, seed_dev, status);
  dim3 grid((S + kBlk - 1) / kBlk, H, B);
  cudaError_t le;
  if (single)
    le = launch_pdl(attn_fwd_kernel<true>, grid, dim3(kAttnThreads), smem_bytes, static_cast<cudaStream_t>(stream), tq, tk, tv, static_cast<__nv_bfloat16*>(o), lse, p);
  else
    le = launch_pdl(attn_fwd_kernel<false>, grid, dim3(kAttnThreads), smem_bytes, static_cast<cudaStream_t>(stream), tq, tk, tv, static_cast<__nv_bfloat16*>(o), lse, p);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

// dq_accum: fp32 scratch [B, H, S, 64]; only touched when a query block meets more than one key block
// (S > 128), may be null otherwise.
extern "C" int fb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                           const float* mask, void* dq, void* dk, void* dv, float* dq_accum, int B, int H, int S,
                           const long long* qkv_strides, const long long* o_strides, const long long* g_strides,
                           float scale, int causal, float p_drop, unsigned long long seed,
                           const unsigned long long* seed_dev, int* status, void* stream) {
  using namespace fb;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  if (S > kBlk && !dq_accum) return -4;
  const long long sb = qkv_strides[0], ss = qkv_strides[1], sh = qkv_strides[2];
  if (!strides_ok(q, sb, ss, sh) || !strides_ok(k, sb, ss, sh) || !strides_ok(v, sb, ss, sh)) return -3;
  if (!strides_ok(o, o_strides[0], o_strides[1], o_strides[2]) || !strides_ok(d_o, o_strides[0], o_strides[1], o_strides[2])) return -3;
  if (!strides_ok(dq, g_strides[0], g_strides[1], g_strides[2]) || !strides_ok(dk, g_strides[0], g_strides[1], g_strides[2]) ||
      !strides_ok(dv, g_strides[0], g_strides[1], g_strides[2]))
    return -3;
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_tmap_bshd(&tq, q, B, H, S, sb, ss, sh))) return r;
  if ((r = make_tmap_bshd(&tk, k, B, H, S, sb, ss, sh))) return r;
  if ((r = make_tmap_bshd(&tv, v, B, H, S, sb, ss, sh))) return r;
  if ((r = make_tmap_bshd(&tdo, d_o, B, H, S, o_strides[0], o_strides[1], o_strides[2]))) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem(false).TOTAL + 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem(true).TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  AttnParams p = make_params(B, H, S, qkv_strides, o_strides, g_strides, mask, scale, causal, p_drop, seed, seed_dev, status);
  dim3 grid(H, B);
  cudaError_t le;
  if (S <= kBlk)
    le = launch_pdl(attn_bwd_kernel<true>, grid, dim3(kAttnThreads), static_cast<size_t>(BwdSmem(true).TOTAL), static_cast<cudaStream_t>(stream),
                    tq, tk, tv, tdo, static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), lse,
                    static_cast<__nv_bfloat16*>(dq), static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), dq_accum, p);
  else
    le = launch_pdl(attn_bwd_kernel<false>, grid, dim3(kAttnThreads), static_cast<size_t>(BwdSmem(false).TOTAL + 1024), static_cast<cudaStream_t>(stream),
                    tq, tk, tv, tdo, static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), lse,
                    static_cast<__nv_bfloat16*>(dq), static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), dq_accum, p);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}
