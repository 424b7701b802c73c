/* C ABI of the flodl-b200 native library.
 *
 * Plays the role of the reference's C shim header (flodl-sys/shim.h): a flat `extern "C"` surface
 * that a binding in any language can call. Where the shim forwards to libtorch, these entry points
 * launch this library's own sm_100a kernels. Conventions:
 *   - every function returns 0 on success, a cudaError_t (> 0) from the launch, or a negative
 *     code for a rejected argument (-2 dtype/mode, -3 alignment, -4 unsupported shape, -5 world);
 *   - pointers are device pointers unless a comment says otherwise;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - nothing here allocates device memory unless its comment says so.
 */
#ifndef FLODL_B200_H_
#define FLODL_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

/* dtype / device tags: same numbering as the reference ABI (flodl-sys/shim.h:920-929). */
#define FLODL_FLOAT16 5
#define FLODL_BFLOAT16 15
#define FLODL_FLOAT32 6
#define FLODL_FLOAT64 7
#define FLODL_INT32 3
#define FLODL_INT64 4
#define FLODL_CPU 0
#define FLODL_CUDA 1

/* GEMM epilogues */
#define FB_EPI_NONE 0
#define FB_EPI_GELU_ERF 1    /* C = gelu(acc + bias); aux (optional) receives acc + bias   */
#define FB_EPI_DGELU_ERF 2   /* C = acc * gelu'(aux)                                        */
#define FB_EPI_GELU_TANH 3
#define FB_EPI_DGELU_TANH 4

/* symmetric-memory collectives */
#define FB_MAX_RANKS 16
#define FB_MAX_BLOCKS 256
#define FB_SIGNAL_POISON_INDEX (FB_MAX_BLOCKS * FB_MAX_RANKS)   /* uint32 index of the "a peer gave up" word */
#define FB_SIGNAL_PAD_BYTES (FB_MAX_BLOCKS * FB_MAX_RANKS * 4 + 256)

typedef struct fb_symm_ctx {
  void* data[FB_MAX_RANKS];  /* peer-mapped payload buffers, indexed by rank            */
  void* sig[FB_MAX_RANKS];   /* peer-mapped signal pads (FB_SIGNAL_PAD_BYTES, zeroed)    */
  void* epochs;              /* local: FB_MAX_BLOCKS uint32, zeroed                      */
  const void* abort;         /* optional device-visible int the host may set to 1        */
  void* status;              /* int: 0 ok, else the code of the wait that gave up (may be host-mapped) */
  void* status_dev;          /* optional device-memory copy of the same word, for kernels that
                                must look at it on their hot path (the optimizers' `skip`) */
  long long timeout_ns;      /* bound of every device-side wait; 0 = 2 s                 */
  void* mc;                  /* multicast (NVLS) address of the payload buffer, or NULL  */
  int rank, world;
} fb_symm_ctx;

/* ---- tensor-core GEMM: D[m,n] = sum_k A(m,k) B(n,k) (bf16 in, fp32 accumulate) ------------ */
/* a_mn = 0: A is [M][lda] (K contiguous); a_mn = 1: A is [K][lda] (M contiguous). Same for B/N.
 * lda, ldb multiples of 8; A, B 16-byte aligned. config: -1 auto, 0 = CTA pair 256x256,
 * 1 = 128x256, 2 = 128x128, 3 = 128x64. split_k > 1 needs c_fp32 and adds into C atomically. */
int fb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_mn, int b_mn, int c_fp32, const void* bias, int bias_fp32, int epi,
                 void* aux, long long ldaux, const float* alpha, int accumulate, int split_k, int config,
                 int* status, void* stream);
/* Same, plus an optional device buffer of 8 int64 per CTA that receives a coarse timeline (tuning aid). */
int fb_gemm_bf16_ts(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                    long long ldc, int a_mn, int b_mn, int c_fp32, const void* bias, int bias_fp32, int epi,
                    void* aux, long long ldaux, const float* alpha, int accumulate, int split_k, int config,
                    int* status, long long* ts, void* stream);
/* Same, with device-side problem sizes: the kernel works on min(M, *m_dyn) rows and min(K, *k_dyn) of the
 * reduction (either pointer may be NULL). The values are read on the device after the preceding kernels of
 * the stream have finished, so a captured graph replays with whatever an earlier kernel computed. Rows of
 * A past *m_dyn inside the last tile, and rows of both operands past *k_dyn inside the last 64-wide K
 * block, are still read: the producer of the operands zero-fills them. */
int fb_gemm_bf16_dyn(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int a_mn, int b_mn, int c_fp32, const void* bias, int bias_fp32, int epi,
                     void* aux, long long ldaux, const float* alpha, int accumulate, int split_k, int config,
                     int* status, long long* ts, const int* m_dyn, const int* k_dyn, void* stream);
int fb_gemm_pick_config(int M, int N, int K, int split_k);

/* ---- attention ----------------------------------------------------------------------------- */
/* q,k,v,o,do,dq,dk,dv: bf16 [B, S, H, 64] with the given element strides for (batch, seq, head);
 * Strides are host arrays {batch, seq, head} in elements (multiples of 8); q/k/v share one set, o/dO another,
 * dq/dk/dv a third. mask: optional fp32 additive [B, S] key mask. lse: fp32 [B, H, S]. */
int fb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const float* mask, int B, int H,
                int S, const long long* qkv_strides, const long long* o_strides, float scale, int causal, float p_drop,
                unsigned long long seed, const unsigned long long* seed_dev, int* status, void* stream);
int fb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                const float* mask, void* dq, void* dk, void* dv, float* dq_accum, int B, int H, int S,
                const long long* qkv_strides, const long long* o_strides, const long long* g_strides, float scale,
                int causal, float p_drop, unsigned long long seed, const unsigned long long* seed_dev, int* status,
                void* stream);

/* ---- normalisation / activation / loss ----------------------------------------------------- */
int fb_layernorm_fwd(const void* x, const void* residual, const float* gamma, const float* beta, void* y,
                     void* pre_out, float* mean, float* rstd, int rows, int cols, float eps, float p_drop,
                     unsigned long long seed, const unsigned long long* seed_dev, int is_bf16, void* stream);
int fb_layernorm_bwd_grid(int rows);
int fb_layernorm_bwd(const void* dy, const void* pre, const float* mean, const float* rstd, const float* gamma,
                     void* dpre, void* dx_drop, float* partial, float* dgamma, float* dbeta, int accumulate,
                     int rows, int cols, float p_drop, unsigned long long seed, const unsigned long long* seed_dev, int is_bf16,
                     void* stream);
int fb_gelu_fwd(const void* x, void* y, long long n, int tanh_approx, int is_bf16, void* stream);
int fb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int tanh_approx, int is_bf16, void* stream);
int fb_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, const unsigned long long* seed_dev,
               int is_bf16, void* stream);
/* out[c] += sum over rows of x[r][c] (the caller zeroes `out`, or passes a gradient slot to accumulate into). */
int fb_colsum(const void* x, float* out, int rows, int cols, long long ld, int is_bf16, void* stream);
/* As fb_colsum over the first min(rows, *rows_dyn) rows (device-side count). */
int fb_colsum_dyn(const void* x, float* out, int rows, int cols, long long ld, int is_bf16, const int* rows_dyn, void* stream);
/* Row compaction for losses that ignore most rows (masked-LM): idx[i] = position of the i-th row whose target is
 * not `ignore_index`, targets_c[i] its target (ignore_index past the count), counts = {n, n rounded up to 256 and
 * clipped to rows}. One launch; idx and targets_c hold `rows` entries. */
int fb_compact_targets(const long long* targets, int rows, long long ignore_index, int* idx, long long* targets_c,
                       int* counts, void* stream);
/* xc[i] = x[idx[i]] for i < counts[0], zero rows up to counts[1], later rows untouched (bf16 or fp32 rows of `cols`). */
int fb_gather_rows(const void* x, long long ld, const int* idx, const int* counts, void* xc, long long ldc, int rows,
                   int cols, int is_bf16, void* stream);
/* dx[idx[i]] = dxc[i] for i < counts[0]; dx must be zeroed by the caller. */
int fb_scatter_rows(const void* dxc, long long ldc, const int* idx, const int* counts, void* dx, long long ld, int rows,
                    int cols, int is_bf16, void* stream);
int fb_embedding_bwd(const void* dy, const long long* ids, float* dw, long long tokens, int dim, long long vocab,
                     long long padding_idx, int is_bf16, void* stream);
int fb_cast(const void* x, void* y, long long n, float scale, int in_bf16, int out_bf16, void* stream);
int fb_softmax_ce(const void* logits, long long ld, const long long* targets, int rows, int V,
                  long long ignore_index, void* dlogits, long long ldd, float* count_inv, float* row_loss,
                  float* loss, int is_bf16, void* stream);
/* As fb_softmax_ce for compacted rows: `counts` = {n, n_pad} on the device; rows past n_pad are neither read nor
 * written, rows in [n, n_pad) get a zero gradient. */
int fb_softmax_ce_dyn(const void* logits, long long ld, const long long* targets, int rows, int V,
                      long long ignore_index, void* dlogits, long long ldd, float* count_inv, float* row_loss,
                      float* loss, int is_bf16, const int* counts, void* stream);
int fb_scale_rows(void* x, long long ld, int rows, int cols, const float* scalar, int is_bf16, void* stream);

/* ---- batch norm (NCHW, training), fused ReLU / residual add --------------------------------- */
/* Convolution filter gradient for channels-last bf16 tensors on the tensor cores (csrc/kernels/conv_tcgen05.cu).
   x: [N,H,W,Ci], dy: [N,Ho,Wo,Co]; dw: [Co][kh][kw][Ci] fp32, the gradient is added to it. */
int fb_conv_wgrad_supported(int N, int H, int W, int Ci, int Co, int kh, int kw, int stride, int pad);
int fb_conv_wgrad(const void* x, const void* dy, float* dw, int N, int H, int W, int Ci, int Co, int kh, int kw,
                  int stride, int pad, int* status, void* stream);

/* Forward convolution and stride-1 data gradient for channels-last bf16 tensors (same file). The filter is
   bf16 [Co][k][k][Ci]. `stats` (optional, fp32 [2][Co], zeroed by the caller) receives the per-channel sum
   and sum of squares of the rounded outputs, for the batch normalisation that follows. */
int fb_conv_fprop_supported(int N, int H, int W, int Ci, int Co, int k, int stride, int pad);
int fb_conv_fprop(const void* x, const void* w, void* y, float* stats, int N, int H, int W, int Ci, int Co, int k, int stride,
                  int pad, int* status, void* stream);
/* fb_conv_fprop for the 3x3 stride-1 kernel with a timeline: `ts` (64 int64, device) receives nanosecond
   timestamps of CTA 0: [0] start, [1] after the dependency wait, [2+i] loads of tile i issued,
   [12+i] tile i landed, [22+i] its MMAs issued, [32+i] accumulator ready, [42+i] stored, [52] end. */
int fb_conv_fprop_ts(const void* x, const void* w, void* y, float* stats, int N, int H, int W, int Ci, int Co, int k, int stride,
                     int pad, int* status, long long* ts, void* stream);
int fb_conv_dgrad_supported(int N, int H, int W, int Ci, int Co, int k, int stride, int pad);
int fb_conv_dgrad(const void* dy, const void* w, void* dx, int N, int H, int W, int Ci, int Co, int k, int stride, int pad,
                  int* status, void* stream);
int fb_bn_nhwc_scratch_floats(int C);
int fb_bn_nhwc_fwd(const void* x, const void* residual, const float* gamma, const float* beta, float* running_mean,
                   float* running_var, void* y, float* save_mean, float* save_rstd, float* scratch, unsigned int* counter,
                   long long P, int C, float eps, float momentum, int relu, int training, int is_bf16, void* stream);
int fb_bn_nhwc_fwd_sums(const void* x, const void* residual, const float* gamma, const float* beta, float* running_mean,
                        float* running_var, void* y, float* save_mean, float* save_rstd, const float* sums, long long P, int C,
                        float eps, float momentum, int relu, int is_bf16, void* stream);
int fb_bn_nhwc_bwd(const void* dy, const void* x, const void* y, const float* gamma, const float* save_mean,
                   const float* save_rstd, void* dx, void* dresidual, float* dgamma, float* dbeta, int accumulate,
                   float* scratch, unsigned int* counter, long long P, int C, int relu, int is_bf16, void* stream);
int fb_bn_scratch_floats(int C);
int fb_bn_fwd(const void* x, const void* residual, const float* gamma, const float* beta, float* running_mean,
              float* running_var, void* y, float* save_mean, float* save_rstd, float* scratch, int N, int C, int HW,
              float eps, float momentum, int relu, int training, int is_bf16, void* stream);
int fb_bn_bwd(const void* dy, const void* x, const void* y, const float* gamma, const float* save_mean,
              const float* save_rstd, void* dx, void* dresidual, float* dgamma, float* dbeta, int accumulate,
              float* scratch, int N, int C, int HW, int relu, int is_bf16, void* stream);

/* ---- optimizers / gradient norm -------------------------------------------------------------- */
/* `skip` (optional, device-visible int): when it reads non-zero the launch changes nothing. The
 * collectives raise such a word when a bounded wait gave up, so un-reduced gradients are never applied. */
int fb_adam_step(float* p, const void* g, float* m, float* v, void* p16, long long n, const float* hyper, float b1,
                 float b2, float eps, const float* grad_scale, int g_bf16, const int* skip, void* stream);
/* fb_adam_step with hyper = {lr, 1-b1^t, 1-b2^t, weight_decay} read from HOST memory at launch (no bf16 shadow, no skip word). */
int fb_adam_step_host(float* p, const void* g, float* m, float* v, long long n, const float* hyper_host, float b1, float b2,
                      float eps, int g_bf16, void* stream);
int fb_sgd_step(float* p, const void* g, float* buf, void* p16, long long n, const float* hyper,
                const float* grad_scale, int g_bf16, const int* skip, void* stream);
int fb_grad_norm_parts(long long n);
int fb_grad_norm(const void* g, long long n, float* partial, float max_norm, float extra_scale, float* out,
                 int is_bf16, void* stream);

/* Gradient norm without any allocation (this entry point has no counterpart in the reference).
 * For callers that cannot obtain device memory at the point of the call: a step being captured
 * into a CUDA graph by someone who owns no memory pool, a thread that must keep away from the
 * allocator while a collective is in flight, or a non-PyTorch host of this C ABI that has no
 * allocator to lend. Same result as fb_grad_norm; the per-block partial sums live in a fixed
 * 4 KB array inside the library (held on every GPU that loads it until the process exits).
 *   - n above FB_GRAD_NORM_NOALLOC_MAX_ELEMS is rejected with -4;
 *   - the first call on a device resolves the array's address (with that device current): make it
 *     before any stream capture. Two threads making that first call together is harmless (both
 *     store the same address in an atomic slot);
 *   - every call reuses the array, so calls that may overlap on the GPU must be ordered by the
 *     caller; nothing needs clearing between calls. */
#define FB_GRAD_NORM_NOALLOC_MAX_ELEMS (1LL << 31)
int fb_grad_norm_noalloc(const void* g, long long n, float max_norm, float extra_scale, float* out, int is_bf16,
                         void* stream);
long long fb_grad_norm_noalloc_max(void);

/* ---- bounds-checked debug build ----------------------------------------------------------------
 * Built with FLODL_BOUNDS_CHECK=1, kernels range-check every index they read from device memory and
 * record the first violation as {site, index, limit} instead of making the access. `dev_word` is a
 * device-visible int[4] (host-mapped memory works); attach it once per translation unit. In a
 * regular build the attach functions do nothing. */
int fb_bounds_attach_elementwise(int* dev_word);
int fb_bounds_attach_softmax_ce(int* dev_word);

/* ---- collectives over peer-mapped buffers ---------------------------------------------------- */
int fb_allreduce(const fb_symm_ctx* ctx, long long byte_off, long long n, int is_bf16, const float* weights,
                 int blocks, void* stream);
int fb_allreduce_oneshot(const fb_symm_ctx* ctx, long long byte_off, long long n, int in_bf16, void* out,
                         int out_bf16, const float* weights, int blocks, void* stream);
int fb_param_average(const fb_symm_ctx* params, const fb_symm_ctx* staging, long long n, const float* weights,
                     float alpha, void* p16, float* partial, unsigned int* counter, float* out2, int blocks,
                     void* stream);
int fb_broadcast(const fb_symm_ctx* ctx, long long byte_off, long long nbytes, int root, int blocks, void* stream);
int fb_symm_barrier(const fb_symm_ctx* ctx, int blocks, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLODL_B200_H_ */
