// pybind11 bindings: torch tensors in, `fb_*` kernel launches out (on the current CUDA stream).
// No logic lives here beyond argument checking; the kernels are in csrc/kernels and csrc/comm.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <array>
#include <optional>
#include <vector>

#include "flodl_b200.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

void check(int rc, const char* what) {
  if (rc == 0) return;
  if (rc > 0) {
    TORCH_CHECK(false, what, ": CUDA error ", rc, " (", cudaGetErrorString(static_cast<cudaError_t>(rc)), ")");
  }
  TORCH_CHECK(false, what, ": rejected arguments (code ", rc, ")");
}

bool is_bf16(const Tensor& t) { return t.scalar_type() == at::kBFloat16; }
void want_cuda(const Tensor& t, const char* name) { TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor"); }
void want_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name, " must be a contiguous fp32 CUDA tensor");
}
void want_float_kind(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && (t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16), name,
              " must be fp32 or bf16 on CUDA");
}
template <typename T = void>
T* ptr(const OptTensor& t) { return t.has_value() ? static_cast<T*>(t->data_ptr()) : nullptr; }

const unsigned long long* seed_ptr(const OptTensor& t) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->numel() == 1, "seed_dev must be one int64 on CUDA");
  return reinterpret_cast<const unsigned long long*>(t->data_ptr());
}

// one status word per device, shared by every kernel that has bounded waits
Tensor& status_word(int device) {
  static std::vector<Tensor> words(64);
  TORCH_CHECK(device >= 0 && device < 64);
  if (!words[device].defined())
    words[device] = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device];
}

// ------------------------------------------------------------------------------------------ GEMM
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, const OptTensor& bias, int epi,
          const OptTensor& aux, const OptTensor& alpha, bool accumulate, int split_k, int config, const OptTensor& ts,
          const OptTensor& m_dyn, const OptTensor& k_dyn) {
  want_cuda(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(is_bf16(a) && is_bf16(b), "gemm operands must be bf16");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm takes 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm needs unit inner strides");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm K mismatch: ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm output shape mismatch");
  TORCH_CHECK(out.scalar_type() == at::kFloat || is_bf16(out), "gemm output must be fp32 or bf16");
  if (bias.has_value()) TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be [N]");
  if (aux.has_value()) TORCH_CHECK(is_bf16(*aux) && aux->stride(1) == 1 && aux->size(0) == M && aux->size(1) == N, "aux must be bf16 [M,N]");
  if (alpha.has_value()) TORCH_CHECK(alpha->scalar_type() == at::kFloat && alpha->numel() == 1, "alpha must be one fp32");
  Tensor& st = status_word(a.get_device());
  if (ts.has_value()) TORCH_CHECK(ts->is_cuda() && ts->scalar_type() == at::kLong && ts->numel() >= 8 * 160, "ts must be int64 [>=1280]");
  auto dyn_ptr = [](const OptTensor& t) -> const int* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->numel() >= 1, "dynamic size must be an int32 CUDA tensor");
    return t->data_ptr<int>();
  };
  int rc = fb_gemm_bf16_dyn(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                        out.stride(0), a_mn, b_mn, out.scalar_type() == at::kFloat, ptr<const void>(bias),
                        bias.has_value() && bias->scalar_type() == at::kFloat, epi, ptr<void>(aux),
                        aux.has_value() ? aux->stride(0) : 0, ptr<const float>(alpha), accumulate, split_k, config,
                        st.data_ptr<int>(), ts.has_value() ? reinterpret_cast<long long*>(ts->data_ptr<int64_t>()) : nullptr,
                        dyn_ptr(m_dyn), dyn_ptr(k_dyn), stream_of(a));
  check(rc, "fb_gemm_bf16");
}

int gemm_pick_config(int M, int N, int K, int split_k) { return fb_gemm_pick_config(M, N, K, split_k); }

// Bounds-check record of the debug build (FLODL_BOUNDS_CHECK): one host-mapped int[4] = {site, index, limit, 0}.
int* bounds_word(bool create) {
  static int* host = nullptr;
  if (!host && create) {
    int* dev = nullptr;
    TORCH_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host), 4 * sizeof(int), cudaHostAllocMapped) == cudaSuccess, "cudaHostAlloc");
    host[0] = host[1] = host[2] = host[3] = 0;
    TORCH_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev), host, 0) == cudaSuccess, "cudaHostGetDevicePointer");
    check(fb_bounds_attach_elementwise(dev), "fb_bounds_attach_elementwise");
    check(fb_bounds_attach_softmax_ce(dev), "fb_bounds_attach_softmax_ce");
  }
  return host;
}
bool bounds_check_build() {
#ifdef FLODL_BOUNDS_CHECK
  return FLODL_BOUNDS_CHECK != 0;
#else
  return false;
#endif
}
// (site, index, limit) of the first recorded violation, or (0, 0, 0); `clear` re-arms the record.
std::array<int, 3> bounds_report(bool clear) {
  int* w = bounds_word(true);
  cudaDeviceSynchronize();
  std::array<int, 3> r = {w[0], w[1], w[2]};
  if (clear) w[0] = w[1] = w[2] = 0;
  return r;
}

int read_status(int device) {
  return status_word(device).item<int>();
}
void clear_status(int device) { status_word(device).zero_(); }

// ------------------------------------------------------------------------------------- LayerNorm
std::vector<Tensor> layernorm_fwd(const Tensor& x, const OptTensor& residual, const OptTensor& gamma,
                                  const OptTensor& beta, double eps, double p_drop, uint64_t seed, bool want_pre,
                                  const OptTensor& seed_dev) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
  const int64_t cols = x.size(-1);
  const int64_t rows = x.numel() / cols;
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == x.scalar_type() && residual->numel() == x.numel());
  if (gamma.has_value()) want_f32(*gamma, "gamma");
  if (beta.has_value()) want_f32(*beta, "beta");
  Tensor y = torch::empty_like(x);
  Tensor pre = want_pre ? torch::empty_like(x) : Tensor();
  auto fopts = torch::dtype(torch::kFloat).device(x.device());
  Tensor mean = torch::empty({rows}, fopts), rstd = torch::empty({rows}, fopts);
  int rc = fb_layernorm_fwd(x.data_ptr(), ptr<const void>(residual), ptr<const float>(gamma), ptr<const float>(beta),
                            y.data_ptr(), want_pre ? pre.data_ptr() : nullptr, mean.data_ptr<float>(),
                            rstd.data_ptr<float>(), (int)rows, (int)cols, (float)eps, (float)p_drop, seed, seed_ptr(seed_dev), is_bf16(x),
                            stream_of(x));
  check(rc, "fb_layernorm_fwd");
  return {y, pre, mean, rstd};
}

// returns {dpre, dx_drop (or undefined), dgamma, dbeta}
std::vector<Tensor> layernorm_bwd(const Tensor& dy, const Tensor& pre, const Tensor& mean, const Tensor& rstd,
                                  const OptTensor& gamma, double p_drop, uint64_t seed, bool want_dx_drop,
                                  bool want_param_grads, const OptTensor& dgamma_acc, const OptTensor& dbeta_acc,
                                  const OptTensor& seed_dev) {
  want_float_kind(dy, "dy");
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dy.is_contiguous() && pre.is_contiguous() && dy.scalar_type() == pre.scalar_type());
  const int64_t cols = dy.size(-1);
  const int64_t rows = dy.numel() / cols;
  Tensor dpre = torch::empty_like(dy);
  Tensor dxd = want_dx_drop ? torch::empty_like(dy) : Tensor();
  auto fopts = torch::dtype(torch::kFloat).device(dy.device());
  Tensor partial, dgamma, dbeta;
  bool accumulate = false;
  if (want_param_grads) {
    const int grid = fb_layernorm_bwd_grid((int)rows);
    partial = torch::empty({grid, 2, cols}, fopts);
    if (dgamma_acc.has_value()) {
      want_f32(*dgamma_acc, "dgamma_acc");
      want_f32(*dbeta_acc, "dbeta_acc");
      dgamma = *dgamma_acc;
      dbeta = *dbeta_acc;
      accumulate = true;
    } else {
      dgamma = torch::empty({cols}, fopts);
      dbeta = torch::empty({cols}, fopts);
    }
  }
  int rc = fb_layernorm_bwd(dy.data_ptr(), pre.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                            ptr<const float>(gamma), dpre.data_ptr(), want_dx_drop ? dxd.data_ptr() : nullptr,
                            want_param_grads ? partial.data_ptr<float>() : nullptr,
                            want_param_grads ? dgamma.data_ptr<float>() : nullptr,
                            want_param_grads ? dbeta.data_ptr<float>() : nullptr, accumulate, (int)rows, (int)cols,
                            (float)p_drop, seed, seed_ptr(seed_dev), is_bf16(dy), stream_of(dy));
  check(rc, "fb_layernorm_bwd");
  return {dpre, dxd, dgamma, dbeta};
}

// --------------------------------------------------------------------------------- elementwise
Tensor gelu_fwd(const Tensor& x, bool tanh_approx) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous());
  Tensor y = torch::empty_like(x);
  check(fb_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), tanh_approx, is_bf16(x), stream_of(x)), "fb_gelu_fwd");
  return y;
}
Tensor gelu_bwd(const Tensor& dy, const Tensor& x, bool tanh_approx) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dy.scalar_type() == x.scalar_type());
  Tensor dx = torch::empty_like(x);
  check(fb_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), tanh_approx, is_bf16(x), stream_of(x)), "fb_gelu_bwd");
  return dx;
}
Tensor dropout(const Tensor& x, double p, uint64_t seed, const OptTensor& seed_dev) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous());
  Tensor y = torch::empty_like(x);
  check(fb_dropout(x.data_ptr(), y.data_ptr(), x.numel(), (float)p, seed, seed_ptr(seed_dev), is_bf16(x), stream_of(x)), "fb_dropout");
  return y;
}
void colsum(const Tensor& x, Tensor& out, const OptTensor& rows_dyn) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1);
  want_f32(out, "out");
  TORCH_CHECK(out.numel() == x.size(1));
  if (rows_dyn.has_value()) TORCH_CHECK(rows_dyn->is_cuda() && rows_dyn->scalar_type() == at::kInt);
  check(fb_colsum_dyn(x.data_ptr(), out.data_ptr<float>(), (int)x.size(0), (int)x.size(1), x.stride(0), is_bf16(x),
                      rows_dyn.has_value() ? rows_dyn->data_ptr<int>() : nullptr, stream_of(x)),
        "fb_colsum");
}
// Row compaction (masked-LM): returns {idx int32 [rows], targets_c int64 [rows], counts int32 [2] = {n, n_pad}}.
std::vector<Tensor> compact_targets(const Tensor& targets, int64_t ignore_index) {
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous());
  c10::cuda::CUDAGuard guard(targets.device());
  const int64_t rows = targets.numel();
  Tensor idx = torch::empty({rows}, torch::dtype(torch::kInt32).device(targets.device()));
  Tensor tc = torch::empty({rows}, targets.options());
  Tensor counts = torch::empty({2}, torch::dtype(torch::kInt32).device(targets.device()));
  check(fb_compact_targets(reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), (int)rows, ignore_index, idx.data_ptr<int>(),
                           reinterpret_cast<long long*>(tc.data_ptr<int64_t>()), counts.data_ptr<int>(), stream_of(targets)),
        "fb_compact_targets");
  return {idx, tc, counts};
}
void gather_rows(const Tensor& x, const Tensor& idx, const Tensor& counts, Tensor& xc) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && xc.dim() == 2 && x.stride(1) == 1 && xc.stride(1) == 1 && x.sizes() == xc.sizes() && x.scalar_type() == xc.scalar_type());
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.numel() == x.size(0) && counts.scalar_type() == at::kInt && counts.numel() == 2);
  check(fb_gather_rows(x.data_ptr(), x.stride(0), idx.data_ptr<int>(), counts.data_ptr<int>(), xc.data_ptr(), xc.stride(0), (int)x.size(0),
                       (int)x.size(1), is_bf16(x), stream_of(x)),
        "fb_gather_rows");
}
void scatter_rows(const Tensor& dxc, const Tensor& idx, const Tensor& counts, Tensor& dx) {
  want_float_kind(dxc, "dxc");
  c10::cuda::CUDAGuard guard(dxc.device());
  TORCH_CHECK(dx.dim() == 2 && dxc.dim() == 2 && dx.stride(1) == 1 && dxc.stride(1) == 1 && dx.sizes() == dxc.sizes() && dx.scalar_type() == dxc.scalar_type());
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.numel() == dx.size(0) && counts.scalar_type() == at::kInt && counts.numel() == 2);
  check(fb_scatter_rows(dxc.data_ptr(), dxc.stride(0), idx.data_ptr<int>(), counts.data_ptr<int>(), dx.data_ptr(), dx.stride(0), (int)dx.size(0),
                        (int)dx.size(1), is_bf16(dx), stream_of(dx)),
        "fb_scatter_rows");
}
void embedding_bwd(const Tensor& dy, const Tensor& ids, Tensor& dw, int64_t padding_idx) {
  want_float_kind(dy, "dy");
  want_f32(dw, "dw");
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dy.is_contiguous() && ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous());
  TORCH_CHECK(dw.dim() == 2 && dy.size(-1) == dw.size(1) && dy.numel() / dw.size(1) == ids.numel());
  check(fb_embedding_bwd(dy.data_ptr(), reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dw.data_ptr<float>(), ids.numel(),
                         (int)dw.size(1), dw.size(0), padding_idx, is_bf16(dy), stream_of(dy)),
        "fb_embedding_bwd");
}
void cast_into(const Tensor& x, Tensor& y, double scale) {
  want_float_kind(x, "x");
  want_float_kind(y, "y");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel());
  check(fb_cast(x.data_ptr(), y.data_ptr(), x.numel(), (float)scale, is_bf16(x), is_bf16(y), stream_of(x)), "fb_cast");
}

// ------------------------------------------------------------------------------------------- CE
// logits [rows, V] (unit inner stride). Returns {loss (0-dim fp32), dlogits, count_inv}.
// With `inplace` the gradient overwrites the logits.
std::vector<Tensor> softmax_ce(Tensor& logits, const Tensor& targets, int64_t ignore_index, bool want_grad, bool inplace,
                               const OptTensor& counts) {
  want_float_kind(logits, "logits");
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [rows, V] with unit inner stride");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0));
  const int64_t rows = logits.size(0), V = logits.size(1);
  auto fopts = torch::dtype(torch::kFloat).device(logits.device());
  Tensor count_inv = torch::empty({2}, fopts), row_loss = torch::empty({rows}, fopts), loss = torch::empty({}, fopts);
  Tensor dl;
  if (want_grad) {
    if (inplace) dl = logits;
    else {
      // keep the padded leading dimension so rows stay 16-byte aligned
      const int64_t ld = logits.stride(0);
      dl = torch::empty({rows, ld}, logits.options()).narrow(1, 0, V);
    }
  }
  if (counts.has_value()) TORCH_CHECK(counts->is_cuda() && counts->scalar_type() == at::kInt && counts->numel() == 2);
  int rc = fb_softmax_ce_dyn(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), (int)rows, (int)V, ignore_index,
                             want_grad ? dl.data_ptr() : nullptr, want_grad ? dl.stride(0) : 0, count_inv.data_ptr<float>(),
                             row_loss.data_ptr<float>(), loss.data_ptr<float>(), is_bf16(logits),
                             counts.has_value() ? counts->data_ptr<int>() : nullptr, stream_of(logits));
  check(rc, "fb_softmax_ce");
  return {loss, dl, count_inv};
}
void scale_rows(Tensor& x, const Tensor& scalar) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1);
  TORCH_CHECK(scalar.is_cuda() && scalar.scalar_type() == at::kFloat && scalar.numel() == 1);
  check(fb_scale_rows(x.data_ptr(), x.stride(0), (int)x.size(0), (int)x.size(1), scalar.data_ptr<float>(), is_bf16(x), stream_of(x)), "fb_scale_rows");
}

// ---------------------------------------------------------------------------------- optimizers
void adam_step(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const OptTensor& p16, const Tensor& hyper, double b1,
               double b2, double eps, const OptTensor& grad_scale, uint64_t skip) {
  want_f32(p, "p");
  want_f32(m, "m");
  want_f32(v, "v");
  want_f32(hyper, "hyper");
  c10::cuda::CUDAGuard guard(p.device());
  want_float_kind(g, "g");
  TORCH_CHECK(g.is_contiguous() && g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel() && hyper.numel() >= 4);
  if (p16.has_value()) TORCH_CHECK(is_bf16(*p16) && p16->is_contiguous() && p16->numel() == p.numel());
  check(fb_adam_step(p.data_ptr<float>(), g.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), ptr<void>(p16), p.numel(),
                     hyper.data_ptr<float>(), (float)b1, (float)b2, (float)eps, ptr<const float>(grad_scale), is_bf16(g),
                     reinterpret_cast<const int*>(skip), stream_of(p)),
        "fb_adam_step");
}
// The same update for a list of parameters that do not share a flat buffer: one call from Python, one
// launch per tensor (the per-parameter Python loop cost more than the kernels on small models).
void adam_step_multi(std::vector<Tensor>& ps, const std::vector<Tensor>& gs, std::vector<Tensor>& ms, std::vector<Tensor>& vs,
                     const std::vector<OptTensor>& p16s, const Tensor& hyper, double b1, double b2, double eps,
                     const OptTensor& grad_scale, uint64_t skip) {
  TORCH_CHECK(gs.size() == ps.size() && ms.size() == ps.size() && vs.size() == ps.size() && p16s.size() == ps.size(), "list lengths differ");
  for (size_t i = 0; i < ps.size(); ++i) adam_step(ps[i], gs[i], ms[i], vs[i], p16s[i], hyper, b1, b2, eps, grad_scale, skip);
}
void sgd_step(Tensor& p, const Tensor& g, const OptTensor& buf, const OptTensor& p16, const Tensor& hyper,
              const OptTensor& grad_scale, uint64_t skip) {
  want_f32(p, "p");
  want_f32(hyper, "hyper");
  c10::cuda::CUDAGuard guard(p.device());
  want_float_kind(g, "g");
  TORCH_CHECK(g.is_contiguous() && g.numel() == p.numel() && hyper.numel() >= 4);
  if (buf.has_value()) want_f32(*buf, "buf");
  check(fb_sgd_step(p.data_ptr<float>(), g.data_ptr(), ptr<float>(buf), ptr<void>(p16), p.numel(), hyper.data_ptr<float>(),
                    ptr<const float>(grad_scale), is_bf16(g), reinterpret_cast<const int*>(skip), stream_of(p)),
        "fb_sgd_step");
}
// returns fp32 [2] = {norm * extra_scale, clip coefficient}
Tensor grad_norm(const Tensor& g, double max_norm, double extra_scale) {
  want_float_kind(g, "g");
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_contiguous());
  auto fopts = torch::dtype(torch::kFloat).device(g.device());
  Tensor partial = torch::empty({fb_grad_norm_parts(g.numel())}, fopts);
  Tensor out = torch::empty({2}, fopts);
  check(fb_grad_norm(g.data_ptr(), g.numel(), partial.data_ptr<float>(), (float)max_norm, (float)extra_scale,
                     out.data_ptr<float>(), is_bf16(g), stream_of(g)),
        "fb_grad_norm");
  return out;
}

// ------------------------------------------------------------------------------------ batch norm
// one zeroed word per device for the channels-last BatchNorm "last block folds" counter
Tensor& bn_counter(int device) {
  static std::vector<Tensor> words(64);
  TORCH_CHECK(device >= 0 && device < 64);
  if (!words[device].defined())
    words[device] = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device];
}
bool is_channels_last_4d(const Tensor& t) {
  return t.dim() == 4 && t.is_contiguous(at::MemoryFormat::ChannelsLast) && !t.is_contiguous();
}

std::vector<Tensor> bn_fwd(const Tensor& x, const OptTensor& residual, const OptTensor& gamma, const OptTensor& beta,
                           Tensor& running_mean, Tensor& running_var, double eps, double momentum, bool relu, bool training,
                           const OptTensor& sums) {
  want_float_kind(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  if (sums.has_value()) {
    // statistics already accumulated by the producer of x (fp32 [2, C]: sum, sum of squares)
    TORCH_CHECK(is_channels_last_4d(x) && training, "precomputed sums need a channels-last input in training mode");
    const int64_t C = x.size(1), P = x.numel() / C;
    TORCH_CHECK(sums->is_cuda() && sums->scalar_type() == at::kFloat && sums->is_contiguous() && sums->numel() == 2 * C, "sums must be fp32 [2, C]");
    want_f32(running_mean, "running_mean");
    want_f32(running_var, "running_var");
    if (residual.has_value())
      TORCH_CHECK(is_channels_last_4d(*residual) && residual->scalar_type() == x.scalar_type() && residual->sizes() == x.sizes(),
                  "residual must be channels-last like x");
    auto fopts = torch::dtype(torch::kFloat).device(x.device());
    Tensor y = torch::empty_like(x);
    Tensor mean = torch::empty({C}, fopts), rstd = torch::empty({C}, fopts);
    check(fb_bn_nhwc_fwd_sums(x.data_ptr(), ptr<const void>(residual), ptr<const float>(gamma), ptr<const float>(beta),
                              running_mean.data_ptr<float>(), running_var.data_ptr<float>(), y.data_ptr(), mean.data_ptr<float>(),
                              rstd.data_ptr<float>(), sums->data_ptr<float>(), (long long)P, (int)C, (float)eps, (float)momentum, relu,
                              is_bf16(x), stream_of(x)),
          "fb_bn_nhwc_fwd_sums");
    return {y, mean, rstd};
  }
  if (is_channels_last_4d(x) && training) {
    const int64_t C = x.size(1), P = x.numel() / C;
    want_f32(running_mean, "running_mean");
    want_f32(running_var, "running_var");
    if (residual.has_value())
      TORCH_CHECK(is_channels_last_4d(*residual) && residual->scalar_type() == x.scalar_type() && residual->sizes() == x.sizes(),
                  "residual must be channels-last like x");
    auto fopts = torch::dtype(torch::kFloat).device(x.device());
    Tensor y = torch::empty_like(x);   // keeps the channels-last strides
    Tensor mean = torch::empty({C}, fopts), rstd = torch::empty({C}, fopts);
    Tensor scratch = torch::empty({fb_bn_nhwc_scratch_floats((int)C)}, fopts);
    check(fb_bn_nhwc_fwd(x.data_ptr(), ptr<const void>(residual), ptr<const float>(gamma), ptr<const float>(beta),
                         running_mean.data_ptr<float>(), running_var.data_ptr<float>(), y.data_ptr(), mean.data_ptr<float>(),
                         rstd.data_ptr<float>(), scratch.data_ptr<float>(),
                         reinterpret_cast<unsigned int*>(bn_counter(x.get_device()).data_ptr<int>()), (long long)P, (int)C, (float)eps,
                         (float)momentum, relu, training, is_bf16(x), stream_of(x)),
          "fb_bn_nhwc_fwd");
    return {y, mean, rstd};
  }
  TORCH_CHECK(x.is_contiguous() && x.dim() >= 2);
  const int64_t N = x.size(0), C = x.size(1), HW = x.numel() / (N * C);
  want_f32(running_mean, "running_mean");
  want_f32(running_var, "running_var");
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == x.scalar_type() && residual->numel() == x.numel());
  auto fopts = torch::dtype(torch::kFloat).device(x.device());
  Tensor y = torch::empty_like(x), mean = torch::empty({C}, fopts), rstd = torch::empty({C}, fopts);
  Tensor scratch = torch::empty({fb_bn_scratch_floats((int)C)}, fopts);
  check(fb_bn_fwd(x.data_ptr(), ptr<const void>(residual), ptr<const float>(gamma), ptr<const float>(beta), running_mean.data_ptr<float>(),
                  running_var.data_ptr<float>(), y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), scratch.data_ptr<float>(),
                  (int)N, (int)C, (int)HW, (float)eps, (float)momentum, relu, training, is_bf16(x), stream_of(x)),
        "fb_bn_fwd");
  return {y, mean, rstd};
}
std::vector<Tensor> bn_bwd(const Tensor& dy, const Tensor& x, const Tensor& y, const OptTensor& gamma, const Tensor& mean,
                           const Tensor& rstd, bool relu, bool want_dres, const OptTensor& dgamma_acc, const OptTensor& dbeta_acc) {
  want_float_kind(dy, "dy");
  c10::cuda::CUDAGuard guard(dy.device());
  if (is_channels_last_4d(x)) {
    TORCH_CHECK(is_channels_last_4d(dy) && is_channels_last_4d(y), "channels-last BatchNorm backward needs channels-last dy and y");
    const int64_t C = x.size(1), P = x.numel() / C;
    auto fopts = torch::dtype(torch::kFloat).device(x.device());
    Tensor dx = torch::empty_like(x);
    Tensor dres = want_dres ? torch::empty_like(x) : Tensor();
    Tensor dg, db;
    bool acc = false;
    if (dgamma_acc.has_value()) { dg = *dgamma_acc; db = *dbeta_acc; acc = true; }
    else { dg = torch::empty({C}, fopts); db = torch::empty({C}, fopts); }
    Tensor scratch = torch::empty({fb_bn_nhwc_scratch_floats((int)C)}, fopts);
    check(fb_bn_nhwc_bwd(dy.data_ptr(), x.data_ptr(), y.data_ptr(), ptr<const float>(gamma), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                         dx.data_ptr(), want_dres ? dres.data_ptr() : nullptr, dg.data_ptr<float>(), db.data_ptr<float>(), acc,
                         scratch.data_ptr<float>(), reinterpret_cast<unsigned int*>(bn_counter(x.get_device()).data_ptr<int>()), (long long)P,
                         (int)C, relu, is_bf16(dy), stream_of(dy)),
          "fb_bn_nhwc_bwd");
    return {dx, dres, dg, db};
  }
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && y.is_contiguous());
  const int64_t N = x.size(0), C = x.size(1), HW = x.numel() / (N * C);
  auto fopts = torch::dtype(torch::kFloat).device(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor dres = want_dres ? torch::empty_like(x) : Tensor();
  Tensor dg, db;
  bool acc = false;
  if (dgamma_acc.has_value()) {
    dg = *dgamma_acc;
    db = *dbeta_acc;
    acc = true;
  } else {
    dg = torch::empty({C}, fopts);
    db = torch::empty({C}, fopts);
  }
  Tensor scratch = torch::empty({fb_bn_scratch_floats((int)C)}, fopts);
  check(fb_bn_bwd(dy.data_ptr(), x.data_ptr(), y.data_ptr(), ptr<const float>(gamma), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                  dx.data_ptr(), want_dres ? dres.data_ptr() : nullptr, dg.data_ptr<float>(), db.data_ptr<float>(), acc,
                  scratch.data_ptr<float>(), (int)N, (int)C, (int)HW, relu, is_bf16(dy), stream_of(dy)),
        "fb_bn_bwd");
  return {dx, dres, dg, db};
}

// ------------------------------------------------------------------------------- convolution
bool conv_wgrad_supported(int64_t N, int64_t H, int64_t W, int64_t Ci, int64_t Co, int64_t k, int64_t stride, int64_t pad) {
  return fb_conv_wgrad_supported((int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)k, (int)stride, (int)pad) != 0;
}
// x, dy: channels-last bf16 4-D tensors; dw: fp32 tensor of logical shape [Co,Ci,k,k] whose memory is
// K-R-S-C (channels-last strides), e.g. a flat-buffer gradient slot. The gradient is added to dw.
void conv_wgrad(const Tensor& x, const Tensor& dy, Tensor& dw, int64_t stride, int64_t pad) {
  want_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(is_bf16(x) && is_bf16(dy) && x.dim() == 4 && dy.dim() == 4, "conv_wgrad takes bf16 4-D tensors");
  TORCH_CHECK(x.is_contiguous(at::MemoryFormat::ChannelsLast) && dy.is_contiguous(at::MemoryFormat::ChannelsLast),
              "conv_wgrad needs channels-last x and dy");
  TORCH_CHECK(dw.scalar_type() == at::kFloat && dw.dim() == 4 && dw.is_contiguous(at::MemoryFormat::ChannelsLast),
              "dw must be fp32 with channels-last (K-R-S-C) memory");
  const int64_t N = x.size(0), Ci = x.size(1), H = x.size(2), W = x.size(3), Co = dy.size(1), k = dw.size(2);
  TORCH_CHECK(dw.size(0) == Co && dw.size(1) == Ci && dw.size(3) == k, "dw shape mismatch");
  Tensor& st = status_word(x.get_device());
  check(fb_conv_wgrad(x.data_ptr(), dy.data_ptr(), dw.data_ptr<float>(), (int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)k, (int)stride,
                      (int)pad, st.data_ptr<int>(), stream_of(x)),
        "fb_conv_wgrad");
}

bool conv_fprop_supported(int64_t N, int64_t H, int64_t W, int64_t Ci, int64_t Co, int64_t k, int64_t stride, int64_t pad) {
  return fb_conv_fprop_supported((int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)stride, (int)pad) != 0;
}
bool conv_dgrad_supported(int64_t N, int64_t H, int64_t W, int64_t Ci, int64_t Co, int64_t k, int64_t stride, int64_t pad) {
  return fb_conv_dgrad_supported((int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)stride, (int)pad) != 0;
}
void check_filter(const Tensor& w) {
  TORCH_CHECK(w.is_cuda() && is_bf16(w) && w.dim() == 4 && w.is_contiguous(at::MemoryFormat::ChannelsLast) && w.size(2) == w.size(3),
              "filter must be a square bf16 [Co,Ci,k,k] tensor with channels-last (K-R-S-C) memory");
}
// y = conv2d(x, w) for channels-last bf16 x; `stats` (fp32 [2, Co], zeroed) optionally receives sum / sum of squares of y.
Tensor conv_fprop(const Tensor& x, const Tensor& w, int64_t stride, int64_t pad, const OptTensor& stats, const OptTensor& ts) {
  want_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(is_bf16(x) && x.dim() == 4 && x.is_contiguous(at::MemoryFormat::ChannelsLast), "conv_fprop needs a channels-last bf16 input");
  check_filter(w);
  const int64_t N = x.size(0), Ci = x.size(1), H = x.size(2), W = x.size(3), Co = w.size(0), k = w.size(2);
  TORCH_CHECK(w.size(1) == Ci, "filter/input channel mismatch");
  const int64_t Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  if (stats.has_value()) TORCH_CHECK(stats->is_cuda() && stats->scalar_type() == at::kFloat && stats->is_contiguous() && stats->numel() == 2 * Co, "stats must be fp32 [2, Co]");
  Tensor y = torch::empty({N, Co, Ho, Wo}, x.options().memory_format(at::MemoryFormat::ChannelsLast));
  Tensor& st = status_word(x.get_device());
  if (ts.has_value()) {
    TORCH_CHECK(ts->is_cuda() && ts->scalar_type() == at::kLong && ts->is_contiguous() && ts->numel() >= 64, "ts must be an int64 CUDA tensor of 64 slots");
    check(fb_conv_fprop_ts(x.data_ptr(), w.data_ptr(), y.data_ptr(), ptr<float>(stats), (int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)stride,
                           (int)pad, st.data_ptr<int>(), reinterpret_cast<long long*>(ts->data_ptr<int64_t>()), stream_of(x)),
          "fb_conv_fprop_ts");
    return y;
  }
  check(fb_conv_fprop(x.data_ptr(), w.data_ptr(), y.data_ptr(), ptr<float>(stats), (int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)stride, (int)pad,
                      st.data_ptr<int>(), stream_of(x)),
        "fb_conv_fprop");
  return y;
}
// dx for a stride-1 "same" convolution.
Tensor conv_dgrad(const Tensor& dy, const Tensor& w, int64_t stride, int64_t pad) {
  want_cuda(dy, "dy");
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(is_bf16(dy) && dy.dim() == 4 && dy.is_contiguous(at::MemoryFormat::ChannelsLast), "conv_dgrad needs a channels-last bf16 gradient");
  check_filter(w);
  const int64_t N = dy.size(0), Co = dy.size(1), H = dy.size(2), W = dy.size(3), Ci = w.size(1), k = w.size(2);
  TORCH_CHECK(w.size(0) == Co, "filter/gradient channel mismatch");
  Tensor dx = torch::empty({N, Ci, H, W}, dy.options().memory_format(at::MemoryFormat::ChannelsLast));
  Tensor& st = status_word(dy.get_device());
  check(fb_conv_dgrad(dy.data_ptr(), w.data_ptr(), dx.data_ptr(), (int)N, (int)H, (int)W, (int)Ci, (int)Co, (int)k, (int)stride, (int)pad,
                      st.data_ptr<int>(), stream_of(dy)),
        "fb_conv_dgrad");
  return dx;
}

// ------------------------------------------------------------------------------------ attention
// q, k, v: bf16 views [B, S, H, 64] sharing one stride set (e.g. slices of a fused QKV buffer).
void check_bshd(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && is_bf16(t) && t.dim() == 4 && t.size(3) == 64 && t.stride(3) == 1, name,
              " must be bf16 [B, S, H, 64] with a unit inner stride");
}
std::array<long long, 3> bsh_strides(const Tensor& t) { return {t.stride(0), t.stride(1), t.stride(2)}; }

std::vector<Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const OptTensor& mask, double scale,
                             bool causal, double p_drop, uint64_t seed, const OptTensor& seed_dev) {
  check_bshd(q, "q");
  check_bshd(k, "k");
  check_bshd(v, "v");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(k.strides() == q.strides() && v.strides() == q.strides() && k.sizes() == q.sizes() && v.sizes() == q.sizes(),
              "q, k, v must share shape and strides");
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2);
  if (mask.has_value()) TORCH_CHECK(mask->is_cuda() && mask->scalar_type() == at::kFloat && mask->is_contiguous() && mask->numel() == B * S, "mask must be fp32 [B, S]");
  Tensor o = torch::empty({B, S, H, 64}, q.options());
  Tensor lse = torch::empty({B, H, S}, q.options().dtype(torch::kFloat));
  auto qs = bsh_strides(q), os = bsh_strides(o);
  Tensor& st = status_word(q.get_device());
  check(fb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), ptr<const float>(mask), (int)B,
                    (int)H, (int)S, qs.data(), os.data(), (float)scale, causal, (float)p_drop, seed, seed_ptr(seed_dev),
                    st.data_ptr<int>(), stream_of(q)),
        "fb_attn_fwd");
  return {o, lse};
}

// Returns one fused gradient buffer [B, S, 3, H, 64] (dq, dk, dv are its slices along dim 2).
Tensor attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o, const Tensor& lse,
                const OptTensor& mask, double scale, bool causal, double p_drop, uint64_t seed, const OptTensor& seed_dev) {
  check_bshd(q, "q");
  check_bshd(o, "o");
  check_bshd(d_o, "d_o");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(d_o.strides() == o.strides(), "dO must share o's strides");
  const int64_t B = q.size(0), S = q.size(1), H = q.size(2);
  Tensor dqkv = torch::empty({B, S, 3, H, 64}, q.options());
  Tensor dq = dqkv.select(2, 0), dk = dqkv.select(2, 1), dv = dqkv.select(2, 2);
  Tensor acc;
  if (S > 128) acc = torch::empty({B, H, S, 64}, q.options().dtype(torch::kFloat));
  auto qs = bsh_strides(q), os = bsh_strides(o), gs = bsh_strides(dq);
  Tensor& st = status_word(q.get_device());
  check(fb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                    ptr<const float>(mask), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), acc.defined() ? acc.data_ptr<float>() : nullptr,
                    (int)B, (int)H, (int)S, qs.data(), os.data(), gs.data(), (float)scale, causal, (float)p_drop, seed,
                    seed_ptr(seed_dev), st.data_ptr<int>(), stream_of(q)),
        "fb_attn_bwd");
  return dqkv;
}

}  // namespace

void bind_comm(py::module_& m);     // comm.cpp
void bind_runtime(py::module_& m);  // runtime.cpp
void bind_graph_exec(py::module_& m);  // graph_exec.cpp
void bind_cpu_avg(py::module_& m);     // cpu_avg.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "flodl_b200 native kernels (sm_100a) and runtime";
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("bias") = py::none(), py::arg("epi") = 0, py::arg("aux") = py::none(), py::arg("alpha") = py::none(),
        py::arg("accumulate") = false, py::arg("split_k") = 1, py::arg("config") = -1, py::arg("ts") = py::none(),
        py::arg("m_dyn") = py::none(), py::arg("k_dyn") = py::none());
  m.def("gemm_pick_config", &gemm_pick_config);
  m.def("read_status", &read_status);
  m.def("bounds_check_build", &bounds_check_build);
  m.def("bounds_report", &bounds_report, py::arg("clear") = true);
  m.def("clear_status", &clear_status);
  m.def("layernorm_fwd", &layernorm_fwd, py::arg("x"), py::arg("residual"), py::arg("gamma"), py::arg("beta"), py::arg("eps"),
        py::arg("p_drop"), py::arg("seed"), py::arg("want_pre"), py::arg("seed_dev") = py::none());
  m.def("layernorm_bwd", &layernorm_bwd, py::arg("dy"), py::arg("pre"), py::arg("mean"), py::arg("rstd"), py::arg("gamma"),
        py::arg("p_drop"), py::arg("seed"), py::arg("want_dx_drop"), py::arg("want_param_grads"), py::arg("dgamma_acc"),
        py::arg("dbeta_acc"), py::arg("seed_dev") = py::none());
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("dropout", &dropout, py::arg("x"), py::arg("p"), py::arg("seed"), py::arg("seed_dev") = py::none());
  m.def("colsum", &colsum, py::arg("x"), py::arg("out"), py::arg("rows_dyn") = py::none());
  m.def("compact_targets", &compact_targets);
  m.def("gather_rows", &gather_rows);
  m.def("scatter_rows", &scatter_rows);
  m.def("cast_into", &cast_into);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("softmax_ce", &softmax_ce, py::arg("logits"), py::arg("targets"), py::arg("ignore_index"), py::arg("want_grad"), py::arg("inplace"),
        py::arg("counts") = py::none());
  m.def("scale_rows", &scale_rows);
  m.def("adam_step", &adam_step, py::arg("p"), py::arg("g"), py::arg("m"), py::arg("v"), py::arg("p16"), py::arg("hyper"),
        py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("grad_scale") = py::none(), py::arg("skip") = 0);
  m.def("adam_step_multi", &adam_step_multi, py::arg("ps"), py::arg("gs"), py::arg("ms"), py::arg("vs"), py::arg("p16s"), py::arg("hyper"),
        py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("grad_scale") = py::none(), py::arg("skip") = 0);
  m.def("sgd_step", &sgd_step, py::arg("p"), py::arg("g"), py::arg("buf"), py::arg("p16"), py::arg("hyper"),
        py::arg("grad_scale") = py::none(), py::arg("skip") = 0);
  m.def("grad_norm", &grad_norm);
  m.def("bn_fwd", &bn_fwd, py::arg("x"), py::arg("residual"), py::arg("gamma"), py::arg("beta"), py::arg("running_mean"), py::arg("running_var"),
        py::arg("eps"), py::arg("momentum"), py::arg("relu"), py::arg("training"), py::arg("sums") = py::none());
  m.def("bn_bwd", &bn_bwd);
  m.def("conv_wgrad_supported", &conv_wgrad_supported);
  m.def("conv_fprop_supported", &conv_fprop_supported);
  m.def("conv_dgrad_supported", &conv_dgrad_supported);
  m.def("conv_fprop", &conv_fprop, py::arg("x"), py::arg("w"), py::arg("stride"), py::arg("pad"), py::arg("stats") = py::none(), py::arg("ts") = py::none());
  m.def("conv_dgrad", &conv_dgrad, py::arg("dy"), py::arg("w"), py::arg("stride"), py::arg("pad"));
  m.def("conv_wgrad", &conv_wgrad, py::arg("x"), py::arg("dy"), py::arg("dw"), py::arg("stride"), py::arg("pad"));
  m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("mask"), py::arg("scale"), py::arg("causal"),
        py::arg("p_drop") = 0.0, py::arg("seed") = 0, py::arg("seed_dev") = py::none());
  m.def("attn_bwd", &attn_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("d_o"), py::arg("lse"), py::arg("mask"),
        py::arg("scale"), py::arg("causal"), py::arg("p_drop") = 0.0, py::arg("seed") = 0, py::arg("seed_dev") = py::none());
  bind_comm(m);
  bind_runtime(m);
  bind_graph_exec(m);
  bind_cpu_avg(m);
}
