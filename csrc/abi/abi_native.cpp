// Drop-in C ABI, part 5: the hot ops of a transformer training step on this library's sm_100a kernels,
// as C++ autograd functions. A host that builds its model out of `flodl_linear`, `flodl_native_layer_norm`,
// `flodl_gelu`, `flodl_scaled_dot_product_attention`, `flodl_cross_entropy_loss` and `flodl_dropout`
// and calls `flodl_backward` gets the tcgen05 GEMM, the fused attention and the fused softmax-cross-entropy
// in both directions without knowing about them.
//
// A call takes the native path when its input is on a CUDA device and bf16 is the compute type: the input
// is bf16 already, or autocast is on for CUDA with bf16 (`flodl_autocast_*`). Everything else, and every
// shape the kernels do not cover, returns false and the caller forwards to ATen. FLODL_B200_NATIVE=0
// turns the native paths off (for A/B timing).
#include "abi_common.hpp"

#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/autograd/custom_function.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "flodl_b200.h"

namespace fbabi {
namespace {

using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

std::atomic<long long> g_native_calls{0};
std::atomic<unsigned long long> g_seed_counter{0};

bool natives_on() {
  static const bool on = [] {
    const char* e = std::getenv("FLODL_B200_NATIVE");
    return !(e && (e[0] == '0' || e[0] == 'n' || e[0] == 'f'));
  }();
  return on;
}
// FLODL_B200_NATIVE_OPS=linear,layer_norm,gelu,sdpa,cross_entropy,dropout restricts the native paths to the listed ops
// (for bisecting a numerical difference); unset = all.
bool op_on(const char* name) {
  static const std::string list = [] {
    const char* e = std::getenv("FLODL_B200_NATIVE_OPS");
    return e ? "," + std::string(e) + "," : std::string();
  }();
  return list.empty() || list.find("," + std::string(name) + ",") != std::string::npos;
}
bool autocast_bf16() { return at::autocast::is_autocast_enabled(at::kCUDA) && at::autocast::get_autocast_dtype(at::kCUDA) == at::kBFloat16; }
bool is_bf16(const Tensor& t) { return t.scalar_type() == at::kBFloat16; }
// bf16 is the compute type of an op on `x`
bool bf16_compute(const Tensor& x) {
  if (!natives_on() || !x.defined() || !x.is_cuda() || x.numel() == 0) return false;
  if (is_bf16(x)) return true;
  return x.scalar_type() == at::kFloat && autocast_bf16();
}
void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }
void check(int rc, const char* what) {
  if (rc == 0) return;
  if (rc > 0) TORCH_CHECK(false, what, ": CUDA error ", rc, " (", cudaGetErrorString(static_cast<cudaError_t>(rc)), ")");
  TORCH_CHECK(false, what, ": rejected arguments (code ", rc, ")");
}
// One status word per device for the kernels with bounded waits (GEMM, attention).
int* status_word(int device) {
  static std::mutex mu;
  static std::vector<Tensor> words(64);
  std::lock_guard<std::mutex> lock(mu);
  TORCH_CHECK(device >= 0 && device < 64);
  if (!words[device].defined()) words[device] = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device].data_ptr<int>();
}
int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
// [rows, cols] tensor whose row stride is a multiple of 8 elements (what a TMA descriptor can address)
Tensor new_rows(int64_t rows, int64_t cols, at::ScalarType dt, const at::Device& dev) {
  const int64_t ld = round_up(cols, 8);
  Tensor buf = torch::empty({rows, ld}, torch::dtype(dt).device(dev));
  return ld == cols ? buf : buf.narrow(1, 0, cols);
}
// 2-D bf16 view or copy a TMA descriptor can address: unit inner stride, row stride % 8 == 0, 16-byte base
Tensor operand(const Tensor& t) {
  Tensor x = is_bf16(t) ? t : t.to(at::kBFloat16);
  if (x.stride(1) == 1 && x.stride(0) % 8 == 0 && x.stride(0) >= x.size(1) && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0) return x;
  Tensor out = new_rows(x.size(0), x.size(1), at::kBFloat16, x.device());
  out.copy_(x);
  return out;
}

// ---- bf16 copies of fp32 weights ------------------------------------------------------------------
// A weight is cast once per value: the copy is keyed by the weight's storage and reused while its
// version counter and the library-wide mutation epoch stand still. In-place updates through ATen
// bump the version; the ABI's own raw-pointer optimizer steps call `note_mutation()`.
std::atomic<unsigned long long> g_epoch{1};
struct Shadow {
  c10::weak_intrusive_ptr<c10::TensorImpl> owner;
  uint32_t version;
  unsigned long long epoch;
  Tensor bf16;
};
std::mutex g_shadow_mu;
std::unordered_map<const void*, Shadow> g_shadows;

Tensor shadow_of(const Tensor& w) {
  if (is_bf16(w)) return operand(w);
  const void* key = w.unsafeGetTensorImpl();
  const uint32_t ver = w._version();
  const unsigned long long ep = g_epoch.load(std::memory_order_relaxed);
  std::lock_guard<std::mutex> lock(g_shadow_mu);
  auto it = g_shadows.find(key);
  if (it != g_shadows.end() && !it->second.owner.expired() && it->second.version == ver && it->second.epoch == ep &&
      it->second.bf16.size(0) == w.size(0) && it->second.bf16.size(1) == w.size(1))
    return it->second.bf16;
  Tensor s;
  if (it != g_shadows.end() && !it->second.owner.expired() && it->second.bf16.sizes() == w.sizes()) {
    s = it->second.bf16;  // same weight, new value: refresh in place (no allocation in steady state)
    check(fb_cast(w.contiguous().data_ptr(), s.data_ptr(), w.numel(), 1.0f, 0, 1, stream_of(w)), "fb_cast");
  } else {
    if (g_shadows.size() > 4096) {
      for (auto e = g_shadows.begin(); e != g_shadows.end();) e = e->second.owner.expired() ? g_shadows.erase(e) : std::next(e);
    }
    s = (w.size(1) % 8 == 0) ? torch::empty_like(w, w.options().dtype(at::kBFloat16), at::MemoryFormat::Contiguous) : Tensor();
    if (s.defined() && w.scalar_type() == at::kFloat && w.is_contiguous())
      check(fb_cast(w.data_ptr(), s.data_ptr(), w.numel(), 1.0f, 0, 1, stream_of(w)), "fb_cast");
    else
      s = operand(w.detach());
  }
  g_shadows.insert_or_assign(key, Shadow{c10::weak_intrusive_ptr<c10::TensorImpl>(w.getIntrusivePtr()), ver, ep, s});
  return s;
}

// D = A B^T style product on the tensor cores; see fb_gemm_bf16 for the operand conventions.
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, const Tensor& bias, int epi, const float* alpha, bool accumulate,
          int split_k, int config) {
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb && out.size(0) == M && out.size(1) == N, "gemm: shape mismatch");
  check(fb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), a.stride(0), b.stride(0),
                     out.stride(0), a_mn, b_mn, out.scalar_type() == at::kFloat, bias.defined() ? bias.data_ptr() : nullptr,
                     bias.defined() && bias.scalar_type() == at::kFloat, epi, nullptr, 0, alpha, accumulate, split_k, config,
                     status_word(a.get_device()), stream_of(a)),
        "fb_gemm_bf16");
}
// (config, split_k) of a weight-gradient product: few output tiles and a long reduction (measured on B200)
std::pair<int, int> dw_plan(int64_t m_out, int64_t n_out, int64_t k_red) {
  const int64_t pair_tiles = ((m_out + 255) / 256) * ((n_out + 255) / 256);
  if (pair_tiles >= 148 || k_red < 1024) return {-1, 1};
  if (pair_tiles >= 24) return {0, k_red >= 2048 ? 2 : 1};
  return {2, static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(4, k_red / 512)))};
}
Tensor weight_grad(const Tensor& dy2, const Tensor& x2, at::ScalarType want, const float* alpha = nullptr) {
  const int64_t N = dy2.size(1), K = x2.size(1);
  auto plan = dw_plan(N, K, dy2.size(0));
  auto opts = torch::dtype(torch::kFloat).device(dy2.device());
  Tensor out = plan.second > 1 ? torch::zeros({N, K}, opts) : torch::empty({N, K}, opts);
  gemm(dy2, x2, out, true, true, Tensor(), 0, alpha, plan.second > 1, plan.second, plan.first);
  return want == at::kFloat ? out : out.to(want);
}
Tensor bias_grad(const Tensor& dy2, at::ScalarType want) {
  Tensor out = torch::zeros({dy2.size(1)}, torch::dtype(torch::kFloat).device(dy2.device()));   // the kernel adds into it
  check(fb_colsum(dy2.data_ptr(), out.data_ptr<float>(), static_cast<int>(dy2.size(0)), static_cast<int>(dy2.size(1)), dy2.stride(0), is_bf16(dy2),
                  stream_of(dy2)),
        "fb_colsum");
  return want == at::kFloat ? out : out.to(want);
}
unsigned long long next_seed() {
  // a fresh stream position per call, tied to the default CUDA generator's seed so `flodl_manual_seed` reproduces runs
  const auto& gen = at::cuda::detail::getDefaultCUDAGenerator();
  return gen.current_seed() * 0x9E3779B97F4A7C15ull + g_seed_counter.fetch_add(1, std::memory_order_relaxed) + 1;
}

// ---- linear ----------------------------------------------------------------------------------------
struct LinearFn : public torch::autograd::Function<LinearFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x, const Tensor& w, const Tensor& b) {
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t K = x.size(-1), N = w.size(0);
    Tensor x2 = operand(x.reshape({-1, K}));
    Tensor w16 = shadow_of(w);
    Tensor out = new_rows(x2.size(0), N, at::kBFloat16, x.device());
    Tensor bias = b.defined() ? b.contiguous() : Tensor();
    gemm(x2, w16, out, false, false, bias, 0, nullptr, false, 1, -1);
    ctx->save_for_backward({x2, w16});
    ctx->saved_data["xshape"] = x.sizes().vec();
    ctx->saved_data["xdtype"] = static_cast<int64_t>(x.scalar_type());
    ctx->saved_data["wdtype"] = static_cast<int64_t>(w.scalar_type());
    ctx->saved_data["bdtype"] = static_cast<int64_t>(b.defined() ? b.scalar_type() : at::kFloat);
    ctx->saved_data["has_bias"] = b.defined();
    std::vector<int64_t> oshape = x.sizes().vec();
    oshape.back() = N;
    return out.is_contiguous() ? out.view(oshape) : out.reshape(oshape);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    auto saved = ctx->get_saved_variables();
    const Tensor &x2 = saved[0], &w16 = saved[1];
    c10::cuda::CUDAGuard guard(x2.device());
    const int64_t N = w16.size(0), K = w16.size(1);
    Tensor dy2 = operand(grads[0].reshape({-1, N}));
    Tensor dx, dw, db;
    if (ctx->needs_input_grad(1)) dw = weight_grad(dy2, x2, static_cast<at::ScalarType>(ctx->saved_data["wdtype"].toInt()));
    if (ctx->saved_data["has_bias"].toBool() && ctx->needs_input_grad(2)) db = bias_grad(dy2, static_cast<at::ScalarType>(ctx->saved_data["bdtype"].toInt()));
    if (ctx->needs_input_grad(0)) {
      Tensor dx2 = new_rows(x2.size(0), K, at::kBFloat16, x2.device());
      gemm(dy2, w16, dx2, false, true, Tensor(), 0, nullptr, false, 1, -1);
      dx = dx2.reshape(ctx->saved_data["xshape"].toIntVector());
      const auto xd = static_cast<at::ScalarType>(ctx->saved_data["xdtype"].toInt());
      if (xd != at::kBFloat16) dx = dx.to(xd);
    }
    return {dx, dw, db};
  }
};

// ---- layer norm ------------------------------------------------------------------------------------
struct LayerNormFn : public torch::autograd::Function<LayerNormFn> {
  static variable_list forward(AutogradContext* ctx, const Tensor& x_in, const Tensor& gamma, const Tensor& beta, double eps) {
    c10::cuda::CUDAGuard guard(x_in.device());
    Tensor x = x_in.contiguous();
    const int64_t cols = x.size(-1), rows = x.numel() / cols;
    auto fopts = torch::dtype(torch::kFloat).device(x.device());
    Tensor y = torch::empty_like(x), mean = torch::empty({rows}, fopts), rstd = torch::empty({rows}, fopts);
    check(fb_layernorm_fwd(x.data_ptr(), nullptr, gamma.defined() ? gamma.data_ptr<float>() : nullptr, beta.defined() ? beta.data_ptr<float>() : nullptr,
                           y.data_ptr(), nullptr, mean.data_ptr<float>(), rstd.data_ptr<float>(), static_cast<int>(rows), static_cast<int>(cols),
                           static_cast<float>(eps), 0.0f, 0, nullptr, is_bf16(x), stream_of(x)),
          "fb_layernorm_fwd");
    ctx->save_for_backward({x, mean, rstd, gamma});
    ctx->saved_data["has_beta"] = beta.defined();
    std::vector<int64_t> stat_shape = x.sizes().vec();
    stat_shape.back() = 1;
    Tensor mean_out = mean.view(stat_shape), rstd_out = rstd.view(stat_shape);
    ctx->mark_non_differentiable({mean_out, rstd_out});
    return {y, mean_out, rstd_out};
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    auto saved = ctx->get_saved_variables();
    const Tensor &x = saved[0], &mean = saved[1], &rstd = saved[2], &gamma = saved[3];
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t cols = x.size(-1), rows = x.numel() / cols;
    Tensor dy = grads[0].contiguous();
    if (dy.scalar_type() != x.scalar_type()) dy = dy.to(x.scalar_type());
    auto fopts = torch::dtype(torch::kFloat).device(x.device());
    const bool want_params = (gamma.defined() && ctx->needs_input_grad(1)) || (ctx->saved_data["has_beta"].toBool() && ctx->needs_input_grad(2));
    Tensor dx = torch::empty_like(x), partial, dgamma, dbeta;
    if (want_params) {
      partial = torch::empty({fb_layernorm_bwd_grid(static_cast<int>(rows)), 2, cols}, fopts);
      dgamma = torch::empty({cols}, fopts);
      dbeta = torch::empty({cols}, fopts);
    }
    check(fb_layernorm_bwd(dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), gamma.defined() ? gamma.data_ptr<float>() : nullptr,
                           dx.data_ptr(), nullptr, want_params ? partial.data_ptr<float>() : nullptr, want_params ? dgamma.data_ptr<float>() : nullptr,
                           want_params ? dbeta.data_ptr<float>() : nullptr, 0, static_cast<int>(rows), static_cast<int>(cols), 0.0f, 0, nullptr, is_bf16(x),
                           stream_of(x)),
          "fb_layernorm_bwd");
    return {dx, gamma.defined() ? dgamma : Tensor(), ctx->saved_data["has_beta"].toBool() ? dbeta : Tensor(), Tensor()};
  }
};

// ---- GELU ------------------------------------------------------------------------------------------
struct GeluFn : public torch::autograd::Function<GeluFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x_in, bool tanh_approx) {
    c10::cuda::CUDAGuard guard(x_in.device());
    Tensor x = x_in.contiguous();
    Tensor y = torch::empty_like(x);
    check(fb_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), tanh_approx, is_bf16(x), stream_of(x)), "fb_gelu_fwd");
    ctx->save_for_backward({x});
    ctx->saved_data["tanh"] = tanh_approx;
    return y;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    const Tensor x = ctx->get_saved_variables()[0];
    c10::cuda::CUDAGuard guard(x.device());
    Tensor dy = grads[0].contiguous();
    if (dy.scalar_type() != x.scalar_type()) dy = dy.to(x.scalar_type());
    Tensor dx = torch::empty_like(x);
    check(fb_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), ctx->saved_data["tanh"].toBool(), is_bf16(x), stream_of(x)), "fb_gelu_bwd");
    return {dx, Tensor()};
  }
};

// ---- dropout ---------------------------------------------------------------------------------------
// The mask is a function of (seed, element index): the backward pass re-applies the kernel to dy with the seed of
// the forward pass instead of storing a mask.
struct DropoutFn : public torch::autograd::Function<DropoutFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& x_in, double p) {
    c10::cuda::CUDAGuard guard(x_in.device());
    Tensor x = x_in.contiguous();
    Tensor y = torch::empty_like(x);
    const unsigned long long seed = next_seed();
    check(fb_dropout(x.data_ptr(), y.data_ptr(), x.numel(), static_cast<float>(p), seed, nullptr, is_bf16(x), stream_of(x)), "fb_dropout");
    ctx->saved_data["seed"] = static_cast<int64_t>(seed);
    ctx->saved_data["p"] = p;
    return y;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    Tensor dy = grads[0].contiguous();
    c10::cuda::CUDAGuard guard(dy.device());
    Tensor dx = torch::empty_like(dy);
    check(fb_dropout(dy.data_ptr(), dx.data_ptr(), dy.numel(), static_cast<float>(ctx->saved_data["p"].toDouble()),
                     static_cast<unsigned long long>(ctx->saved_data["seed"].toInt()), nullptr, is_bf16(dy), stream_of(dy)),
          "fb_dropout");
    return {dx, Tensor()};
  }
};

// ---- attention -------------------------------------------------------------------------------------
// Inputs arrive as [B, H, S, 64] (any strides); the kernels address [B, S, H, 64] through (batch, seq, head)
// strides, which a permuted view provides without a copy.
std::array<long long, 3> bsh(const Tensor& t) { return {t.stride(0), t.stride(1), t.stride(2)}; }
bool attn_view_ok(const Tensor& t) {
  return is_bf16(t) && t.stride(3) == 1 && t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0 &&
         reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
}
struct AttnFn : public torch::autograd::Function<AttnFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, const Tensor& mask, double p, bool causal,
                        double scale) {
    c10::cuda::CUDAGuard guard(q_in.device());
    Tensor q = q_in.permute({0, 2, 1, 3}), k = k_in.permute({0, 2, 1, 3}), v = v_in.permute({0, 2, 1, 3});  // [B, S, H, 64] views
    const int64_t B = q.size(0), S = q.size(1), H = q.size(2);
    if (!(attn_view_ok(q) && attn_view_ok(k) && attn_view_ok(v) && k.strides() == q.strides() && v.strides() == q.strides())) {
      Tensor packed = torch::empty({3, B, S, H, 64}, q.options().dtype(at::kBFloat16));
      packed.select(0, 0).copy_(q);
      packed.select(0, 1).copy_(k);
      packed.select(0, 2).copy_(v);
      q = packed.select(0, 0);
      k = packed.select(0, 1);
      v = packed.select(0, 2);
    }
    Tensor o = torch::empty({B, S, H, 64}, q.options());
    Tensor lse = torch::empty({B, H, S}, q.options().dtype(torch::kFloat));
    const unsigned long long seed = p > 0.0 ? next_seed() : 0ull;
    auto qs = bsh(q), os = bsh(o);
    check(fb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), mask.defined() ? mask.data_ptr<float>() : nullptr,
                      static_cast<int>(B), static_cast<int>(H), static_cast<int>(S), qs.data(), os.data(), static_cast<float>(scale), causal,
                      static_cast<float>(p), seed, nullptr, status_word(q.get_device()), stream_of(q)),
          "fb_attn_fwd");
    ctx->save_for_backward({q, k, v, o, lse, mask});
    ctx->saved_data["p"] = p;
    ctx->saved_data["causal"] = causal;
    ctx->saved_data["scale"] = scale;
    ctx->saved_data["seed"] = static_cast<int64_t>(seed);
    ctx->saved_data["qd"] = static_cast<int64_t>(q_in.scalar_type());
    ctx->saved_data["kd"] = static_cast<int64_t>(k_in.scalar_type());
    ctx->saved_data["vd"] = static_cast<int64_t>(v_in.scalar_type());
    return o.permute({0, 2, 1, 3});  // [B, H, S, 64] view, so the host's transpose(1, 2) + reshape is free
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    auto saved = ctx->get_saved_variables();
    const Tensor &q = saved[0], &k = saved[1], &v = saved[2], &o = saved[3], &lse = saved[4], &mask = saved[5];
    c10::cuda::CUDAGuard guard(q.device());
    const int64_t B = q.size(0), S = q.size(1), H = q.size(2);
    Tensor d_o = grads[0].permute({0, 2, 1, 3});
    if (!is_bf16(d_o)) d_o = d_o.to(at::kBFloat16);
    if (d_o.strides() != o.strides()) d_o = d_o.contiguous();
    Tensor dqkv = torch::empty({B, S, 3, H, 64}, q.options());
    Tensor dq = dqkv.select(2, 0), dk = dqkv.select(2, 1), dv = dqkv.select(2, 2);
    Tensor acc;
    if (S > 128) acc = torch::empty({B, H, S, 64}, q.options().dtype(torch::kFloat));
    auto qs = bsh(q), os = bsh(o), gs = bsh(dq);
    check(fb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                      mask.defined() ? mask.data_ptr<float>() : nullptr, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                      acc.defined() ? acc.data_ptr<float>() : nullptr, static_cast<int>(B), static_cast<int>(H), static_cast<int>(S), qs.data(), os.data(),
                      gs.data(), static_cast<float>(ctx->saved_data["scale"].toDouble()), ctx->saved_data["causal"].toBool(),
                      static_cast<float>(ctx->saved_data["p"].toDouble()), static_cast<unsigned long long>(ctx->saved_data["seed"].toInt()), nullptr,
                      status_word(q.get_device()), stream_of(q)),
          "fb_attn_bwd");
    auto back = [&](const Tensor& g, const char* key) {
      Tensor r = g.permute({0, 2, 1, 3});
      const auto dt = static_cast<at::ScalarType>(ctx->saved_data[key].toInt());
      return dt == at::kBFloat16 ? r : r.to(dt);
    };
    return {back(dq, "qd"), back(dk, "kd"), back(dv, "vd"), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

// ---- softmax cross-entropy ---------------------------------------------------------------------------
// One kernel produces the mean loss and d(loss)/d(logits); backward scales that buffer by the upstream scalar.
struct CrossEntropyFn : public torch::autograd::Function<CrossEntropyFn> {
  static Tensor forward(AutogradContext* ctx, const Tensor& logits_in, const Tensor& target, int64_t ignore_index) {
    c10::cuda::CUDAGuard guard(logits_in.device());
    Tensor logits = logits_in.stride(1) == 1 ? logits_in : logits_in.contiguous();
    const int64_t rows = logits.size(0), V = logits.size(1);
    auto fopts = torch::dtype(torch::kFloat).device(logits.device());
    Tensor count_inv = torch::empty({2}, fopts), row_loss = torch::empty({rows}, fopts), loss = torch::empty({}, fopts);
    const bool want_grad = ctx->needs_input_grad(0);
    Tensor dl;
    if (want_grad) dl = torch::empty({rows, logits.stride(0)}, logits.options()).narrow(1, 0, V);
    Tensor tgt = target.contiguous();
    check(fb_softmax_ce(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(tgt.data_ptr<int64_t>()), static_cast<int>(rows),
                        static_cast<int>(V), ignore_index, want_grad ? dl.data_ptr() : nullptr, want_grad ? dl.stride(0) : 0, count_inv.data_ptr<float>(),
                        row_loss.data_ptr<float>(), loss.data_ptr<float>(), is_bf16(logits), stream_of(logits)),
          "fb_softmax_ce");
    if (want_grad) ctx->save_for_backward({dl});
    return loss;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grads) {
    Tensor dl = ctx->get_saved_variables()[0];
    c10::cuda::CUDAGuard guard(dl.device());
    Tensor g = grads[0].to(at::kFloat).reshape({1}).contiguous();
    check(fb_scale_rows(dl.data_ptr(), dl.stride(0), static_cast<int>(dl.size(0)), static_cast<int>(dl.size(1)), g.data_ptr<float>(), is_bf16(dl), stream_of(dl)),
          "fb_scale_rows");
    return {dl, Tensor(), Tensor()};
  }
};

}  // namespace

void note_mutation() { g_epoch.fetch_add(1, std::memory_order_relaxed); }

bool native_linear(const Tensor& x, const Tensor& w, const Tensor& b, Tensor* out) {
  if (!op_on("linear") || !bf16_compute(x) || w.dim() != 2 || !w.is_cuda() || x.dim() < 1 || x.size(-1) != w.size(1) || x.size(-1) % 8 != 0) return false;
  if (!(w.scalar_type() == at::kFloat || is_bf16(w))) return false;
  if (b.defined() && !(b.is_cuda() && (b.scalar_type() == at::kFloat || is_bf16(b)) && b.numel() == w.size(0))) return false;
  if (x.numel() / x.size(-1) >= (1ll << 31) || w.size(0) >= (1ll << 31)) return false;
  *out = LinearFn::apply(x, w, b);
  g_native_calls.fetch_add(1, std::memory_order_relaxed);
  return true;
}

bool native_layer_norm(const Tensor& x, const Tensor& w, const Tensor& b, int64_t size, double eps, Tensor* out, Tensor* mean, Tensor* rstd) {
  if (!op_on("layer_norm") || !natives_on() || !x.defined() || !x.is_cuda() || x.numel() == 0 || x.size(-1) != size) return false;
  if (!(is_bf16(x) || x.scalar_type() == at::kFloat)) return false;
  if (size > 1024 || size % (is_bf16(x) ? 8 : 4) != 0) return false;
  auto affine_ok = [&](const Tensor& t) { return !t.defined() || (t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == size); };
  if (!affine_ok(w) || !affine_ok(b)) return false;
  auto res = LayerNormFn::apply(x, w, b, eps);
  *out = res[0];
  *mean = res[1];
  *rstd = res[2];
  g_native_calls.fetch_add(1, std::memory_order_relaxed);
  return true;
}

bool native_gelu(const Tensor& x, bool tanh_approx, Tensor* out) {
  if (!op_on("gelu") || !natives_on() || !x.defined() || !x.is_cuda() || x.numel() == 0 || !(is_bf16(x) || x.scalar_type() == at::kFloat)) return false;
  *out = GeluFn::apply(x, tanh_approx);
  g_native_calls.fetch_add(1, std::memory_order_relaxed);
  return true;
}

bool native_dropout(const Tensor& x, double p, bool training, Tensor* out) {
  if (!training || p <= 0.0 || p >= 1.0 || !op_on("dropout")) return false;
  if (!natives_on() || !x.defined() || !x.is_cuda() || x.numel() == 0 || !(is_bf16(x) || x.scalar_type() == at::kFloat)) return false;
  *out = DropoutFn::apply(x, p);
  g_native_calls.fetch_add(1, std::memory_order_relaxed);
  return true;
}

bool native_sdpa(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, double p, bool causal, double scale, Tensor* out) {
  if (!op_on("sdpa") || !bf16_compute(q) || q.dim() != 4 || q.size(3) != 64) return false;
  if (k.sizes() != q.sizes() || v.sizes() != q.sizes() || !k.is_cuda() || !v.is_cuda()) return false;
  Tensor m;
  if (mask.defined()) {
    // key-padding masks only: something that broadcasts from [B or 1, 1, 1, S]
    if (mask.dim() != 4 || mask.size(1) != 1 || mask.size(2) != 1 || mask.size(3) != q.size(2)) return false;
    if (mask.size(0) != q.size(0) && mask.size(0) != 1) return false;
    Tensor flat = mask.expand({q.size(0), 1, 1, q.size(2)}).reshape({q.size(0), q.size(2)});
    if (flat.scalar_type() == at::kBool)
      m = torch::zeros(flat.sizes(), flat.options().dtype(at::kFloat)).masked_fill_(flat.logical_not(), -std::numeric_limits<float>::infinity());
    else
      m = flat.to(at::kFloat).contiguous();
  }
  const double sc = scale > 0.0 ? scale : 0.125;
  *out = AttnFn::apply(q, k, v, m, p, causal, sc);
  g_native_calls.fetch_add(1, std::memory_order_relaxed);
  return true;
}

bool native_cross_entropy(const Tensor& logits, const Tensor& target, int64_t reduction, int64_t ignore_index, double smoothing, Tensor* out) {
  if (!op_on("cross_entropy") || !natives_on() || !logits.defined() || !logits.is_cuda() || logits.dim() != 2 || logits.numel() == 0) return false;
  if (reduction != 1 || smoothing != 0.0 || !(is_bf16(logits) || logits.scalar_type() == at::kFloat)) return false;
  if (!target.is_cuda() || target.scalar_type() != at::kLong || target.dim() != 1 || target.size(0) != logits.size(0)) return false;
  if (logits.size(0) >= (1ll << 31) || logits.size(1) >= (1ll << 31)) return false;
  *out = CrossEntropyFn::apply(logits, target, ignore_index);
  g_native_calls.fetch_add(1, std::memory_order_relaxed);
  return true;
}

extern "C" __attribute__((visibility("default"))) long long flodl_b200_native_calls(void) { return g_native_calls.load(); }

}  // namespace fbabi
