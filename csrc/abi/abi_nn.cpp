// Drop-in C ABI, part 2: neural-network ops (normalisation, convolution, pooling, attention, linear,
// recurrent cells and sequences, losses, dropout, embedding). Ops with a native sm_100a path try it
// first (`native_*` in abi_native.cpp) and fall back to ATen.
#include "abi_common.hpp"

using namespace fbabi;

#define FB_API extern "C" __attribute__((visibility("default")))

static at::IntArrayRef two(const int64_t* p) { return at::IntArrayRef(p, 2); }
static at::IntArrayRef three(const int64_t* p) { return at::IntArrayRef(p, 3); }

// ---- normalisation ---------------------------------------------------------------------------------------
FB_API char* flodl_native_layer_norm(Handle input, Handle weight, Handle bias, int64_t normalized_size, double eps, Handle* output,
                                     Handle* mean, Handle* rstd) {
  return guarded([&] {
    Tensor o, m, r;
    if (!native_layer_norm(ref(input), opt(weight), opt(bias), normalized_size, eps, &o, &m, &r)) {
      auto res = at::native_layer_norm(ref(input), {normalized_size}, optional_of(weight), optional_of(bias), eps);
      o = std::get<0>(res);
      m = std::get<1>(res);
      r = std::get<2>(res);
    }
    *output = box(o);
    *mean = box(m);
    *rstd = box(r);
  });
}
FB_API char* flodl_group_norm(Handle input, int64_t num_groups, Handle weight, Handle bias, double eps, Handle* result) {
  return guarded([&] { *result = box(at::group_norm(ref(input), num_groups, optional_of(weight), optional_of(bias), eps)); });
}
FB_API char* flodl_instance_norm(Handle input, Handle weight, Handle bias, Handle running_mean, Handle running_var, int use_input_stats,
                                 double momentum, double eps, Handle* result) {
  return guarded([&] {
    *result = box(at::instance_norm(ref(input), optional_of(weight), optional_of(bias), optional_of(running_mean), optional_of(running_var),
                                    use_input_stats != 0, momentum, eps, /*cudnn_enabled=*/true));
  });
}
FB_API char* flodl_batch_norm(Handle input, Handle weight, Handle bias, Handle running_mean, Handle running_var, int training, double momentum,
                              double eps, Handle* result) {
  return guarded([&] {
    *result = box(at::batch_norm(ref(input), optional_of(weight), optional_of(bias), optional_of(running_mean), optional_of(running_var),
                                 training != 0, momentum, eps, /*cudnn_enabled=*/true));
  });
}
FB_API char* flodl_normalize(Handle t, double p, int dim, Handle* result) {
  return guarded([&] {
    const Tensor& x = ref(t);
    *result = box(x / x.norm(p, at::IntArrayRef{dim}, true).clamp_min(1e-12));
  });
}
FB_API char* flodl_cosine_similarity(Handle a, Handle b, int64_t dim, double eps, Handle* result) {
  return guarded([&] { *result = box(at::cosine_similarity(ref(a), ref(b), dim, eps)); });
}
FB_API char* flodl_cdist(Handle x, Handle y, double p, Handle* result) { return guarded([&] { *result = box(at::cdist(ref(x), ref(y), p)); }); }

// ---- convolution / pooling -----------------------------------------------------------------------------------
FB_API char* flodl_conv2d(Handle input, Handle weight, Handle bias, int64_t* stride, int64_t* padding, int64_t* dilation, int64_t groups,
                          Handle* result) {
  return guarded([&] { *result = box(at::conv2d(ref(input), ref(weight), optional_of(bias), two(stride), two(padding), two(dilation), groups)); });
}
FB_API char* flodl_conv1d(Handle input, Handle weight, Handle bias, int64_t stride, int64_t padding, int64_t dilation, int64_t groups,
                          Handle* result) {
  return guarded([&] { *result = box(at::conv1d(ref(input), ref(weight), optional_of(bias), {stride}, {padding}, {dilation}, groups)); });
}
FB_API char* flodl_conv3d(Handle input, Handle weight, Handle bias, int64_t* stride, int64_t* padding, int64_t* dilation, int64_t groups,
                          Handle* result) {
  return guarded([&] { *result = box(at::conv3d(ref(input), ref(weight), optional_of(bias), three(stride), three(padding), three(dilation), groups)); });
}
FB_API char* flodl_conv_transpose2d(Handle input, Handle weight, Handle bias, int64_t* stride, int64_t* padding, int64_t* output_padding,
                                    int64_t* dilation, int64_t groups, Handle* result) {
  return guarded([&] {
    *result = box(at::conv_transpose2d(ref(input), ref(weight), optional_of(bias), two(stride), two(padding), two(output_padding), groups, two(dilation)));
  });
}
FB_API char* flodl_conv_transpose1d(Handle input, Handle weight, Handle bias, int64_t stride, int64_t padding, int64_t output_padding,
                                    int64_t dilation, int64_t groups, Handle* result) {
  return guarded([&] {
    *result = box(at::conv_transpose1d(ref(input), ref(weight), optional_of(bias), {stride}, {padding}, {output_padding}, groups, {dilation}));
  });
}
FB_API char* flodl_conv_transpose3d(Handle input, Handle weight, Handle bias, int64_t* stride, int64_t* padding, int64_t* output_padding,
                                    int64_t* dilation, int64_t groups, Handle* result) {
  return guarded([&] {
    *result = box(at::conv_transpose3d(ref(input), ref(weight), optional_of(bias), three(stride), three(padding), three(output_padding), groups,
                                       three(dilation)));
  });
}
FB_API char* flodl_max_pool2d(Handle input, int64_t* kernel, int64_t* stride, int64_t* padding, int64_t* dilation, int ceil_mode, Handle* result) {
  return guarded([&] { *result = box(at::max_pool2d(ref(input), two(kernel), two(stride), two(padding), two(dilation), ceil_mode != 0)); });
}
FB_API char* flodl_avg_pool2d(Handle input, int64_t* kernel, int64_t* stride, int64_t* padding, int ceil_mode, int count_include_pad,
                              Handle* result) {
  return guarded([&] { *result = box(at::avg_pool2d(ref(input), two(kernel), two(stride), two(padding), ceil_mode != 0, count_include_pad != 0)); });
}
FB_API char* flodl_adaptive_avg_pool2d(Handle input, int64_t* output_size, Handle* result) {
  return guarded([&] { *result = box(at::adaptive_avg_pool2d(ref(input), two(output_size))); });
}
FB_API char* flodl_adaptive_max_pool2d(Handle input, int64_t* output_size, Handle* result) {
  return guarded([&] { *result = box(std::get<0>(at::adaptive_max_pool2d(ref(input), two(output_size)))); });
}
FB_API char* flodl_max_pool1d(Handle input, int64_t kernel, int64_t stride, int64_t padding, int64_t dilation, int ceil_mode, Handle* result) {
  return guarded([&] { *result = box(at::max_pool1d(ref(input), {kernel}, {stride}, {padding}, {dilation}, ceil_mode != 0)); });
}
FB_API char* flodl_avg_pool1d(Handle input, int64_t kernel, int64_t stride, int64_t padding, int ceil_mode, int count_include_pad,
                              Handle* result) {
  return guarded([&] { *result = box(at::avg_pool1d(ref(input), {kernel}, {stride}, {padding}, ceil_mode != 0, count_include_pad != 0)); });
}
FB_API char* flodl_im2col(Handle input, int64_t* kernel, int64_t* dilation, int64_t* padding, int64_t* stride, Handle* result) {
  return guarded([&] { *result = box(at::im2col(ref(input), two(kernel), two(dilation), two(padding), two(stride))); });
}
FB_API char* flodl_col2im(Handle input, int64_t* output_size, int64_t* kernel, int64_t* dilation, int64_t* padding, int64_t* stride,
                          Handle* result) {
  return guarded([&] { *result = box(at::col2im(ref(input), two(output_size), two(kernel), two(dilation), two(padding), two(stride))); });
}
FB_API char* flodl_pixel_shuffle(Handle input, int64_t factor, Handle* result) { return guarded([&] { *result = box(at::pixel_shuffle(ref(input), factor)); }); }
FB_API char* flodl_pixel_unshuffle(Handle input, int64_t factor, Handle* result) {
  return guarded([&] { *result = box(at::pixel_unshuffle(ref(input), factor)); });
}
FB_API char* flodl_interpolate(Handle input, int64_t* output_size, int ndim, int mode, int align_corners, Handle* result) {
  return guarded([&] {
    const Tensor& x = ref(input);
    const at::IntArrayRef size(output_size, static_cast<size_t>(ndim));
    const bool ac = align_corners != 0;
    switch (mode) {
      case 0:
        *result = box(ndim == 1 ? at::upsample_nearest1d(x, size) : ndim == 2 ? at::upsample_nearest2d(x, size) : at::upsample_nearest3d(x, size));
        break;
      case 1: *result = box(ndim == 1 ? at::upsample_linear1d(x, size, ac) : at::upsample_bilinear2d(x, size, ac)); break;
      case 2: *result = box(at::upsample_bicubic2d(x, size, ac)); break;
      case 3: *result = box(at::upsample_trilinear3d(x, size, ac)); break;
      default: TORCH_CHECK(false, "interpolate: unknown mode ", mode);
    }
  });
}
FB_API char* flodl_grid_sample(Handle input, Handle grid, int mode, int padding_mode, int align_corners, Handle* result) {
  return guarded([&] { *result = box(at::grid_sampler(ref(input), ref(grid), mode, padding_mode, align_corners != 0)); });
}
FB_API char* flodl_bilinear(Handle x1, Handle x2, Handle weight, Handle bias, Handle* result) {
  return guarded([&] { *result = box(at::bilinear(ref(x1), ref(x2), ref(weight), optional_of(bias))); });
}

// ---- attention / linear / recurrent ---------------------------------------------------------------------------
FB_API char* flodl_scaled_dot_product_attention(Handle query, Handle key, Handle value, Handle attn_mask, double dropout_p, int is_causal,
                                                double scale, Handle* result) {
  return guarded([&] {
    Tensor out;
    if (!native_sdpa(ref(query), ref(key), ref(value), opt(attn_mask), dropout_p, is_causal != 0, scale, &out)) {
      out = at::scaled_dot_product_attention(ref(query), ref(key), ref(value), optional_of(attn_mask), dropout_p, is_causal != 0,
                                             scale > 0.0 ? c10::optional<double>(scale) : c10::nullopt);
    }
    *result = box(out);
  });
}
FB_API char* flodl_linear(Handle input, Handle weight, Handle bias, Handle* result) {
  return guarded([&] {
    Tensor out;
    *result = box(native_linear(ref(input), ref(weight), opt(bias), &out) ? out : at::linear(ref(input), ref(weight), optional_of(bias)));
  });
}
FB_API char* flodl_gru_cell(Handle input, Handle hx, Handle w_ih, Handle w_hh, Handle b_ih, Handle b_hh, Handle* result) {
  return guarded([&] { *result = box(at::gru_cell(ref(input), ref(hx), ref(w_ih), ref(w_hh), optional_of(b_ih), optional_of(b_hh))); });
}
FB_API char* flodl_lstm_cell(Handle input, Handle hx, Handle cx, Handle w_ih, Handle w_hh, Handle b_ih, Handle b_hh, Handle* h_out, Handle* c_out) {
  return guarded([&] {
    auto r = at::lstm_cell(ref(input), {ref(hx), ref(cx)}, ref(w_ih), ref(w_hh), optional_of(b_ih), optional_of(b_hh));
    *h_out = box(std::get<0>(r));
    *c_out = box(std::get<1>(r));
  });
}

namespace {
// Parameters of a cuDNN sequence op, optionally packed into the one contiguous buffer cuDNN wants
// (done once here instead of on every forward). mode: 2 = LSTM, 3 = GRU (cuDNN's numbering).
struct RnnParams {
  std::vector<Tensor> params;
};
void pack_for_cudnn(std::vector<Tensor>& ps, int64_t mode, int64_t num_layers, bool batch_first) {
  if (ps.empty() || !ps[0].is_cuda() || !at::cudnn_is_acceptable(ps[0])) return;
  const int64_t gates = mode == 2 ? 4 : 3;
  const int64_t hidden = ps[0].size(0) / gates;
  const int64_t input_size = ps[0].size(1);
  at::_cudnn_rnn_flatten_weight(ps, /*weight_stride0=*/4, input_size, mode, hidden, /*proj_size=*/0, num_layers, batch_first, /*bidirectional=*/false);
}
std::vector<Tensor> gather_params(const Handle* params, int64_t n) {
  std::vector<Tensor> out;
  out.reserve(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) out.push_back(ref(params[i]));
  return out;
}
void run_lstm(const Tensor& x, const Tensor& h0, const Tensor& c0, const std::vector<Tensor>& ps, int64_t layers, bool batch_first, Handle* out,
              Handle* hn, Handle* cn) {
  auto r = at::lstm(x, {h0, c0}, ps, /*has_biases=*/true, layers, /*dropout=*/0.0, /*train=*/true, /*bidirectional=*/false, batch_first);
  *out = box(std::get<0>(r));
  *hn = box(std::get<1>(r));
  *cn = box(std::get<2>(r));
}
void run_gru(const Tensor& x, const Tensor& h0, const std::vector<Tensor>& ps, int64_t layers, bool batch_first, Handle* out, Handle* hn) {
  auto r = at::gru(x, h0, ps, /*has_biases=*/true, layers, /*dropout=*/0.0, /*train=*/true, /*bidirectional=*/false, batch_first);
  *out = box(std::get<0>(r));
  *hn = box(std::get<1>(r));
}
}  // namespace

FB_API char* flodl_lstm(Handle input, Handle h_0, Handle c_0, const Handle* params, int64_t num_params, int64_t num_layers, bool batch_first,
                        bool flatten, Handle* output, Handle* h_n, Handle* c_n) {
  return guarded([&] {
    auto ps = gather_params(params, num_params);
    if (flatten) pack_for_cudnn(ps, 2, num_layers, batch_first);
    run_lstm(ref(input), ref(h_0), ref(c_0), ps, num_layers, batch_first, output, h_n, c_n);
  });
}
FB_API char* flodl_gru(Handle input, Handle h_0, const Handle* params, int64_t num_params, int64_t num_layers, bool batch_first, bool flatten,
                       Handle* output, Handle* h_n) {
  return guarded([&] {
    auto ps = gather_params(params, num_params);
    if (flatten) pack_for_cudnn(ps, 3, num_layers, batch_first);
    run_gru(ref(input), ref(h_0), ps, num_layers, batch_first, output, h_n);
  });
}
FB_API char* flodl_rnn_params_create(const Handle* params, int64_t num_params, int64_t mode, int64_t num_layers, bool batch_first, bool flatten,
                                     void** out) {
  return guarded([&] {
    auto rp = std::make_unique<RnnParams>();
    rp->params = gather_params(params, num_params);
    if (flatten) pack_for_cudnn(rp->params, mode, num_layers, batch_first);
    *out = rp.release();
  });
}
FB_API void flodl_rnn_params_free(void* rp) { delete static_cast<RnnParams*>(rp); }
FB_API char* flodl_lstm_cached(Handle input, Handle h_0, Handle c_0, void* rp, int64_t num_layers, bool batch_first, Handle* output, Handle* h_n,
                               Handle* c_n) {
  return guarded([&] { run_lstm(ref(input), ref(h_0), ref(c_0), static_cast<RnnParams*>(rp)->params, num_layers, batch_first, output, h_n, c_n); });
}
FB_API char* flodl_gru_cached(Handle input, Handle h_0, void* rp, int64_t num_layers, bool batch_first, Handle* output, Handle* h_n) {
  return guarded([&] { run_gru(ref(input), ref(h_0), static_cast<RnnParams*>(rp)->params, num_layers, batch_first, output, h_n); });
}

// ---- losses (reduction: 0 none, 1 mean, 2 sum) ----------------------------------------------------------------
FB_API char* flodl_mse_loss(Handle pred, Handle target, int64_t reduction, Handle* result) {
  return guarded([&] { *result = box(at::mse_loss(ref(pred), ref(target), reduction)); });
}
FB_API char* flodl_cross_entropy_loss(Handle pred, Handle target, int64_t reduction, int64_t ignore_index, double label_smoothing, Handle* result) {
  return guarded([&] {
    Tensor out;
    if (!native_cross_entropy(ref(pred), ref(target), reduction, ignore_index, label_smoothing, &out))
      out = at::cross_entropy_loss(ref(pred), ref(target), c10::nullopt, reduction, ignore_index, label_smoothing);
    *result = box(out);
  });
}
FB_API char* flodl_bce_with_logits_loss(Handle pred, Handle target, int64_t reduction, Handle* result) {
  return guarded([&] { *result = box(at::binary_cross_entropy_with_logits(ref(pred), ref(target), c10::nullopt, c10::nullopt, reduction)); });
}
FB_API char* flodl_bce_loss(Handle pred, Handle target, int64_t reduction, Handle* result) {
  return guarded([&] { *result = box(at::binary_cross_entropy(ref(pred), ref(target), c10::nullopt, reduction)); });
}
FB_API char* flodl_l1_loss(Handle pred, Handle target, int64_t reduction, Handle* result) {
  return guarded([&] { *result = box(at::l1_loss(ref(pred), ref(target), reduction)); });
}
FB_API char* flodl_smooth_l1_loss(Handle pred, Handle target, int64_t reduction, double beta, Handle* result) {
  return guarded([&] { *result = box(at::smooth_l1_loss(ref(pred), ref(target), reduction, beta)); });
}
FB_API char* flodl_kl_div_loss(Handle input, Handle target, int64_t reduction, int log_target, Handle* result) {
  return guarded([&] { *result = box(at::kl_div(ref(input), ref(target), reduction, log_target != 0)); });
}
FB_API char* flodl_nll_loss(Handle input, Handle target, int64_t reduction, int64_t ignore_index, Handle* result) {
  return guarded([&] { *result = box(at::nll_loss(ref(input), ref(target), c10::nullopt, reduction, ignore_index)); });
}
FB_API char* flodl_ctc_loss(Handle log_probs, Handle targets, Handle input_lengths, Handle target_lengths, int64_t blank, int64_t reduction,
                            Handle* result) {
  return guarded([&] { *result = box(at::ctc_loss(ref(log_probs), ref(targets), ref(input_lengths), ref(target_lengths), blank, reduction, false)); });
}

// ---- dropout / embedding --------------------------------------------------------------------------------------
FB_API char* flodl_dropout(Handle input, double p, int training, Handle* result) {
  return guarded([&] {
    Tensor out;
    *result = box(native_dropout(ref(input), p, training != 0, &out) ? out : at::dropout(ref(input), p, training != 0));
  });
}
FB_API char* flodl_feature_dropout(Handle input, double p, int training, Handle* result) {
  return guarded([&] { *result = box(at::feature_dropout(ref(input), p, training != 0)); });
}
FB_API char* flodl_embedding(Handle weight, Handle indices, int64_t padding_idx, int scale_grad_by_freq, int sparse, Handle* result) {
  return guarded([&] { *result = box(at::embedding(ref(weight), ref(indices), padding_idx, scale_grad_by_freq != 0, sparse != 0)); });
}
FB_API char* flodl_embedding_bag(Handle weight, Handle indices, Handle offsets, int64_t mode, Handle* result) {
  return guarded([&] { *result = box(std::get<0>(at::embedding_bag(ref(weight), ref(indices), ref(offsets), false, mode))); });
}
