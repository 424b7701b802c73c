// Drop-in C ABI, part 1: tensor creation, lifecycle, metadata, arithmetic, math, reductions, comparisons,
// shape and indexing. One table entry per function; the bodies are the ATen call the name says.
// Function names and argument lists are those of the interface hosts are written against
// (flodl-sys/shim.h); see abi_common.hpp for the conventions.
#include "abi_common.hpp"

using namespace fbabi;

#define FB_API extern "C" __attribute__((visibility("default")))

// ---- table macros ------------------------------------------------------------------------------------
#define FB_UNARY(NAME, EXPR) \
  FB_API char* flodl_##NAME(Handle t, Handle* result) { return guarded([&] { const Tensor& x = ref(t); *result = box(EXPR); }); }
#define FB_BINARY(NAME, EXPR) \
  FB_API char* flodl_##NAME(Handle a_, Handle b_, Handle* result) { \
    return guarded([&] { const Tensor& a = ref(a_); const Tensor& b = ref(b_); *result = box(EXPR); }); }
#define FB_SCALAR(NAME, EXPR) \
  FB_API char* flodl_##NAME(Handle t, double s, Handle* result) { return guarded([&] { const Tensor& x = ref(t); *result = box(EXPR); }); }
#define FB_DIMRED(NAME, EXPR) \
  FB_API char* flodl_##NAME(Handle t, int dim, int keepdim, Handle* result) { \
    return guarded([&] { const Tensor& x = ref(t); const bool keep = keepdim != 0; *result = box(EXPR); }); }
#define FB_CREATE(NAME, FN) \
  FB_API char* flodl_##NAME(int64_t* shape, int ndim, int dtype, int dev_type, int dev_index, Handle* result) { \
    return guarded([&] { *result = box(FN(dims(shape, ndim), options_of(dtype, dev_type, dev_index))); }); }
#define FB_LIKE(NAME, EXPR) FB_UNARY(NAME, EXPR)

// ---- creation ----------------------------------------------------------------------------------------
FB_CREATE(zeros, at::zeros)
FB_CREATE(ones, at::ones)
FB_CREATE(rand, at::rand)
FB_CREATE(randn, at::randn)
FB_CREATE(empty, at::empty)
FB_API char* flodl_full(int64_t* shape, int ndim, double value, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(at::full(dims(shape, ndim), value, options_of(dtype, dev_type, dev_index))); });
}
FB_API char* flodl_from_blob(void* data, int64_t* shape, int ndim, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] {
    // the caller keeps ownership of `data`: take a private copy, then move it where it was asked for
    Tensor t = at::from_blob(data, dims(shape, ndim), at::TensorOptions().dtype(dtype_of(dtype))).clone();
    *result = box(dev_type == 1 ? t.to(device_of(dev_type, dev_index)) : t);
  });
}
FB_API char* flodl_linspace(double start, double end, int64_t steps, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(at::linspace(start, end, steps, options_of(dtype, dev_type, dev_index))); });
}
FB_API char* flodl_arange(double start, double end, double step, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(at::arange(start, end, step, options_of(dtype, dev_type, dev_index))); });
}
FB_API char* flodl_eye(int64_t n, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(at::eye(n, options_of(dtype, dev_type, dev_index))); });
}
FB_API char* flodl_randperm(int64_t n, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(at::randperm(n, options_of(dtype, dev_type, dev_index))); });
}
FB_API char* flodl_randint(int64_t low, int64_t high, int64_t* shape, int ndim, int dtype, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(at::randint(low, high, dims(shape, ndim), options_of(dtype, dev_type, dev_index))); });
}
FB_API char* flodl_multinomial(Handle probs, int64_t num_samples, int replacement, Handle* result) {
  return guarded([&] { *result = box(at::multinomial(ref(probs), num_samples, replacement != 0)); });
}
FB_LIKE(zeros_like, at::zeros_like(x))
FB_LIKE(ones_like, at::ones_like(x))
FB_LIKE(rand_like, at::rand_like(x))
FB_LIKE(randn_like, at::randn_like(x))
FB_LIKE(bernoulli, at::bernoulli(x))
FB_SCALAR(full_like, at::full_like(x, s))
FB_API char* flodl_one_hot(Handle t, int64_t num_classes, Handle* result) {
  return guarded([&] { *result = box(at::one_hot(ref(t), num_classes).to(at::kFloat)); });
}

// ---- lifecycle / metadata / data access ----------------------------------------------------------------
FB_API void flodl_free_tensor(Handle t) { delete static_cast<Tensor*>(t); }
FB_API void flodl_free_string(char* s) { std::free(s); }
FB_UNARY(shallow_clone, Tensor(x))
FB_API int flodl_ndim(Handle t) { return static_cast<int>(ref(t).dim()); }
FB_API int64_t flodl_shape(Handle t, int dim) { return ref(t).size(dim); }
FB_API int flodl_dtype(Handle t) { return tag_of(ref(t).scalar_type()); }
FB_API int flodl_device_type(Handle t) { return ref(t).is_cuda() ? 1 : 0; }
FB_API int flodl_device_index(Handle t) { return ref(t).is_cuda() ? static_cast<int>(ref(t).device().index()) : 0; }
FB_API int64_t flodl_numel(Handle t) { return ref(t).numel(); }
FB_API int flodl_is_contiguous(Handle t) { return ref(t).is_contiguous() ? 1 : 0; }
FB_API char* flodl_copy_data(Handle t, void* buffer, int64_t buffer_bytes) {
  return guarded([&] {
    Tensor host = ref(t).detach().to(at::kCPU).contiguous();
    const int64_t need = host.numel() * static_cast<int64_t>(host.element_size());
    TORCH_CHECK(buffer_bytes >= need, "buffer too small: need ", need, " bytes, got ", buffer_bytes);
    std::memcpy(buffer, host.data_ptr(), static_cast<size_t>(need));
  });
}

// ---- arithmetic ----------------------------------------------------------------------------------------
FB_BINARY(add, a + b)
FB_BINARY(sub, a - b)
FB_BINARY(mul, a * b)
FB_BINARY(div, a / b)
FB_BINARY(matmul, at::matmul(a, b))
FB_BINARY(atan2, at::atan2(a, b))
FB_BINARY(maximum, at::maximum(a, b))
FB_BINARY(minimum, at::minimum(a, b))
FB_BINARY(fmod_tensor, at::fmod(a, b))
FB_BINARY(remainder_tensor, at::remainder(a, b))
FB_SCALAR(add_scalar, x + s)
FB_SCALAR(mul_scalar, x * s)
FB_SCALAR(div_scalar, x / s)
FB_SCALAR(pow_scalar, at::pow(x, s))
FB_SCALAR(clamp_min, at::clamp_min(x, s))
FB_SCALAR(clamp_max, at::clamp_max(x, s))
FB_SCALAR(fmod_scalar, at::fmod(x, s))
FB_SCALAR(remainder_scalar, at::remainder(x, s))
FB_SCALAR(leaky_relu, at::leaky_relu(x, s))
FB_SCALAR(elu, at::elu(x, s))
FB_UNARY(neg, -x)

// ---- activations and element-wise math --------------------------------------------------------------------
FB_UNARY(relu, at::relu(x))
FB_UNARY(sigmoid, at::sigmoid(x))
FB_UNARY(tanh_op, at::tanh(x))
FB_UNARY(silu, at::silu(x))
FB_UNARY(mish, at::mish(x))
FB_UNARY(selu, at::selu(x))
FB_UNARY(hardswish, at::hardswish(x))
FB_UNARY(hardsigmoid, at::hardsigmoid(x))
FB_UNARY(exp, at::exp(x))
FB_UNARY(log, at::log(x))
FB_UNARY(sqrt, at::sqrt(x))
FB_UNARY(abs, at::abs(x))
FB_UNARY(log1p, at::log1p(x))
FB_UNARY(expm1, at::expm1(x))
FB_UNARY(log2, at::log2(x))
FB_UNARY(log10, at::log10(x))
FB_UNARY(sin, at::sin(x))
FB_UNARY(cos, at::cos(x))
FB_UNARY(tan, at::tan(x))
FB_UNARY(asin, at::asin(x))
FB_UNARY(acos, at::acos(x))
FB_UNARY(atan, at::atan(x))
FB_UNARY(sign, at::sign(x))
FB_UNARY(floor, at::floor(x))
FB_UNARY(ceil, at::ceil(x))
FB_UNARY(round, at::round(x))
FB_UNARY(reciprocal, at::reciprocal(x))
FB_UNARY(erf, at::erf(x))
FB_UNARY(erfc, at::erfc(x))
FB_UNARY(trunc, at::trunc(x))
FB_UNARY(frac, at::frac(x))
FB_UNARY(contiguous, x.contiguous())
FB_API char* flodl_gelu(Handle t, Handle* result) {
  return guarded([&] {
    Tensor out;
    *result = box(native_gelu(ref(t), false, &out) ? out : at::gelu(ref(t)));
  });
}
FB_API char* flodl_gelu_tanh(Handle t, Handle* result) {
  return guarded([&] {
    Tensor out;
    *result = box(native_gelu(ref(t), true, &out) ? out : at::gelu(ref(t), "tanh"));
  });
}
FB_API char* flodl_softmax(Handle t, int dim, Handle* result) { return guarded([&] { *result = box(at::softmax(ref(t), dim)); }); }
FB_API char* flodl_log_softmax(Handle t, int dim, Handle* result) { return guarded([&] { *result = box(at::log_softmax(ref(t), dim)); }); }
FB_API char* flodl_softplus(Handle t, double beta, double threshold, Handle* result) {
  return guarded([&] { *result = box(at::softplus(ref(t), beta, threshold)); });
}
FB_BINARY(prelu, at::prelu(a, b))
FB_API char* flodl_clamp(Handle t, double lo, double hi, Handle* result) { return guarded([&] { *result = box(at::clamp(ref(t), lo, hi)); }); }
FB_API char* flodl_triu(Handle t, int64_t diagonal, Handle* result) { return guarded([&] { *result = box(at::triu(ref(t), diagonal)); }); }
FB_API char* flodl_tril(Handle t, int64_t diagonal, Handle* result) { return guarded([&] { *result = box(at::tril(ref(t), diagonal)); }); }
FB_API char* flodl_lerp(Handle a, Handle b, double weight, Handle* result) {
  return guarded([&] { *result = box(at::lerp(ref(a), ref(b), weight)); });
}
FB_API char* flodl_lerp_tensor(Handle a, Handle b, Handle weight, Handle* result) {
  return guarded([&] { *result = box(at::lerp(ref(a), ref(b), ref(weight))); });
}
FB_API char* flodl_isclose(Handle a, Handle b, double rtol, double atol, Handle* result) {
  return guarded([&] { *result = box(as_mask(at::isclose(ref(a), ref(b), rtol, atol), ref(a))); });
}
FB_API char* flodl_addmm(Handle bias, Handle m1, Handle m2, double beta, double alpha, Handle* result) {
  return guarded([&] { *result = box(at::addmm(ref(bias), ref(m1), ref(m2), beta, alpha)); });
}
FB_API char* flodl_addcmul(Handle self, Handle t1, Handle t2, double value, Handle* result) {
  return guarded([&] { *result = box(at::addcmul(ref(self), ref(t1), ref(t2), value)); });
}
FB_API char* flodl_addcdiv(Handle self, Handle t1, Handle t2, double value, Handle* result) {
  return guarded([&] { *result = box(at::addcdiv(ref(self), ref(t1), ref(t2), value)); });
}

// ---- reductions ------------------------------------------------------------------------------------------
FB_UNARY(sum, x.sum())
FB_UNARY(mean, x.mean())
FB_UNARY(prod, x.prod())
FB_UNARY(min, x.min())
FB_UNARY(max, x.max())
FB_UNARY(norm, x.norm())
FB_UNARY(var, x.var())
FB_UNARY(std_op, x.std())
FB_UNARY(median, x.median())
FB_UNARY(count_nonzero, at::count_nonzero(x))
FB_UNARY(nonzero, at::nonzero(x))
FB_DIMRED(sum_dim, x.sum(dim, keep))
FB_DIMRED(mean_dim, x.mean(dim, keep))
FB_DIMRED(prod_dim, x.prod(dim, keep))
FB_DIMRED(logsumexp, at::logsumexp(x, dim, keep))
FB_DIMRED(min_dim, std::get<0>(x.min(dim, keep)))
FB_DIMRED(max_dim, std::get<0>(x.max(dim, keep)))
FB_DIMRED(argmax, x.argmax(dim, keep))
FB_DIMRED(argmin, x.argmin(dim, keep))
FB_DIMRED(var_dim, x.var(at::IntArrayRef{dim}, true, keep))
FB_DIMRED(std_dim, x.std(at::IntArrayRef{dim}, true, keep))
FB_API char* flodl_cumsum(Handle t, int dim, Handle* result) { return guarded([&] { *result = box(ref(t).cumsum(dim)); }); }
FB_API char* flodl_cumprod(Handle t, int dim, Handle* result) { return guarded([&] { *result = box(ref(t).cumprod(dim)); }); }
FB_API char* flodl_count_nonzero_dim(Handle t, int dim, Handle* result) {
  return guarded([&] { *result = box(at::count_nonzero(ref(t), at::IntArrayRef{dim})); });
}
FB_API char* flodl_norm_p_dim(Handle t, double p, int dim, int keepdim, Handle* result) {
  return guarded([&] { *result = box(ref(t).norm(p, at::IntArrayRef{dim}, keepdim != 0)); });
}
FB_API char* flodl_sum_dims(Handle t, int64_t* ds, int n, int keepdim, Handle* result) {
  return guarded([&] { *result = box(ref(t).sum(dims(ds, n), keepdim != 0)); });
}
FB_API char* flodl_median_dim(Handle t, int dim, int keepdim, Handle* values, Handle* indices) {
  return guarded([&] {
    auto r = ref(t).median(dim, keepdim != 0);
    *values = box(std::get<0>(r));
    *indices = box(std::get<1>(r));
  });
}
FB_API char* flodl_unique(Handle t, int sorted, int return_inverse, Handle* output, Handle* inverse) {
  return guarded([&] {
    auto r = at::_unique2(ref(t), sorted != 0, return_inverse != 0, false);
    *output = box(std::get<0>(r));
    *inverse = return_inverse ? box(std::get<1>(r)) : nullptr;
  });
}
FB_BINARY(searchsorted, at::searchsorted(a, b))
FB_API char* flodl_topk(Handle t, int64_t k, int dim, int largest, int sorted, Handle* values, Handle* indices) {
  return guarded([&] {
    auto r = ref(t).topk(k, dim, largest != 0, sorted != 0);
    *values = box(std::get<0>(r));
    *indices = box(std::get<1>(r));
  });
}
FB_API char* flodl_sort(Handle t, int dim, int descending, Handle* values, Handle* indices) {
  return guarded([&] {
    auto r = ref(t).sort(dim, descending != 0);
    *values = box(std::get<0>(r));
    *indices = box(std::get<1>(r));
  });
}
FB_API char* flodl_argsort(Handle t, int dim, int descending, Handle* result) {
  return guarded([&] { *result = box(ref(t).argsort(dim, descending != 0)); });
}
FB_API char* flodl_all_finite(Handle t, int* result) {
  return guarded([&] { *result = at::isfinite(ref(t)).all().item<bool>() ? 1 : 0; });
}

// ---- comparisons and predicates (float masks) ------------------------------------------------------------------
#define FB_CMP_SCALAR(NAME, OP) FB_SCALAR(NAME, as_mask(OP(x, s), x))
#define FB_CMP_TENSOR(NAME, OP) FB_BINARY(NAME, as_mask(OP(a, b), a))
FB_CMP_SCALAR(gt_scalar, at::gt)
FB_CMP_SCALAR(ge_scalar, at::ge)
FB_CMP_SCALAR(le_scalar, at::le)
FB_CMP_SCALAR(lt_scalar, at::lt)
FB_CMP_SCALAR(eq_scalar, at::eq)
FB_CMP_SCALAR(ne_scalar, at::ne)
FB_CMP_TENSOR(gt_tensor, at::gt)
FB_CMP_TENSOR(lt_tensor, at::lt)
FB_CMP_TENSOR(ge_tensor, at::ge)
FB_CMP_TENSOR(le_tensor, at::le)
FB_CMP_TENSOR(eq_tensor, at::eq)
FB_CMP_TENSOR(ne_tensor, at::ne)
FB_UNARY(isnan, as_mask(at::isnan(x), x))
FB_UNARY(isinf, as_mask(at::isinf(x), x))
FB_UNARY(logical_not, as_mask(at::logical_not(x), x))
FB_UNARY(any, as_mask(x.to(at::kBool).any(), x))
FB_UNARY(all, as_mask(x.to(at::kBool).all(), x))
FB_BINARY(logical_and, as_mask(at::logical_and(a, b), a))
FB_BINARY(logical_or, as_mask(at::logical_or(a, b), a))
FB_API char* flodl_where(Handle cond, Handle x, Handle y, Handle* result) {
  return guarded([&] { *result = box(at::where(ref(cond).to(at::kBool), ref(x), ref(y))); });
}
FB_API char* flodl_masked_fill(Handle t, Handle mask, double value, Handle* result) {
  return guarded([&] { *result = box(ref(t).masked_fill(ref(mask).to(at::kBool), value)); });
}

// ---- shape -----------------------------------------------------------------------------------------------------
FB_API char* flodl_reshape(Handle t, int64_t* shape, int ndim, Handle* result) {
  return guarded([&] { *result = box(ref(t).reshape(dims(shape, ndim))); });
}
FB_API char* flodl_expand(Handle t, int64_t* shape, int ndim, Handle* result) {
  return guarded([&] { *result = box(ref(t).expand(dims(shape, ndim)).contiguous()); });
}
FB_API char* flodl_transpose(Handle t, int d0, int d1, Handle* result) { return guarded([&] { *result = box(ref(t).transpose(d0, d1)); }); }
FB_API char* flodl_permute(Handle t, int64_t* ds, int n, Handle* result) { return guarded([&] { *result = box(ref(t).permute(dims(ds, n))); }); }
FB_API char* flodl_select(Handle t, int dim, int64_t index, Handle* result) { return guarded([&] { *result = box(ref(t).select(dim, index)); }); }
FB_API char* flodl_narrow(Handle t, int dim, int64_t start, int64_t length, Handle* result) {
  return guarded([&] { *result = box(ref(t).narrow(dim, start, length)); });
}
FB_API char* flodl_squeeze(Handle t, int dim, Handle* result) { return guarded([&] { *result = box(ref(t).squeeze(dim).contiguous()); }); }
FB_API char* flodl_unsqueeze(Handle t, int dim, Handle* result) { return guarded([&] { *result = box(ref(t).unsqueeze(dim)); }); }
FB_API char* flodl_flatten(Handle t, int start, int end, Handle* result) { return guarded([&] { *result = box(ref(t).flatten(start, end)); }); }
FB_API char* flodl_diagonal(Handle t, int64_t offset, int d1, int d2, Handle* result) {
  return guarded([&] { *result = box(ref(t).diagonal(offset, d1, d2)); });
}
FB_API char* flodl_movedim(Handle t, int64_t src, int64_t dst, Handle* result) { return guarded([&] { *result = box(ref(t).movedim(src, dst)); }); }
FB_API char* flodl_tile(Handle t, int64_t* reps, int n, Handle* result) { return guarded([&] { *result = box(ref(t).tile(dims(reps, n))); }); }
FB_API char* flodl_repeat(Handle t, int64_t* reps, int n, Handle* result) { return guarded([&] { *result = box(ref(t).repeat(dims(reps, n))); }); }
FB_API char* flodl_flip(Handle t, int64_t* ds, int n, Handle* result) { return guarded([&] { *result = box(ref(t).flip(dims(ds, n))); }); }
FB_API char* flodl_roll(Handle t, int64_t shift, int dim, Handle* result) { return guarded([&] { *result = box(ref(t).roll(shift, dim)); }); }
FB_API char* flodl_pad(Handle t, int64_t* padding, int n, double value, Handle* result) {
  return guarded([&] { *result = box(at::constant_pad_nd(ref(t), dims(padding, n), value)); });
}
FB_API char* flodl_pad_mode(Handle t, int64_t* padding, int n, int mode, double value, Handle* result) {
  return guarded([&] {
    static const char* kModes[4] = {"constant", "reflect", "replicate", "circular"};
    TORCH_CHECK(mode >= 0 && mode < 4, "pad_mode: unknown mode ", mode);
    *result = box(mode == 0 ? at::constant_pad_nd(ref(t), dims(padding, n), value) : at::pad(ref(t), dims(padding, n), kModes[mode]));
  });
}
FB_API char* flodl_chunk(Handle t, int chunks, int dim, Handle** results, int* count) {
  return guarded([&] { give_list(ref(t).chunk(chunks, dim), results, count); });
}
FB_API char* flodl_split(Handle t, int64_t split_size, int dim, Handle** results, int* count) {
  return guarded([&] { give_list(ref(t).split(split_size, dim), results, count); });
}
FB_API char* flodl_unbind(Handle t, int dim, Handle** results, int* count) {
  return guarded([&] { give_list(ref(t).unbind(dim), results, count); });
}
FB_API char* flodl_meshgrid(Handle* tensors, int count, Handle** results, int* result_count) {
  return guarded([&] { give_list(at::meshgrid(list_of(tensors, count), "ij"), results, result_count); });
}
FB_API char* flodl_cat2(Handle a, Handle b, int dim, Handle* result) { return guarded([&] { *result = box(at::cat({ref(a), ref(b)}, dim)); }); }
FB_API char* flodl_cat(Handle* tensors, int count, int dim, Handle* result) {
  return guarded([&] { *result = box(at::cat(list_of(tensors, count), dim)); });
}
FB_API char* flodl_stack(Handle* tensors, int count, int dim, Handle* result) {
  return guarded([&] { *result = box(at::stack(list_of(tensors, count), dim)); });
}

// ---- indexing / scatter ------------------------------------------------------------------------------------------
FB_API char* flodl_gather(Handle t, int dim, Handle index, Handle* result) { return guarded([&] { *result = box(ref(t).gather(dim, ref(index))); }); }
FB_API char* flodl_scatter(Handle t, int dim, Handle index, Handle src, Handle* result) {
  return guarded([&] { *result = box(ref(t).scatter(dim, ref(index), ref(src))); });
}
FB_API char* flodl_scatter_add(Handle t, int dim, Handle index, Handle src, Handle* result) {
  return guarded([&] { *result = box(ref(t).scatter_add(dim, ref(index), ref(src))); });
}
FB_API char* flodl_index_select(Handle t, int dim, Handle index, Handle* result) {
  return guarded([&] { *result = box(ref(t).index_select(dim, ref(index))); });
}
FB_API char* flodl_index_add(Handle t, int dim, Handle index, Handle src, Handle* result) {
  return guarded([&] { *result = box(ref(t).index_add(dim, ref(index), ref(src))); });
}
FB_API char* flodl_select_scatter(Handle input, Handle src, int dim, int64_t index, Handle* result) {
  return guarded([&] { *result = box(at::select_scatter(ref(input), ref(src), dim, index)); });
}
FB_API char* flodl_narrow_scatter(Handle input, Handle src, int dim, int64_t start, Handle* result) {
  return guarded([&] { *result = box(at::slice_scatter(ref(input), ref(src), dim, start, start + ref(src).size(dim))); });
}

// ---- device / dtype -----------------------------------------------------------------------------------------------
FB_API char* flodl_to_device(Handle t, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(ref(t).to(device_of(dev_type, dev_index))); });
}
FB_API char* flodl_to_device_async(Handle t, int dev_type, int dev_index, Handle* result) {
  return guarded([&] { *result = box(ref(t).to(device_of(dev_type, dev_index), /*non_blocking=*/true)); });
}
FB_API char* flodl_to_dtype(Handle t, int dtype, Handle* result) { return guarded([&] { *result = box(ref(t).to(dtype_of(dtype))); }); }
FB_API char* flodl_pin_memory(Handle t, Handle* result) { return guarded([&] { *result = box(ref(t).pin_memory()); }); }
FB_API int flodl_is_pinned(Handle t) { return ref(t).is_pinned() ? 1 : 0; }
FB_API char* flodl_to_channels_last(Handle t, Handle* result) {
  return guarded([&] { *result = box(ref(t).contiguous(at::MemoryFormat::ChannelsLast)); });
}
FB_API int flodl_is_channels_last(Handle t) { return ref(t).dim() == 4 && ref(t).is_contiguous(at::MemoryFormat::ChannelsLast) ? 1 : 0; }
FB_API char* flodl_copy_(Handle dst, Handle src, int non_blocking) {
  return guarded([&] { ref(dst).copy_(ref(src), non_blocking != 0); });
}
