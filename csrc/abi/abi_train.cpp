// Drop-in C ABI, part 3: autograd plumbing, autocast, in-place ops, optimizer steps, multi-tensor
// helpers, gradient clipping, device queries, CUDA graphs / events / streams.
#include "abi_common.hpp"

#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <ATen/cuda/CUDAGraph.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <malloc.h>
#include <torch/csrc/autograd/functions/accumulate_grad.h>

#include <cmath>
#include <deque>
#include <unordered_set>

#include "flodl_b200.h"

using namespace fbabi;

#define FB_API extern "C" __attribute__((visibility("default")))

// ---- autograd ------------------------------------------------------------------------------------------------
FB_API char* flodl_set_requires_grad(Handle t, int requires_grad, Handle* result) {
  return guarded([&] { *result = box(ref(t).set_requires_grad(requires_grad != 0)); });
}
FB_API int flodl_requires_grad(Handle t) { return ref(t).requires_grad() ? 1 : 0; }
FB_API int flodl_is_leaf(Handle t) { return ref(t).is_leaf() ? 1 : 0; }
FB_API char* flodl_backward(Handle t) { return guarded([&] { ref(t).backward(); }); }
FB_API char* flodl_grad(Handle t, Handle* result) {
  return guarded([&] {
    const Tensor& g = ref(t).grad();
    *result = g.defined() ? box(g) : nullptr;
  });
}
FB_API char* flodl_set_grad(Handle t, Handle grad) { return guarded([&] { ref(t).mutable_grad() = ref(grad); }); }
FB_API char* flodl_zero_grad(Handle t) {
  return guarded([&] {
    if (ref(t).grad().defined()) ref(t).mutable_grad().zero_();
  });
}
FB_API void flodl_zero_grad_set_to_none(Handle t) { ref(t).mutable_grad() = Tensor(); }
FB_API char* flodl_detach(Handle t, Handle* result) { return guarded([&] { *result = box(ref(t).detach()); }); }
FB_API char* flodl_detach_(Handle t) { return guarded([&] { ref(t).detach_(); }); }
// Keeps the gradient-accumulator node of a leaf alive (and with it the stream it was created on).
FB_API char* flodl_ensure_grad_accumulator(Handle t, void** handle_out) {
  return guarded([&] {
    *handle_out = nullptr;
    const Tensor& x = ref(t);
    if (x.is_leaf() && x.requires_grad())
      *handle_out = new std::shared_ptr<torch::autograd::Node>(torch::autograd::impl::grad_accumulator(x));
  });
}
FB_API void flodl_grad_accumulator_delete(void* handle) { delete static_cast<std::shared_ptr<torch::autograd::Node>*>(handle); }
FB_API int64_t flodl_autograd_node_count(Handle t) {
  auto root = ref(t).grad_fn();
  if (!root) return 0;
  std::unordered_set<torch::autograd::Node*> seen{root.get()};
  std::deque<torch::autograd::Node*> todo{root.get()};
  while (!todo.empty()) {
    auto* n = todo.front();
    todo.pop_front();
    for (const auto& e : n->next_edges())
      if (e.function && seen.insert(e.function.get()).second) todo.push_back(e.function.get());
  }
  return static_cast<int64_t>(seen.size());
}
FB_API void* flodl_no_grad_guard_new(void) { return new at::NoGradGuard(); }
FB_API void flodl_no_grad_guard_delete(void* g) { delete static_cast<at::NoGradGuard*>(g); }
FB_API int flodl_is_grad_enabled(void) { return at::GradMode::is_enabled() ? 1 : 0; }

// ---- autocast ------------------------------------------------------------------------------------------------
namespace {
struct AutocastScope {
  at::DeviceType dev;
  bool was_enabled;
  at::ScalarType was_dtype;
  AutocastScope(at::DeviceType d, at::ScalarType t) : dev(d), was_enabled(at::autocast::is_autocast_enabled(d)), was_dtype(at::autocast::get_autocast_dtype(d)) {
    at::autocast::set_autocast_enabled(d, true);
    at::autocast::set_autocast_dtype(d, t);
    at::autocast::increment_nesting();
  }
  ~AutocastScope() {
    if (at::autocast::decrement_nesting() == 0) at::autocast::clear_cache();
    at::autocast::set_autocast_enabled(dev, was_enabled);
    at::autocast::set_autocast_dtype(dev, was_dtype);
  }
};
at::DeviceType dev_type_of(int tag) { return tag == 1 ? at::kCUDA : at::kCPU; }
}  // namespace
FB_API void* flodl_autocast_guard_new(int device_type, int dtype) { return new AutocastScope(dev_type_of(device_type), dtype_of(dtype)); }
FB_API void flodl_autocast_guard_delete(void* g) { delete static_cast<AutocastScope*>(g); }
FB_API int flodl_is_autocast_enabled(int device_type) { return at::autocast::is_autocast_enabled(dev_type_of(device_type)) ? 1 : 0; }

// ---- in-place ------------------------------------------------------------------------------------------------
FB_API char* flodl_add_(Handle t, Handle o) { return guarded([&] { ref(t).add_(ref(o)); }); }
FB_API char* flodl_sub_(Handle t, Handle o) { return guarded([&] { ref(t).sub_(ref(o)); }); }
FB_API char* flodl_mul_(Handle t, Handle o) { return guarded([&] { ref(t).mul_(ref(o)); }); }
FB_API char* flodl_div_(Handle t, Handle o) { return guarded([&] { ref(t).div_(ref(o)); }); }
FB_API char* flodl_mul_scalar_(Handle t, double s) { return guarded([&] { ref(t).mul_(s); }); }
FB_API char* flodl_add_scalar_(Handle t, double s) { return guarded([&] { ref(t).add_(s); }); }
FB_API char* flodl_div_scalar_(Handle t, double s) { return guarded([&] { ref(t).div_(s); }); }
FB_API char* flodl_fill_(Handle t, double v) { return guarded([&] { ref(t).fill_(v); }); }
FB_API char* flodl_zero_(Handle t) { return guarded([&] { ref(t).zero_(); }); }

// ---- optimizer steps -------------------------------------------------------------------------------------------
namespace {
// One parameter, AdamW form: p *= 1 - lr*wd; m, v updated; p -= (lr / bc1) * m / (sqrt(v / bc2) + eps).
// fp32 contiguous CUDA tensors take this library's single fused kernel; anything else the ATen op chain.
void adam_one(const Tensor& param, const Tensor& grad, Tensor& m, Tensor& v, double lr, double b1, double b2, double eps, double wd, int64_t step) {
  Tensor p = param.detach();
  const double bc1 = 1.0 - std::pow(b1, static_cast<double>(step)), bc2 = 1.0 - std::pow(b2, static_cast<double>(step));
  const bool fused = p.is_cuda() && p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat &&
                     (grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16) && p.is_contiguous() && grad.is_contiguous() &&
                     m.is_contiguous() && v.is_contiguous() && p.numel() % 4 == 0 && (reinterpret_cast<uintptr_t>(p.data_ptr()) & 15) == 0;
  if (fused) {
    c10::cuda::CUDAGuard guard(p.device());
    const float hyper[4] = {static_cast<float>(lr), static_cast<float>(bc1), static_cast<float>(bc2), static_cast<float>(wd)};
    const int rc = fb_adam_step_host(p.data_ptr<float>(), grad.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), p.numel(), hyper,
                                     static_cast<float>(b1), static_cast<float>(b2), static_cast<float>(eps), grad.scalar_type() == at::kBFloat16,
                                     at::cuda::getCurrentCUDAStream(p.get_device()).stream());
    TORCH_CHECK(rc == 0, "fb_adam_step_host failed with code ", rc);
    param.unsafeGetTensorImpl()->bump_version();  // the kernel wrote through the raw pointer
    note_mutation();
    return;
  }
  if (wd > 0.0) p.mul_(1.0 - lr * wd);
  m.mul_(b1).add_(grad, 1.0 - b1);
  v.mul_(b2).addcmul_(grad, grad, 1.0 - b2);
  p.addcdiv_(m, (v / bc2).sqrt_().add_(eps), -(lr / bc1));
}
}  // namespace
FB_API char* flodl_adam_step(Handle param, Handle grad, Handle m, Handle v, double lr, double beta1, double beta2, double eps, double weight_decay,
                             int64_t step) {
  return guarded([&] {
    at::NoGradGuard ng;
    adam_one(ref(param), ref(grad), ref(m), ref(v), lr, beta1, beta2, eps, weight_decay, step);
  });
}
FB_API char* flodl_adam_step_batched(Handle* params, Handle* grads, Handle* ms, Handle* vs, double* lrs, int count, double beta1, double beta2,
                                     double eps, double weight_decay, int64_t step) {
  return guarded([&] {
    at::NoGradGuard ng;
    for (int i = 0; i < count; ++i) adam_one(ref(params[i]), ref(grads[i]), ref(ms[i]), ref(vs[i]), lrs[i], beta1, beta2, eps, weight_decay, step);
  });
}
namespace {
char* fused_adam_lists(bool decoupled, Handle* params, Handle* grads, Handle* ms, Handle* vs, int count, double lr, double b1, double b2, double eps,
                       double wd, int64_t step, Handle grad_scale, Handle found_inf) {
  return guarded([&] {
    if (count <= 0) return;
    at::NoGradGuard ng;
    auto P = list_of(params, count), G = list_of(grads, count), M = list_of(ms, count), V = list_of(vs, count);
    std::vector<Tensor> max_sq, steps;
    // the multi-tensor kernel reads the step count from one fp32 scalar per parameter and does not advance it
    const Tensor s = at::full({}, static_cast<double>(step), at::TensorOptions().dtype(at::kFloat).device(P[0].device()));
    steps.assign(static_cast<size_t>(count), s);
    if (decoupled) at::_fused_adamw_(P, G, M, V, max_sq, steps, lr, b1, b2, wd, eps, false, false, optional_of(grad_scale), optional_of(found_inf));
    else at::_fused_adam_(P, G, M, V, max_sq, steps, lr, b1, b2, wd, eps, false, false, optional_of(grad_scale), optional_of(found_inf));
    note_mutation();
  });
}
}  // namespace
FB_API char* flodl_fused_adam_(Handle* params, Handle* grads, Handle* ms, Handle* vs, int count, double lr, double beta1, double beta2, double eps,
                               double weight_decay, int64_t step, Handle grad_scale, Handle found_inf) {
  return fused_adam_lists(false, params, grads, ms, vs, count, lr, beta1, beta2, eps, weight_decay, step, grad_scale, found_inf);
}
FB_API char* flodl_fused_adamw_(Handle* params, Handle* grads, Handle* ms, Handle* vs, int count, double lr, double beta1, double beta2, double eps,
                                double weight_decay, int64_t step, Handle grad_scale, Handle found_inf) {
  return fused_adam_lists(true, params, grads, ms, vs, count, lr, beta1, beta2, eps, weight_decay, step, grad_scale, found_inf);
}
// Global L2 norm of the gradients of `params`; gradients are scaled in place by max_norm / (norm + 1e-6) when the
// norm exceeds max_norm. The norm before scaling goes to *total_norm_out.
FB_API char* flodl_clip_grad_norm(Handle* params, int count, double max_norm, double* total_norm_out) {
  return guarded([&] {
    std::vector<Tensor> grads;
    for (int i = 0; i < count; ++i)
      if (ref(params[i]).grad().defined()) grads.push_back(ref(params[i]).mutable_grad());
    *total_norm_out = 0.0;
    if (grads.empty()) return;
    const double total = at::stack(at::_foreach_norm(grads, 2.0)).norm().item<double>();
    *total_norm_out = total;
    if (total > max_norm) at::_foreach_mul_(grads, max_norm / (total + 1e-6));
  });
}

// ---- multi-tensor helpers ----------------------------------------------------------------------------------------
FB_API char* flodl_foreach_add_scalar_(Handle* ts, int n, double s) {
  return guarded([&] { if (n > 0) at::_foreach_add_(list_of(ts, n), s); });
}
FB_API char* flodl_foreach_mul_scalar_(Handle* ts, int n, double s) {
  return guarded([&] { if (n > 0) at::_foreach_mul_(list_of(ts, n), s); });
}
FB_API char* flodl_foreach_zero_(Handle* ts, int n) {
  return guarded([&] { if (n > 0) at::_foreach_zero_(list_of(ts, n)); });
}
FB_API char* flodl_foreach_add_list_(Handle* a, Handle* b, int n, double alpha) {
  return guarded([&] { if (n > 0) at::_foreach_add_(list_of(a, n), list_of(b, n), alpha); });
}
FB_API char* flodl_foreach_norm(Handle* ts, int n, double ord, Handle* results) {
  return guarded([&] {
    if (n <= 0) return;
    auto norms = at::_foreach_norm(list_of(ts, n), ord);
    for (int i = 0; i < n; ++i) results[i] = box(norms[static_cast<size_t>(i)]);
  });
}
FB_API char* flodl_foreach_lerp_scalar_(Handle* a, Handle* b, int n, double weight) {
  return guarded([&] { if (n > 0) at::_foreach_lerp_(list_of(a, n), list_of(b, n), weight); });
}
FB_API char* flodl_foreach_sqrt_(Handle* ts, int n) {
  return guarded([&] { if (n > 0) at::_foreach_sqrt_(list_of(ts, n)); });
}

// ---- device queries ------------------------------------------------------------------------------------------------
FB_API int flodl_cuda_is_available(void) { return torch::cuda::is_available() ? 1 : 0; }
FB_API int flodl_cuda_device_count(void) { return static_cast<int>(torch::cuda::device_count()); }
FB_API int flodl_force_cuda_link(void) { return torch::cuda::is_available() ? static_cast<int>(at::cuda::device_count()) : 0; }
FB_API void flodl_set_cudnn_benchmark(int enable) { at::globalContext().setBenchmarkCuDNN(enable != 0); }
FB_API void flodl_manual_seed(uint64_t seed) { torch::manual_seed(seed); }
FB_API void flodl_cuda_manual_seed_all(uint64_t seed) {
  if (torch::cuda::is_available()) torch::cuda::manual_seed_all(seed);
}
FB_API void flodl_set_current_device(int index) { c10::cuda::set_device(static_cast<c10::DeviceIndex>(index)); }
FB_API int flodl_get_current_device(void) { return static_cast<int>(c10::cuda::current_device()); }
FB_API void flodl_cuda_synchronize(int index) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(index));
  c10::cuda::device_synchronize();
}
FB_API char* flodl_cuda_mem_info(int index, uint64_t* used, uint64_t* total) {
  return guarded([&] {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(index));
    size_t f = 0, t = 0;
    TORCH_CHECK(cudaMemGetInfo(&f, &t) == cudaSuccess, "cudaMemGetInfo failed");
    *used = t - f;
    *total = t;
  });
}
namespace {
uint64_t allocator_stat(int index, int which) {   // 0 allocated now, 1 active now, 2 peak active, 3 peak reserved
  auto st = c10::cuda::CUDACachingAllocator::getDeviceStats(static_cast<c10::DeviceIndex>(index));
  const auto agg = static_cast<size_t>(c10::CachingAllocator::StatType::AGGREGATE);
  switch (which) {
    case 0: return static_cast<uint64_t>(st.allocated_bytes[agg].current);
    case 1: return static_cast<uint64_t>(st.active_bytes[agg].current);
    case 2: return static_cast<uint64_t>(st.active_bytes[agg].peak);
    default: return static_cast<uint64_t>(st.reserved_bytes[agg].peak);
  }
}
}  // namespace
FB_API char* flodl_cuda_alloc_bytes(int index, uint64_t* out) { return guarded([&] { *out = allocator_stat(index, 0); }); }
FB_API char* flodl_cuda_active_bytes(int index, uint64_t* out) { return guarded([&] { *out = allocator_stat(index, 1); }); }
FB_API char* flodl_cuda_peak_active_bytes(int index, uint64_t* out) { return guarded([&] { *out = allocator_stat(index, 2); }); }
FB_API char* flodl_cuda_peak_reserved_bytes(int index, uint64_t* out) { return guarded([&] { *out = allocator_stat(index, 3); }); }
FB_API void flodl_cuda_reset_peak_stats(int index) { c10::cuda::CUDACachingAllocator::resetPeakStats(static_cast<c10::DeviceIndex>(index)); }
FB_API void flodl_cuda_empty_cache(void) { c10::cuda::CUDACachingAllocator::emptyCache(); }
FB_API char* flodl_cuda_device_name(int index, char* buf, int buf_len) {
  return guarded([&] {
    cudaDeviceProp prop;
    TORCH_CHECK(cudaGetDeviceProperties(&prop, index) == cudaSuccess, "cudaGetDeviceProperties failed");
    std::strncpy(buf, prop.name, static_cast<size_t>(buf_len > 0 ? buf_len - 1 : 0));
    if (buf_len > 0) buf[buf_len - 1] = '\0';
  });
}
FB_API char* flodl_cuda_compute_capability(int index, int* major, int* minor) {
  return guarded([&] {
    cudaDeviceProp prop;
    TORCH_CHECK(cudaGetDeviceProperties(&prop, index) == cudaSuccess, "cudaGetDeviceProperties failed");
    *major = prop.major;
    *minor = prop.minor;
  });
}
// GPU utilisation in percent through NVML, opened lazily and read-only; -1 when NVML is not there.
FB_API int flodl_cuda_utilization(int index) {
  struct Util { unsigned gpu, memory; };
  using InitFn = int (*)();
  using HandleFn = int (*)(unsigned, void**);
  using RatesFn = int (*)(void*, Util*);
  static void* lib = dlopen("libnvidia-ml.so.1", RTLD_LAZY);
  if (!lib) return -1;
  static auto init = reinterpret_cast<InitFn>(dlsym(lib, "nvmlInit_v2"));
  static auto by_index = reinterpret_cast<HandleFn>(dlsym(lib, "nvmlDeviceGetHandleByIndex_v2"));
  static auto rates = reinterpret_cast<RatesFn>(dlsym(lib, "nvmlDeviceGetUtilizationRates"));
  static bool ready = init && by_index && rates && init() == 0;
  if (!ready) return -1;
  void* dev = nullptr;
  Util u{};
  if (by_index(static_cast<unsigned>(index), &dev) != 0 || rates(dev, &u) != 0) return -1;
  return static_cast<int>(u.gpu);
}
FB_API int flodl_malloc_trim(void) { return malloc_trim(0); }

// ---- CUDA graphs ------------------------------------------------------------------------------------------------------
namespace {
// A graph plus the side stream its capture runs on; the current stream is put back when capture ends or is abandoned.
class GraphBox {
 public:
  void begin(uint64_t pool_hi, uint64_t pool_lo, int mode) {
    auto side = at::cuda::getStreamFromPool(false);
    at::cuda::CUDAEvent fence;
    fence.record(at::cuda::getCurrentCUDAStream());
    fence.block(side);                               // work already queued runs before the capture starts
    stream_ = side;
    at::cuda::setCurrentCUDAStream(side);
    open_ = true;
    try {
      graph_.capture_begin({pool_hi, pool_lo}, static_cast<cudaStreamCaptureMode>(mode));
    } catch (...) {
      leave();
      throw;
    }
  }
  void end() {
    graph_.capture_end();
    if (stream_) {
      at::cuda::CUDAEvent fence;
      fence.record(*stream_);
      fence.block(at::cuda::getDefaultCUDAStream());
    }
    leave();
  }
  void replay() { graph_.replay(); }
  void reset() { graph_.reset(); }
  at::cuda::MempoolId_t pool() { return graph_.pool(); }
  ~GraphBox() {
    if (open_ && stream_) {                          // abandoned in mid-capture: end it so the stream is usable again
      cudaStreamCaptureStatus st;
      if (cudaStreamIsCapturing(stream_->stream(), &st) == cudaSuccess && st == cudaStreamCaptureStatusActive) {
        cudaGraph_t g = nullptr;
        cudaStreamEndCapture(stream_->stream(), &g);
        if (g) cudaGraphDestroy(g);
      }
      leave();
    }
  }

 private:
  void leave() {
    open_ = false;
    at::cuda::setCurrentCUDAStream(at::cuda::getDefaultCUDAStream());
  }
  at::cuda::CUDAGraph graph_;
  c10::optional<at::cuda::CUDAStream> stream_;
  bool open_ = false;
};
}  // namespace
FB_API char* flodl_cuda_graph_new(void** out) { return guarded([&] { *out = new GraphBox(); }); }
FB_API char* flodl_cuda_graph_capture_begin(void* g, uint64_t pool_hi, uint64_t pool_lo, int mode) {
  return guarded([&] { static_cast<GraphBox*>(g)->begin(pool_hi, pool_lo, mode); });
}
FB_API char* flodl_cuda_graph_capture_end(void* g) { return guarded([&] { static_cast<GraphBox*>(g)->end(); }); }
FB_API char* flodl_cuda_graph_replay(void* g) { return guarded([&] { static_cast<GraphBox*>(g)->replay(); }); }
FB_API char* flodl_cuda_graph_reset(void* g) { return guarded([&] { static_cast<GraphBox*>(g)->reset(); }); }
FB_API void flodl_cuda_graph_delete(void* g) { delete static_cast<GraphBox*>(g); }
FB_API void flodl_cuda_graph_pool(void* g, uint64_t* hi, uint64_t* lo) {
  auto p = static_cast<GraphBox*>(g)->pool();
  *hi = p.first;
  *lo = p.second;
}
FB_API void flodl_cuda_graph_pool_handle(uint64_t* hi, uint64_t* lo) {
  auto p = at::cuda::graph_pool_handle();
  *hi = p.first;
  *lo = p.second;
}

// ---- CUDA events / streams -----------------------------------------------------------------------------------------------
FB_API char* flodl_cuda_event_new(int flags, void** out) {
  return guarded([&] { *out = new at::cuda::CUDAEvent(flags == 1 ? cudaEventDisableTiming : cudaEventDefault); });
}
FB_API char* flodl_cuda_event_record(void* e) { return guarded([&] { static_cast<at::cuda::CUDAEvent*>(e)->record(at::cuda::getCurrentCUDAStream()); }); }
FB_API char* flodl_cuda_event_record_on_stream(void* e, void* s) {
  return guarded([&] { static_cast<at::cuda::CUDAEvent*>(e)->record(*static_cast<at::cuda::CUDAStream*>(s)); });
}
FB_API char* flodl_cuda_event_synchronize(void* e) { return guarded([&] { static_cast<at::cuda::CUDAEvent*>(e)->synchronize(); }); }
FB_API char* flodl_cuda_event_elapsed_time(void* a, void* b, float* ms) {
  return guarded([&] { *ms = static_cast<at::cuda::CUDAEvent*>(a)->elapsed_time(*static_cast<at::cuda::CUDAEvent*>(b)); });
}
FB_API int flodl_cuda_event_query(void* e) { return static_cast<at::cuda::CUDAEvent*>(e)->query() ? 1 : 0; }
FB_API void flodl_cuda_event_delete(void* e) { delete static_cast<at::cuda::CUDAEvent*>(e); }

FB_API char* flodl_cuda_stream_new(int index, int high_priority, void** out) {
  return guarded([&] { *out = new at::cuda::CUDAStream(at::cuda::getStreamFromPool(high_priority != 0, static_cast<c10::DeviceIndex>(index))); });
}
FB_API char* flodl_cuda_stream_synchronize(void* s) { return guarded([&] { static_cast<at::cuda::CUDAStream*>(s)->synchronize(); }); }
FB_API char* flodl_cuda_stream_wait_event(void* s, void* e) {
  return guarded([&] { static_cast<at::cuda::CUDAEvent*>(e)->block(*static_cast<at::cuda::CUDAStream*>(s)); });
}
FB_API int flodl_cuda_stream_query(void* s) { return static_cast<at::cuda::CUDAStream*>(s)->query() ? 1 : 0; }
FB_API void flodl_cuda_stream_set_current(void* s) { at::cuda::setCurrentCUDAStream(*static_cast<at::cuda::CUDAStream*>(s)); }
FB_API void* flodl_cuda_stream_get_current(int index) { return new at::cuda::CUDAStream(at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(index))); }
FB_API void flodl_cuda_stream_restore_default(int index) {
  at::cuda::setCurrentCUDAStream(at::cuda::getDefaultCUDAStream(static_cast<c10::DeviceIndex>(index)));
}
FB_API void flodl_cuda_stream_delete(void* s) { delete static_cast<at::cuda::CUDAStream*>(s); }
