// Shared plumbing of the drop-in C ABI (`libflodl_b200_shim.so`).
//
// The library exports the `flodl_*` functions a host written against the reference's C interface
// (flodl-sys/shim.h) links to: same names, same argument lists, same conventions -
//   * a tensor handle is an opaque pointer the library allocates and `flodl_free_tensor` releases;
//   * a fallible function returns NULL on success or a malloc'd message the caller frees with
//     `flodl_free_string`; arrays handed back (`flodl_chunk`, `flodl_meshgrid`, ...) are malloc'd too;
//   * dtype tags 3/4/5/6/7/15 = i32/i64/f16/f32/f64/bf16, device tags 0/1 = CPU/CUDA.
// Most functions forward to ATen. The ones on a transformer / ResNet training step's hot path
// (linear, layer norm, GELU, attention, cross-entropy, dropout) run this
// library's sm_100a kernels when their inputs are on a CUDA device and autocast selects bf16
// (csrc/abi/abi_native.cpp), as C++ autograd functions, so a host that drives training through this
// ABI gets them without changing a line.
#pragma once

#include <torch/torch.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace fbabi {

using at::Tensor;
using Handle = void*;

inline char* fail(const std::string& msg) {
  char* out = static_cast<char*>(std::malloc(msg.size() + 1));
  if (out) std::memcpy(out, msg.c_str(), msg.size() + 1);
  return out;
}

// Runs `body`; any C++ exception becomes the returned message.
template <typename F>
inline char* guarded(F&& body) {
  try {
    body();
    return nullptr;
  } catch (const std::exception& e) {
    return fail(e.what());
  } catch (...) {
    return fail("unknown C++ exception");
  }
}

inline Tensor& ref(Handle h) { return *static_cast<Tensor*>(h); }
inline Handle box(Tensor t) { return new Tensor(std::move(t)); }
inline Tensor opt(Handle h) { return h ? ref(h) : Tensor(); }
inline c10::optional<Tensor> optional_of(Handle h) { return h ? c10::optional<Tensor>(ref(h)) : c10::nullopt; }

inline at::ScalarType dtype_of(int tag) {
  switch (tag) {
    case 3: return at::kInt;
    case 4: return at::kLong;
    case 5: return at::kHalf;
    case 7: return at::kDouble;
    case 15: return at::kBFloat16;
    default: return at::kFloat;
  }
}
inline int tag_of(at::ScalarType t) {
  switch (t) {
    case at::kInt: return 3;
    case at::kLong: return 4;
    case at::kHalf: return 5;
    case at::kDouble: return 7;
    case at::kBFloat16: return 15;
    default: return 6;
  }
}
inline at::Device device_of(int type, int index) {
  return type == 1 ? at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(index)) : at::Device(at::kCPU);
}
inline at::TensorOptions options_of(int dtype, int dev_type, int dev_index) {
  return at::TensorOptions().dtype(dtype_of(dtype)).device(device_of(dev_type, dev_index));
}
inline at::IntArrayRef dims(const int64_t* p, int n) { return at::IntArrayRef(p, static_cast<size_t>(n)); }
inline std::vector<Tensor> list_of(Handle* hs, int n) {
  std::vector<Tensor> out;
  out.reserve(static_cast<size_t>(n));
  for (int i = 0; i < n; ++i) out.push_back(ref(hs[i]));
  return out;
}
// malloc'd array of fresh handles (the caller frees the array with flodl_free_string)
inline void give_list(const std::vector<Tensor>& ts, Handle** out, int* count) {
  *count = static_cast<int>(ts.size());
  *out = static_cast<Handle*>(std::malloc(sizeof(Handle) * (ts.empty() ? 1 : ts.size())));
  for (size_t i = 0; i < ts.size(); ++i) (*out)[i] = box(ts[i]);
}
// comparison / predicate results: 0.0 / 1.0 in the input's floating dtype (fp32 for integer inputs)
inline Tensor as_mask(const Tensor& b, const Tensor& like) {
  return b.to(like.is_floating_point() ? like.scalar_type() : at::kFloat);
}

// ---- hot ops with a native sm_100a path (abi_native.cpp) -------------------------------------------
// Each returns true and fills the outputs when it took the native path, false to let the caller use ATen.
bool native_linear(const Tensor& x, const Tensor& w, const Tensor& b, Tensor* out);
bool native_layer_norm(const Tensor& x, const Tensor& w, const Tensor& b, int64_t size, double eps, Tensor* out, Tensor* mean,
                       Tensor* rstd);
bool native_gelu(const Tensor& x, bool tanh_approx, Tensor* out);
bool native_sdpa(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, double p, bool causal, double scale, Tensor* out);
bool native_cross_entropy(const Tensor& logits, const Tensor& target, int64_t reduction, int64_t ignore_index, double smoothing,
                          Tensor* out);
bool native_dropout(const Tensor& x, double p, bool training, Tensor* out);
// Tells the native paths that parameters changed under them (invalidates the cached bf16 weight copies).
void note_mutation();
// How many calls took a native path so far (for tests and for `flodl_b200_native_calls`).
extern "C" long long flodl_b200_native_calls(void);

}  // namespace fbabi
