// Symmetric (peer-mapped) memory and the collectives that run on it.
//
// One process drives one GPU. A SymmAlloc is a raw cudaMalloc block that is exported with CUDA IPC;
// the Python layer exchanges the 64-byte handles through torch.distributed's store and every rank
// maps every peer's block, which gives the pointer table the kernels in csrc/comm index by rank.
// A VmmAlloc is the same thing built on the virtual-memory-management API (file descriptors instead
// of IPC handles), which is what an NVLink-switch multicast object can be bound to (csrc/runtime/vmm.cpp).
// This is the counterpart of the reference's NCCL communicator objects
// (flodl-sys/ops_cuda.cpp:265-562, flodl/src/distributed/nccl.rs:56-571): `SymmComm` is what
// `NcclRankComm` is there, `abort()` is what `NcclAbortHandle::abort` is there (a host flag the
// device-side waits poll, instead of `ncclCommAbort`).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <cstring>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "fb_vmm.hpp"
#include "flodl_b200.h"

namespace {

using torch::Tensor;

void cuda_check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

void* cur_stream(int device) { return at::cuda::getCurrentCUDAStream(device).stream(); }

struct SymmAlloc {
  void* ptr = nullptr;
  size_t nbytes = 0;
  int device = 0;

  SymmAlloc(size_t bytes, int dev) : nbytes(bytes), device(dev) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(dev));
    cuda_check(cudaMalloc(&ptr, bytes), "cudaMalloc(symmetric)");
    cuda_check(cudaMemset(ptr, 0, bytes), "cudaMemset(symmetric)");
    cuda_check(cudaDeviceSynchronize(), "sync");
  }
  ~SymmAlloc() { release(); }
  void release() {
    if (ptr) {
      cudaFree(ptr);
      ptr = nullptr;
    }
  }
  py::bytes ipc_handle() const {
    cudaIpcMemHandle_t h;
    cuda_check(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
    return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
  }
  uint64_t address() const { return reinterpret_cast<uint64_t>(ptr); }
  // Non-owning view; the caller keeps this object alive for as long as the tensor is used.
  Tensor tensor(py::object dtype, int64_t byte_offset, int64_t numel) const {
    auto st = torch::python::detail::py_object_to_dtype(dtype);
    TORCH_CHECK(byte_offset >= 0 && static_cast<size_t>(byte_offset + numel * c10::elementSize(st)) <= nbytes,
                "view exceeds the allocation");
    auto opts = torch::TensorOptions().dtype(st).device(torch::kCUDA, device);
    return at::from_blob(static_cast<char*>(ptr) + byte_offset, {numel}, opts);
  }
};


// VMM-backed symmetric block with an optional multicast (NVLS) mapping; see fb_vmm.hpp.
struct VmmAlloc {
  fb::VmmBlock block;
  VmmAlloc(size_t bytes, int dev) : block(bytes, dev) {}
  uint64_t address() const { return block.address(); }
  size_t nbytes() const { return block.size(); }
  Tensor tensor(py::object dtype, int64_t byte_offset, int64_t numel) const {
    auto st = torch::python::detail::py_object_to_dtype(dtype);
    TORCH_CHECK(byte_offset >= 0 && static_cast<size_t>(byte_offset + numel * c10::elementSize(st)) <= block.size(),
                "view exceeds the allocation");
    auto opts = torch::TensorOptions().dtype(st).device(torch::kCUDA, block.device());
    return at::from_blob(reinterpret_cast<char*>(block.address()) + byte_offset, {numel}, opts);
  }
};

uint64_t open_ipc(const std::string& handle) {
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<uint64_t>(p);
}
void close_ipc(uint64_t p) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(p)); }

struct SymmComm {
  fb_symm_ctx ctx;
  int device;
  Tensor epochs, status_dev;
  int* abort_host = nullptr;  // mapped pinned words: [0] abort (host -> device), [1] status (device -> host)
  int* abort_dev = nullptr;

  SymmComm(int rank, int world, std::vector<uint64_t> data, std::vector<uint64_t> sig, int dev, int64_t timeout_ns)
      : device(dev) {
    TORCH_CHECK(world >= 1 && world <= FB_MAX_RANKS && (int)data.size() == world && (int)sig.size() == world);
    std::memset(&ctx, 0, sizeof(ctx));
    for (int i = 0; i < world; ++i) {
      ctx.data[i] = reinterpret_cast<void*>(data[i]);
      ctx.sig[i] = reinterpret_cast<void*>(sig[i]);
    }
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(dev));
    epochs = torch::zeros({FB_MAX_BLOCKS}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev));
    status_dev = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev));
    cuda_check(cudaHostAlloc(reinterpret_cast<void**>(&abort_host), 64 * sizeof(int), cudaHostAllocMapped), "cudaHostAlloc");
    std::memset(abort_host, 0, 64 * sizeof(int));
    cuda_check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&abort_dev), abort_host, 0), "cudaHostGetDevicePointer");
    ctx.epochs = epochs.data_ptr();
    ctx.status = abort_dev + 32;   // its own cache line; the host reads it without a device sync
    ctx.status_dev = status_dev.data_ptr();
    ctx.abort = abort_dev;
    ctx.timeout_ns = timeout_ns;
    ctx.rank = rank;
    ctx.world = world;
  }
  ~SymmComm() {
    if (abort_host) cudaFreeHost(abort_host);
  }
  // A second context over other payload buffers that shares nothing but rank/world (used for staging).
  void set_data(std::vector<uint64_t> data) {
    TORCH_CHECK((int)data.size() == ctx.world);
    for (int i = 0; i < ctx.world; ++i) ctx.data[i] = reinterpret_cast<void*>(data[i]);
  }
  void abort() { *abort_host = 1; }
  void clear_abort() { *abort_host = 0; }
  bool aborted() const { return *abort_host != 0; }
  // The status word is host-mapped: `poll_status` reads what has arrived so far without waiting for
  // the device, `read_status` first waits for the device to finish what it was given.
  int poll_status() const { return *reinterpret_cast<volatile int*>(abort_host + 32); }
  int read_status() {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    cudaDeviceSynchronize();
    return poll_status();
  }
  void clear_status() {
    *reinterpret_cast<volatile int*>(abort_host + 32) = 0;
    status_dev.zero_();
  }
  // Device-memory copy of the status word: what kernels on the hot path (the optimizers' skip check) read.
  uint64_t status_device_address() const { return reinterpret_cast<uint64_t>(status_dev.data_ptr()); }
  void set_mc(uint64_t addr) { ctx.mc = reinterpret_cast<void*>(addr); }
  bool has_mc() const { return ctx.mc != nullptr; }
  // After a wait gave up the per-block epochs of the ranks no longer agree: start again from zero
  // (every rank, between two host barriers, with the signal pad zeroed as well).
  void reset_epochs() { epochs.zero_(); }
  void set_timeout_ns(int64_t t) { ctx.timeout_ns = t; }

  static std::vector<float> wvec(const std::optional<std::vector<float>>& w, int world) {
    if (!w.has_value()) return {};
    TORCH_CHECK((int)w->size() == world, "weights must have one entry per rank");
    return *w;
  }
  void rc(int r, const char* what) {
    TORCH_CHECK(r >= 0, what, ": rejected arguments (code ", r, ")");
    TORCH_CHECK(r == 0, what, ": CUDA error ", cudaGetErrorString(static_cast<cudaError_t>(r)));
  }

  void allreduce(int64_t byte_off, int64_t n, bool is_bf16, std::optional<std::vector<float>> weights, int blocks) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    auto w = wvec(weights, ctx.world);
    rc(fb_allreduce(&ctx, byte_off, n, is_bf16, w.empty() ? nullptr : w.data(), blocks, cur_stream(device)), "fb_allreduce");
  }
  void allreduce_oneshot(int64_t byte_off, int64_t n, bool in_bf16, Tensor& out, std::optional<std::vector<float>> weights,
                         int blocks) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == n);
    TORCH_CHECK(out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16);
    auto w = wvec(weights, ctx.world);
    rc(fb_allreduce_oneshot(&ctx, byte_off, n, in_bf16, out.data_ptr(), out.scalar_type() == at::kBFloat16,
                            w.empty() ? nullptr : w.data(), blocks, cur_stream(device)),
       "fb_allreduce_oneshot");
  }
  // Returns fp32 [2] = {sum (post-pre)^2, sum post^2}.
  Tensor param_average(const SymmComm& staging, int64_t n, std::optional<std::vector<float>> weights, double alpha,
                       std::optional<Tensor> p16, int blocks) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    auto fopts = torch::dtype(torch::kFloat).device(torch::kCUDA, device);
    if (!avg_partial.defined()) {
      avg_partial = torch::zeros({2 * FB_MAX_BLOCKS}, fopts);
      avg_counter = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
      avg_out = torch::zeros({2}, fopts);
    }
    if (p16.has_value()) TORCH_CHECK(p16->scalar_type() == at::kBFloat16 && p16->is_contiguous() && p16->numel() == n);
    auto w = wvec(weights, ctx.world);
    rc(fb_param_average(&ctx, &staging.ctx, n, w.empty() ? nullptr : w.data(), (float)alpha,
                        p16.has_value() ? p16->data_ptr() : nullptr, avg_partial.data_ptr<float>(),
                        reinterpret_cast<unsigned int*>(avg_counter.data_ptr<int>()), avg_out.data_ptr<float>(), blocks,
                        cur_stream(device)),
       "fb_param_average");
    return avg_out;
  }
  void broadcast(int64_t byte_off, int64_t nbytes, int root, int blocks) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    rc(fb_broadcast(&ctx, byte_off, nbytes, root, blocks, cur_stream(device)), "fb_broadcast");
  }
  void barrier(int blocks) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    rc(fb_symm_barrier(&ctx, blocks, cur_stream(device)), "fb_symm_barrier");
  }

  Tensor avg_partial, avg_counter, avg_out;
};

}  // namespace

void bind_comm(py::module_& m) {
  py::class_<VmmAlloc, std::shared_ptr<VmmAlloc>>(m, "VmmAlloc")
      .def(py::init<size_t, int>(), py::arg("nbytes"), py::arg("device"))
      .def("address", &VmmAlloc::address)
      .def_property_readonly("nbytes", &VmmAlloc::nbytes)
      .def("tensor", &VmmAlloc::tensor, py::arg("dtype"), py::arg("byte_offset"), py::arg("numel"))
      .def("export_fd", [](VmmAlloc& a) { return a.block.export_fd(); })
      .def("import_peer", [](VmmAlloc& a, int fd) { return a.block.import_peer(fd); })
      .def("mc_create", [](VmmAlloc& a, int world) { return a.block.mc_create(world); })
      .def("mc_import", [](VmmAlloc& a, int fd) { a.block.mc_import(fd); })
      .def("mc_add_device", [](VmmAlloc& a) { a.block.mc_add_device(); })
      .def("mc_bind", [](VmmAlloc& a) { a.block.mc_bind(); })
      .def("mc_map", [](VmmAlloc& a) { return a.block.mc_map(); })
      .def("mc_address", [](VmmAlloc& a) { return a.block.mc_address(); })
      .def("release", [](VmmAlloc& a) { a.block.release(); });
  m.def("multicast_supported", [](int device) { return fb::VmmBlock::multicast_supported(device); });
  py::class_<SymmAlloc, std::shared_ptr<SymmAlloc>>(m, "SymmAlloc")
      .def(py::init<size_t, int>(), py::arg("nbytes"), py::arg("device"))
      .def("ipc_handle", &SymmAlloc::ipc_handle)
      .def("address", &SymmAlloc::address)
      .def("tensor", &SymmAlloc::tensor, py::arg("dtype"), py::arg("byte_offset"), py::arg("numel"))
      .def("release", &SymmAlloc::release)
      .def_readonly("nbytes", &SymmAlloc::nbytes);
  m.def("open_ipc", [](py::bytes h) { return open_ipc(std::string(h)); });
  m.def("close_ipc", &close_ipc);
  m.attr("SIGNAL_PAD_BYTES") = py::int_(FB_SIGNAL_PAD_BYTES);
  m.attr("MAX_RANKS") = py::int_(FB_MAX_RANKS);
  m.attr("MAX_BLOCKS") = py::int_(FB_MAX_BLOCKS);
  py::class_<SymmComm, std::shared_ptr<SymmComm>>(m, "SymmComm")
      .def(py::init<int, int, std::vector<uint64_t>, std::vector<uint64_t>, int, int64_t>(), py::arg("rank"), py::arg("world"),
           py::arg("data"), py::arg("sig"), py::arg("device"), py::arg("timeout_ns") = 0)
      .def("set_data", &SymmComm::set_data)
      .def("abort", &SymmComm::abort)
      .def("clear_abort", &SymmComm::clear_abort)
      .def("aborted", &SymmComm::aborted)
      .def("read_status", &SymmComm::read_status)
      .def("poll_status", &SymmComm::poll_status)
      .def("status_device_address", &SymmComm::status_device_address)
      .def("set_mc", &SymmComm::set_mc)
      .def("has_mc", &SymmComm::has_mc)
      .def("reset_epochs", &SymmComm::reset_epochs)
      .def("clear_status", &SymmComm::clear_status)
      .def("set_timeout_ns", &SymmComm::set_timeout_ns)
      .def("allreduce", &SymmComm::allreduce, py::arg("byte_off"), py::arg("n"), py::arg("is_bf16"),
           py::arg("weights") = py::none(), py::arg("blocks") = 32)
      .def("allreduce_oneshot", &SymmComm::allreduce_oneshot, py::arg("byte_off"), py::arg("n"), py::arg("in_bf16"),
           py::arg("out"), py::arg("weights") = py::none(), py::arg("blocks") = 32)
      .def("param_average", &SymmComm::param_average, py::arg("staging"), py::arg("n"), py::arg("weights") = py::none(),
           py::arg("alpha") = 1.0, py::arg("p16") = py::none(), py::arg("blocks") = 32)
      .def("broadcast", &SymmComm::broadcast, py::arg("byte_off"), py::arg("nbytes"), py::arg("root"), py::arg("blocks") = 32)
      .def("barrier", &SymmComm::barrier, py::arg("blocks") = 1);
}
