// VmmBlock: symmetric device memory over the CUDA VMM API with an optional NVLS multicast mapping.
// See csrc/include/fb_vmm.hpp for the contract.
#include "fb_vmm.hpp"

#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <mutex>
#include <stdexcept>

namespace fb {
namespace {

// Driver entry points, resolved once through the runtime (no link-time dependency on libcuda).
struct Driver {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  bool ok = false;
  std::string why;
};

template <typename F>
bool resolve(const char* name, F& fn, std::string& why) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    (void)cudaGetLastError();
    why = std::string("driver entry point not available: ") + name;
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
    ok = ok && resolve("cuMemCreate", d.MemCreate, d.why);
    ok = ok && resolve("cuMemRelease", d.MemRelease, d.why);
    ok = ok && resolve("cuMemGetAllocationGranularity", d.MemGetAllocationGranularity, d.why);
    ok = ok && resolve("cuMemAddressReserve", d.MemAddressReserve, d.why);
    ok = ok && resolve("cuMemAddressFree", d.MemAddressFree, d.why);
    ok = ok && resolve("cuMemMap", d.MemMap, d.why);
    ok = ok && resolve("cuMemUnmap", d.MemUnmap, d.why);
    ok = ok && resolve("cuMemSetAccess", d.MemSetAccess, d.why);
    ok = ok && resolve("cuMemExportToShareableHandle", d.MemExportToShareableHandle, d.why);
    ok = ok && resolve("cuMemImportFromShareableHandle", d.MemImportFromShareableHandle, d.why);
    ok = ok && resolve("cuMulticastCreate", d.MulticastCreate, d.why);
    ok = ok && resolve("cuMulticastAddDevice", d.MulticastAddDevice, d.why);
    ok = ok && resolve("cuMulticastBindMem", d.MulticastBindMem, d.why);
    ok = ok && resolve("cuMulticastUnbind", d.MulticastUnbind, d.why);
    ok = ok && resolve("cuMulticastGetGranularity", d.MulticastGetGranularity, d.why);
    ok = ok && resolve("cuDeviceGet", d.DeviceGet, d.why);
    ok = ok && resolve("cuDeviceGetAttribute", d.DeviceGetAttribute, d.why);
    ok = ok && resolve("cuGetErrorString", d.GetErrorString, d.why);
    d.ok = ok;
  });
  return d;
}

void check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* s = nullptr;
  Driver& d = driver();
  if (d.GetErrorString) d.GetErrorString(r, &s);
  throw std::runtime_error(std::string(what) + ": " + (s ? s : "unknown driver error") + " (" + std::to_string(static_cast<int>(r)) + ")");
}

Driver& need_driver() {
  Driver& d = driver();
  if (!d.ok) throw std::runtime_error(d.why.empty() ? "CUDA driver not available" : d.why);
  return d;
}

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

CUmemAccessDesc rw_access(int device) {
  CUmemAccessDesc a{};
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = device;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return a;
}

size_t round_up(size_t x, size_t g) { return (x + g - 1) / g * g; }

}  // namespace

bool VmmBlock::multicast_supported(int device) {
  Driver& d = driver();
  if (!d.ok) return false;
  (void)cudaFree(nullptr);   // make sure the primary context exists
  CUdevice dev;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
  return v != 0;
}

VmmBlock::VmmBlock(size_t nbytes, int device) : device_(device) {
  Driver& d = need_driver();
  if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
  (void)cudaFree(nullptr);
  CUmemAllocationProp prop = alloc_prop(device);
  size_t gran = 0;
  check(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (multicast_supported(device)) {
    // The bound range must be a multiple of the multicast granularity; the recommended value is used
    // when it is modest, the minimum otherwise.
    CUmulticastObjectProp mp{};
    mp.numDevices = 2;
    mp.size = gran;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mmin = 0, mrec = 0;
    if (d.MulticastGetGranularity(&mmin, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mmin > gran) gran = round_up(mmin, gran);
    if (d.MulticastGetGranularity(&mrec, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mrec > gran &&
        mrec <= (size_t(32) << 20))
      gran = round_up(mrec, gran);
  }
  size_ = round_up(nbytes > 0 ? nbytes : 1, gran);
  CUmemGenericAllocationHandle h;
  check(d.MemCreate(&h, size_, &prop, 0), "cuMemCreate");
  handle_ = h;
  CUdeviceptr va = 0;
  CUresult r = d.MemAddressReserve(&va, size_, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    d.MemRelease(h);
    handle_ = 0;
    check(r, "cuMemAddressReserve");
  }
  r = d.MemMap(va, size_, 0, h, 0);
  if (r == CUDA_SUCCESS) {
    CUmemAccessDesc a = rw_access(device);
    r = d.MemSetAccess(va, size_, &a, 1);
    if (r != CUDA_SUCCESS) d.MemUnmap(va, size_);
  }
  if (r != CUDA_SUCCESS) {
    d.MemAddressFree(va, size_);
    d.MemRelease(h);
    handle_ = 0;
    check(r, "cuMemMap/cuMemSetAccess");
  }
  local_va_ = va;
  if (cudaMemset(reinterpret_cast<void*>(va), 0, size_) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    release();
    throw std::runtime_error("cudaMemset on the VMM block failed");
  }
}

VmmBlock::~VmmBlock() { release(); }

int VmmBlock::export_fd() {
  Driver& d = need_driver();
  int fd = -1;
  check(d.MemExportToShareableHandle(&fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  return fd;
}

uint64_t VmmBlock::import_peer(int fd) {
  Driver& d = need_driver();
  cudaSetDevice(device_);
  CUmemGenericAllocationHandle h;
  check(d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle");
  CUdeviceptr va = 0;
  CUresult r = d.MemAddressReserve(&va, size_, 0, 0, 0);
  if (r == CUDA_SUCCESS) {
    r = d.MemMap(va, size_, 0, h, 0);
    if (r == CUDA_SUCCESS) {
      CUmemAccessDesc a = rw_access(device_);
      r = d.MemSetAccess(va, size_, &a, 1);
      if (r != CUDA_SUCCESS) d.MemUnmap(va, size_);
    }
    if (r != CUDA_SUCCESS) d.MemAddressFree(va, size_);
  }
  if (r != CUDA_SUCCESS) {
    d.MemRelease(h);
    check(r, "mapping a peer block");
  }
  peers_.push_back({h, va});
  return va;
}

int VmmBlock::mc_create(int world) {
  Driver& d = need_driver();
  cudaSetDevice(device_);
  CUmulticastObjectProp mp{};
  mp.numDevices = static_cast<unsigned>(world);
  mp.size = size_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  check(d.MulticastCreate(&h, &mp), "cuMulticastCreate");
  mc_handle_ = h;
  int fd = -1;
  CUresult r = d.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    d.MemRelease(h);
    mc_handle_ = 0;
    check(r, "cuMemExportToShareableHandle(multicast)");
  }
  return fd;
}

void VmmBlock::mc_import(int fd) {
  Driver& d = need_driver();
  cudaSetDevice(device_);
  CUmemGenericAllocationHandle h;
  check(d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle(multicast)");
  mc_handle_ = h;
}

void VmmBlock::mc_add_device() {
  Driver& d = need_driver();
  CUdevice dev;
  check(d.DeviceGet(&dev, device_), "cuDeviceGet");
  check(d.MulticastAddDevice(mc_handle_, dev), "cuMulticastAddDevice");
}

void VmmBlock::mc_bind() {
  Driver& d = need_driver();
  cudaSetDevice(device_);
  check(d.MulticastBindMem(mc_handle_, 0, handle_, 0, size_, 0), "cuMulticastBindMem");
  mc_bound_ = true;
}

uint64_t VmmBlock::mc_map() {
  Driver& d = need_driver();
  cudaSetDevice(device_);
  CUdeviceptr va = 0;
  check(d.MemAddressReserve(&va, size_, 0, 0, 0), "cuMemAddressReserve(multicast)");
  CUresult r = d.MemMap(va, size_, 0, mc_handle_, 0);
  if (r == CUDA_SUCCESS) {
    CUmemAccessDesc a = rw_access(device_);
    r = d.MemSetAccess(va, size_, &a, 1);
    if (r != CUDA_SUCCESS) d.MemUnmap(va, size_);
  }
  if (r != CUDA_SUCCESS) {
    d.MemAddressFree(va, size_);
    check(r, "mapping the multicast object");
  }
  mc_va_ = va;
  return va;
}

void VmmBlock::release() {
  Driver& d = driver();
  if (!d.ok) return;
  if (handle_ == 0 && mc_handle_ == 0 && peers_.empty()) return;
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  if (mc_va_) {
    d.MemUnmap(mc_va_, size_);
    d.MemAddressFree(mc_va_, size_);
    mc_va_ = 0;
  }
  if (mc_bound_) {
    CUdevice dev;
    if (d.DeviceGet(&dev, device_) == CUDA_SUCCESS) d.MulticastUnbind(mc_handle_, dev, 0, size_);
    mc_bound_ = false;
  }
  if (mc_handle_) {
    d.MemRelease(mc_handle_);
    mc_handle_ = 0;
  }
  for (auto& p : peers_) {
    d.MemUnmap(p.va, size_);
    d.MemAddressFree(p.va, size_);
    d.MemRelease(p.handle);
  }
  peers_.clear();
  if (local_va_) {
    d.MemUnmap(local_va_, size_);
    d.MemAddressFree(local_va_, size_);
    local_va_ = 0;
  }
  if (handle_) {
    d.MemRelease(handle_);
    handle_ = 0;
  }
}

}  // namespace fb
