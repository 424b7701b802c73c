// Symmetric device memory built on the CUDA virtual-memory-management API, with an optional
// NVLink-switch multicast mapping (NVLS).
//
// A `VmmBlock` is one physical allocation on this process's GPU (`cuMemCreate`) mapped into its
// address space. It can be exported as a POSIX file descriptor, the peers import that descriptor
// and map the same physical memory (`cuMemImportFromShareableHandle` + `cuMemMap`), which gives
// every rank the table of peer pointers the collectives index by rank. When the GPUs sit behind an
// NVSwitch that supports it, the blocks of all ranks are additionally bound to one multicast object
// (`cuMulticastCreate` / `cuMulticastAddDevice` / `cuMulticastBindMem`); the address that object is
// mapped at is the operand of `multimem.ld_reduce` (the switch reads the same offset on every GPU
// and returns the sum) and `multimem.st` (the switch writes every GPU's copy).
//
// This replaces the NCCL communicator set-up of the reference (flodl-sys/ops_cuda.cpp:265-324,
// 451-472). Nothing here links against libcuda: the driver entry points are resolved at run time
// through the CUDA runtime, so the library still loads on a machine without a GPU.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace fb {

class VmmBlock {
 public:
  // Allocates `nbytes` (rounded up to the allocation / multicast granularity) on `device`, zeroed.
  // Throws std::runtime_error with the driver's message when the platform cannot do it.
  VmmBlock(size_t nbytes, int device);
  ~VmmBlock();
  VmmBlock(const VmmBlock&) = delete;
  VmmBlock& operator=(const VmmBlock&) = delete;

  size_t size() const { return size_; }            // bytes actually allocated
  int device() const { return device_; }
  uint64_t address() const { return local_va_; }   // local mapping of the local block

  // True when the device reports CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED.
  static bool multicast_supported(int device);

  // ---- peer mapping -------------------------------------------------------------------------
  int export_fd();                                 // caller owns (and closes) the descriptor
  uint64_t import_peer(int fd);                    // maps a peer's block; closes nothing

  // ---- multicast (every rank makes these calls in this order, with a host barrier between
  //      add_device and bind, and between bind and the first kernel) --------------------------
  int mc_create(int world);                        // rank 0: creates the object, returns its fd
  void mc_import(int fd);                          // other ranks
  void mc_add_device();
  void mc_bind();                                  // binds the local block at offset 0
  uint64_t mc_map();                               // maps the object; returns the multicast address
  uint64_t mc_address() const { return mc_va_; }

  // Unbinds and unmaps everything (idempotent). Call on every rank, after a device synchronise and
  // a host barrier, before any rank's process exits: a block must not stay bound to a multicast
  // object whose team is being torn down.
  void release();

 private:
  size_t size_ = 0;
  int device_ = 0;
  uint64_t handle_ = 0;      // CUmemGenericAllocationHandle of the local block
  uint64_t local_va_ = 0;
  uint64_t mc_handle_ = 0;
  uint64_t mc_va_ = 0;
  bool mc_bound_ = false;
  struct Peer { uint64_t handle, va; };
  std::vector<Peer> peers_;
};

}  // namespace fb
