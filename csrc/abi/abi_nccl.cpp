// Drop-in C ABI, part 4: NCCL collectives. Two shapes, as in the interface hosts are written against:
//   * a GROUP of communicators for several devices driven by one process (`flodl_nccl_init` over
//     `ncclCommInitAll`): all-reduce / broadcast take one tensor per device and run in one NCCL group;
//   * a RANK communicator (`flodl_nccl_init_rank` from a shared unique id, one per process or thread):
//     all-reduce takes any number of tensors of this rank and batches them in one NCCL group.
// `flodl_nccl_split_rank` moves one device's communicator out of a group so a worker thread can own it.
// Ops: 0 sum, 1 prod, 2 max, 3 min, 4 avg (= ncclRedOp_t).
#include "abi_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <nccl.h>

#include <atomic>

using namespace fbabi;

#define FB_API extern "C" __attribute__((visibility("default")))

namespace {

ncclDataType_t nccl_type(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return ncclFloat32;
    case at::kDouble: return ncclFloat64;
    case at::kHalf: return ncclFloat16;
    case at::kBFloat16: return ncclBfloat16;
    case at::kInt: return ncclInt32;
    case at::kLong: return ncclInt64;
    case at::kByte: return ncclUint8;
    case at::kChar: return ncclInt8;
    default: TORCH_CHECK(false, "NCCL: unsupported dtype ", t);
  }
}
void ok(ncclResult_t r, const char* what) { TORCH_CHECK(r == ncclSuccess, what, ": ", ncclGetErrorString(r)); }

struct Group {
  std::vector<ncclComm_t> comms;
  std::vector<int> devices;
  ~Group() {
    for (auto c : comms)
      if (c) ncclCommDestroy(c);
  }
};
struct RankComm {
  ncclComm_t comm = nullptr;
  std::atomic<bool> aborted{false};
  ~RankComm() {
    if (comm && !aborted.load()) ncclCommDestroy(comm);
  }
};
cudaStream_t stream_for(void** streams, int i, int device) {
  if (streams && streams[i]) return static_cast<at::cuda::CUDAStream*>(streams[i])->stream();
  return at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream();
}

// Closes an NCCL group on every path out of the scope.
struct GroupScope {
  bool open = false;
  GroupScope() { ok(ncclGroupStart(), "ncclGroupStart"); open = true; }
  void close() {
    if (open) {
      open = false;
      ok(ncclGroupEnd(), "ncclGroupEnd");
    }
  }
  ~GroupScope() {
    if (open) ncclGroupEnd();
  }
};

}  // namespace

FB_API char* flodl_nccl_init(int ndev, const int* devlist, void** handle_out) {
  return guarded([&] {
    auto g = std::make_unique<Group>();
    g->comms.assign(static_cast<size_t>(ndev), nullptr);
    g->devices.assign(devlist, devlist + ndev);
    ok(ncclCommInitAll(g->comms.data(), ndev, devlist), "ncclCommInitAll");
    *handle_out = g.release();
  });
}
FB_API void flodl_nccl_destroy(void* handle) { delete static_cast<Group*>(handle); }
FB_API int flodl_nccl_size(void* handle) { return static_cast<int>(static_cast<Group*>(handle)->comms.size()); }
FB_API char* flodl_nccl_all_reduce(void* handle, Handle* tensors, void** streams, int op) {
  return guarded([&] {
    auto* g = static_cast<Group*>(handle);
    GroupScope scope;
    for (size_t i = 0; i < g->comms.size(); ++i) {
      Tensor& t = ref(tensors[i]);
      TORCH_CHECK(g->comms[i], "NCCL: the communicator of device slot ", i, " was moved out of this group");
      c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(g->devices[i]));
      ok(ncclAllReduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), nccl_type(t.scalar_type()), static_cast<ncclRedOp_t>(op), g->comms[i],
                       stream_for(streams, static_cast<int>(i), g->devices[i])),
         "ncclAllReduce");
    }
    scope.close();
  });
}
FB_API char* flodl_nccl_broadcast(void* handle, Handle* tensors, void** streams, int root) {
  return guarded([&] {
    auto* g = static_cast<Group*>(handle);
    GroupScope scope;
    for (size_t i = 0; i < g->comms.size(); ++i) {
      Tensor& t = ref(tensors[i]);
      TORCH_CHECK(g->comms[i], "NCCL: the communicator of device slot ", i, " was moved out of this group");
      c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(g->devices[i]));
      ok(ncclBroadcast(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), nccl_type(t.scalar_type()), root, g->comms[i],
                       stream_for(streams, static_cast<int>(i), g->devices[i])),
         "ncclBroadcast");
    }
    scope.close();
  });
}

FB_API char* flodl_nccl_get_unique_id(void* uid_out) {
  return guarded([&] {
    ncclUniqueId id;
    ok(ncclGetUniqueId(&id), "ncclGetUniqueId");
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    std::memcpy(uid_out, &id, sizeof(id));
  });
}
FB_API char* flodl_nccl_init_rank(int rank, int nranks, const void* uid, void** handle_out) {
  return guarded([&] {
    ncclUniqueId id;
    std::memcpy(&id, uid, sizeof(id));
    auto rc = std::make_unique<RankComm>();
    ok(ncclCommInitRank(&rc->comm, nranks, id, rank), "ncclCommInitRank");
    *handle_out = rc.release();
  });
}
FB_API void flodl_nccl_destroy_rank(void* handle) { delete static_cast<RankComm*>(handle); }
FB_API char* flodl_nccl_all_reduce_rank(void* handle, Handle* tensors, int ntensors, void* stream, int op) {
  return guarded([&] {
    auto* rc = static_cast<RankComm*>(handle);
    TORCH_CHECK(rc->comm && !rc->aborted.load(), "NCCL: communicator was aborted");
    cudaStream_t st = stream ? static_cast<at::cuda::CUDAStream*>(stream)->stream() : at::cuda::getCurrentCUDAStream().stream();
    GroupScope scope;
    for (int i = 0; i < ntensors; ++i) {
      Tensor& t = ref(tensors[i]);
      ok(ncclAllReduce(t.data_ptr(), t.data_ptr(), static_cast<size_t>(t.numel()), nccl_type(t.scalar_type()), static_cast<ncclRedOp_t>(op), rc->comm, st),
         "ncclAllReduce");
    }
    scope.close();
  });
}
// Unblocks a collective that is stuck (callable from any thread, once); the handle stays valid for destroy.
FB_API char* flodl_nccl_abort_rank(void* handle) {
  return guarded([&] {
    auto* rc = static_cast<RankComm*>(handle);
    if (!rc || !rc->comm) return;
    bool expected = false;
    if (!rc->aborted.compare_exchange_strong(expected, true)) return;
    ncclComm_t c = rc->comm;
    rc->comm = nullptr;
    ok(ncclCommAbort(c), "ncclCommAbort");
  });
}
FB_API char* flodl_nccl_split_rank(void* group_handle, int rank, void** rank_handle_out) {
  return guarded([&] {
    auto* g = static_cast<Group*>(group_handle);
    TORCH_CHECK(rank >= 0 && static_cast<size_t>(rank) < g->comms.size() && g->comms[static_cast<size_t>(rank)], "NCCL: no communicator at slot ", rank);
    auto rc = std::make_unique<RankComm>();
    rc->comm = g->comms[static_cast<size_t>(rank)];
    g->comms[static_cast<size_t>(rank)] = nullptr;
    *rank_handle_out = rc.release();
  });
}
