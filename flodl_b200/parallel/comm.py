"""Process group, streams/events and symmetric (peer-mapped) memory.

One process drives one GPU; `torch.distributed` (NCCL on GPUs, gloo on CPU) is the rendezvous and
the baseline collective backend, the way the reference uses NCCL communicators
(flodl/src/distributed/nccl.rs:56-571). What the reference does with `ncclAllReduce` /
`ncclBroadcast` this package does with its own kernels over `SymmetricBuffer`s: a raw CUDA
allocation per rank, exported through CUDA IPC, mapped by every peer, plus a small signal pad for
the device-side barriers. `ReduceOp` keeps the reference's numbering (= `ncclRedOp_t`, nccl.rs:37-48).
"""
from __future__ import annotations

import os
from enum import IntEnum
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _ext
from ..tensor import TensorError


class ReduceOp(IntEnum):
    Sum = 0
    Prod = 1
    Max = 2
    Min = 3
    Avg = 4

    def torch(self):
        return {0: dist.ReduceOp.SUM, 1: dist.ReduceOp.PRODUCT, 2: dist.ReduceOp.MAX, 3: dist.ReduceOp.MIN, 4: dist.ReduceOp.AVG}[int(self)]


# ---- process group -------------------------------------------------------------------------------
def init_process_group(backend: Optional[str] = None, timeout_s: float = 600.0) -> None:
    """Idempotent: reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* (torchrun) and joins the group;
    a single process without those variables is a world of one and needs no group."""
    if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    import datetime
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank())
    dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), timeout=datetime.timedelta(seconds=timeout_s),
                            **({"device_id": torch.device("cuda", local_rank())} if use_cuda else {}))


def is_initialized() -> bool:
    return dist.is_initialized()


def world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def destroy_process_group() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


# ---- streams / events (flodl/src/distributed/cuda_stream.rs, cuda_event.rs) -----------------------
class CudaStream:
    def __init__(self, device=None, high_priority: bool = False):
        self.s = torch.cuda.Stream(device=device, priority=-1 if high_priority else 0)

    @classmethod
    def new(cls, device=None, high_priority=False): return cls(device, high_priority)
    def synchronize(self) -> None: self.s.synchronize()
    def wait_event(self, ev: "CudaEvent") -> None: self.s.wait_event(ev.e)
    def wait_stream(self, other) -> None: self.s.wait_stream(other.s if isinstance(other, CudaStream) else other)
    def query(self) -> bool: return self.s.query()
    def guard(self): return torch.cuda.stream(self.s)


StreamGuard = lambda stream: stream.guard()  # noqa: E731  (`StreamGuard::new(stream)`)


class CudaEvent:
    def __init__(self, timing: bool = False):
        self.e = torch.cuda.Event(enable_timing=timing)

    @classmethod
    def new(cls, timing=False): return cls(timing)
    def record(self) -> None: self.e.record()
    def record_on(self, stream: CudaStream) -> None: self.e.record(stream.s)
    def synchronize(self) -> None: self.e.synchronize()
    def is_complete(self) -> bool: return self.e.query()
    def elapsed_ms(self, end: "CudaEvent") -> float: return self.e.elapsed_time(end.e)


# ---- symmetric memory ----------------------------------------------------------------------------
def _exchange(obj, group=None) -> list:
    if not dist.is_initialized():
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


class SymmetricBuffer:
    """`nbytes` of device memory on every rank, each rank holding a pointer to every peer's block.

    `view(dtype, offset_bytes, numel)` gives a tensor over the LOCAL block. Collective calls take
    byte offsets and run on the current CUDA stream; they must be issued in the same order, with
    the same sizes and block counts, on every rank. Device-side waits are bounded
    (`timeout_s`); `check()` turns a recorded give-up into an exception and `abort()` makes every
    pending wait on this rank return at once (the role `NcclAbortHandle` plays in the reference,
    nccl.rs:384-417)."""

    def __init__(self, nbytes: int, device: Optional[int] = None, timeout_s: float = 2.0, group=None):
        C = _ext.require()
        self.C = C
        self.device = torch.cuda.current_device() if device is None else device
        self.nbytes = (nbytes + 255) // 256 * 256
        self.rank, self.world = rank(), world_size()
        if self.world > C.MAX_RANKS:
            raise TensorError(f"world size {self.world} exceeds {C.MAX_RANKS}")
        self.data = C.SymmAlloc(self.nbytes, self.device)
        self.sig = C.SymmAlloc(C.SIGNAL_PAD_BYTES, self.device)
        handles = _exchange((self.data.ipc_handle(), self.sig.ipc_handle()), group)
        self._opened: List[int] = []
        dptrs, sptrs = [], []
        for r, (hd, hs) in enumerate(handles):
            if r == self.rank:
                dptrs.append(self.data.address())
                sptrs.append(self.sig.address())
            else:
                pd, ps = C.open_ipc(hd), C.open_ipc(hs)
                self._opened += [pd, ps]
                dptrs.append(pd)
                sptrs.append(ps)
        self.peer_ptrs = dptrs
        self.comm = C.SymmComm(self.rank, self.world, dptrs, sptrs, self.device, int(timeout_s * 1e9))
        barrier()

    def view(self, dtype: torch.dtype, offset_bytes: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // esz if numel is None else numel
        return self.data.tensor(dtype, offset_bytes, n)

    # collectives (current stream)
    def all_reduce(self, offset_bytes: int, numel: int, dtype: torch.dtype, weights: Optional[Sequence[float]] = None,
                   blocks: int = 32) -> None:
        """In place over [offset, offset + numel): two-shot reduce-scatter + all-gather, result is the
        weighted sum (default weights 1/world = average) on every rank."""
        self.comm.allreduce(offset_bytes, numel, dtype == torch.bfloat16, None if weights is None else list(weights), blocks)

    def all_reduce_into(self, offset_bytes: int, numel: int, dtype: torch.dtype, out: torch.Tensor,
                        weights: Optional[Sequence[float]] = None, blocks: int = 32) -> None:
        """One-shot: every rank reads all peers and writes `out` (fp32 or bf16, local)."""
        self.comm.allreduce_oneshot(offset_bytes, numel, dtype == torch.bfloat16, out, None if weights is None else list(weights), blocks)

    def broadcast(self, offset_bytes: int, nbytes: int, root: int = 0, blocks: int = 32) -> None:
        self.comm.broadcast(offset_bytes, nbytes, root, blocks)

    def barrier(self, blocks: int = 1) -> None:
        self.comm.barrier(blocks)

    def status(self) -> int:
        return self.comm.read_status()

    def check(self) -> None:
        st = self.comm.read_status()
        if st != 0:
            self.comm.clear_status()
            raise TensorError(f"symmetric collective gave up waiting for a peer (status {st}); a rank is late, gone or aborted")

    def abort(self) -> None:
        self.comm.abort()

    def clear_abort(self) -> None:
        self.comm.clear_abort()

    def close(self) -> None:
        for p in self._opened:
            self.C.close_ipc(p)
        self._opened = []


def all_reduce_nccl(tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.Avg) -> None:
    """The reference's path, kept as baseline and fallback: one collective per tensor in one group
    (flodl-sys/ops_cuda.cpp:496-537)."""
    if not dist.is_initialized():
        return
    if dist.get_backend() == "gloo" and op == ReduceOp.Avg:
        for t in tensors:
            dist.all_reduce(t, dist.ReduceOp.SUM)
            t.div_(dist.get_world_size())
        return
    with dist._coalescing_manager(device=tensors[0].device) if hasattr(dist, "_coalescing_manager") and tensors[0].is_cuda else _null():
        for t in tensors:
            dist.all_reduce(t, op.torch())


def broadcast_nccl(tensors: Sequence[torch.Tensor], root: int = 0) -> None:
    if not dist.is_initialized():
        return
    for t in tensors:
        dist.broadcast(t, root)


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


# ---- NCCL-shaped wrappers (flodl/src/distributed/nccl.rs:56-571) ---------------------------------
class NcclUniqueId:
    """The reference passes a 128-byte `ncclUniqueId` between threads to join one communicator.
    Here ranks rendezvous through `torch.distributed`; the id is an opaque 128-byte token kept for
    API parity (`NcclRankComm.init_rank` accepts and ignores it)."""
    BYTES = 128

    def __init__(self, raw: Optional[bytes] = None):
        self.raw = raw if raw is not None else os.urandom(self.BYTES)
        if len(self.raw) != self.BYTES:
            raise TensorError(f"NcclUniqueId must be {self.BYTES} bytes")

    @classmethod
    def new(cls) -> "NcclUniqueId":
        return cls()

    def as_bytes(self) -> bytes:
        return self.raw


class NcclAbortHandle:
    """Unblocks a rank stuck in a collective: sets the host-mapped abort flag of every symmetric
    buffer registered with it (the device-side waits of this library poll that flag) and asks
    the NCCL process group to abort where the installed torch supports it."""

    def __init__(self, buffers: Optional[List["SymmetricBuffer"]] = None):
        self.buffers = list(buffers or [])

    def register(self, buf: "SymmetricBuffer") -> None:
        self.buffers.append(buf)

    def abort(self) -> None:
        for b in self.buffers:
            b.abort()
        if dist.is_initialized():
            pg = dist.distributed_c10d._get_default_group()
            for name in ("abort", "_abort"):
                f = getattr(pg, name, None)
                if callable(f):
                    try:
                        f()
                    except Exception:
                        pass
                    break


class NcclRankComm:
    """This rank's end of the job-wide communicator: multi-tensor all-reduce in one group
    (flodl-sys/ops_cuda.cpp:496-537)."""

    def __init__(self):
        self._abort = NcclAbortHandle()

    @classmethod
    def init_rank(cls, rank: int, world_size: int, uid: Optional[NcclUniqueId] = None) -> "NcclRankComm":
        init_process_group()
        if world_size != globals()["world_size"]() or rank != globals()["rank"]():
            raise TensorError(f"init_rank({rank}, {world_size}) does not match the process group ({globals()['rank']()}, {globals()['world_size']()})")
        return cls()

    def rank(self) -> int: return rank()
    def world_size(self) -> int: return world_size()
    def abort_handle(self) -> NcclAbortHandle: return self._abort

    def all_reduce(self, tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.Sum) -> None:
        all_reduce_nccl(list(tensors), op)

    def all_reduce_on_stream(self, tensors: Sequence[torch.Tensor], op: ReduceOp, stream: CudaStream) -> None:
        with stream.guard():
            all_reduce_nccl(list(tensors), op)


class NcclComms:
    """Group view used by the synchronous path (`NcclComms::new(devices)` in the reference holds one
    communicator per device of the process; here each process holds its own rank's)."""

    def __init__(self, devices: Optional[Sequence] = None):
        init_process_group()
        self._devices = list(devices) if devices is not None else [f"cuda:{i}" for i in range(world_size())]

    @classmethod
    def new(cls, devices: Optional[Sequence] = None) -> "NcclComms":
        return cls(devices)

    def size(self) -> int: return world_size()
    def devices(self) -> List: return list(self._devices)

    def all_reduce(self, tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.Sum) -> None:
        all_reduce_nccl(list(tensors), op)

    def all_reduce_on_streams(self, tensors: Sequence[torch.Tensor], op: ReduceOp, streams: Sequence[CudaStream]) -> None:
        with streams[0].guard():
            all_reduce_nccl(list(tensors), op)

    def broadcast(self, tensors: Sequence[torch.Tensor], root: int = 0) -> None:
        broadcast_nccl(list(tensors), root)

    def broadcast_on_streams(self, tensors: Sequence[torch.Tensor], root: int, streams: Sequence[CudaStream]) -> None:
        with streams[0].guard():
            broadcast_nccl(list(tensors), root)

    def split(self) -> List[NcclRankComm]:
        """One rank communicator per local device: exactly one in a process-per-GPU job."""
        return [NcclRankComm()]
