"""Process group, streams/events and symmetric (peer-mapped) memory.

One process drives one GPU; `torch.distributed` (NCCL on GPUs, gloo on CPU) is the rendezvous and
the baseline collective backend, the way the reference uses NCCL communicators
(flodl/src/distributed/nccl.rs:56-571). What the reference does with `ncclAllReduce` /
`ncclBroadcast` this package does with its own kernels over `SymmetricBuffer`s: one device
allocation per rank, mapped by every peer, plus a small signal pad for the device-side barriers.
Where the NVLink switch supports it the allocations come from the CUDA virtual-memory-management
API and are bound to a multicast object, so the kernels can let the switch do the reduction
(`multimem.ld_reduce` / `multimem.st`, "NVLS"); otherwise, or with `FLODL_B200_NVLS=0`, they are
`cudaMalloc` blocks shared through CUDA IPC and the kernels use plain peer loads and stores.
`ReduceOp` keeps the reference's numbering (= `ncclRedOp_t`, nccl.rs:37-48).
"""
from __future__ import annotations

import atexit
import enum
import os
import socket
import threading
import uuid
import weakref
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
    """Releases every live symmetric buffer (multicast bindings are undone on all ranks together,
    while the group can still synchronise them), then leaves the group."""
    close_all_symmetric()
    if dist.is_initialized():
        dist.destroy_process_group()


# ---- streams / events (flodl/src/distributed/cuda_stream.rs, cuda_event.rs) -----------------------
class CudaStream:
    def __init__(self, device=None, high_priority: bool = False):
        self.s = torch.cuda.Stream(device=device, priority=-1 if high_priority else 0)

    def is_complete(self) -> bool: return self.s.query()
    def device(self): return self.s.device

    @classmethod
    def new(cls, device=None, high_priority=False): return cls(device, high_priority)
    def synchronize(self) -> None: self.s.synchronize()
    def wait_event(self, ev: "CudaEvent") -> None: self.s.wait_event(ev.e)
    def wait_stream(self, other) -> None: self.s.wait_stream(other.s if isinstance(other, CudaStream) else other)
    def query(self) -> bool: return self.s.query()
    def guard(self): return torch.cuda.stream(self.s)


class StreamGuard:
    """Makes `stream` the current stream of its device until the guard is closed: `with StreamGuard(s): ...`,
    or `g = StreamGuard.new(s)` ... `g.close()` (flodl/src/distributed/cuda_stream.rs:120-150)."""

    def __init__(self, stream: CudaStream, enter: bool = False):
        self._ctx = stream.guard()
        self._open = False
        if enter:
            self.__enter__()

    @classmethod
    def new(cls, stream: CudaStream) -> "StreamGuard":
        return cls(stream, enter=True)

    def __enter__(self):
        self._ctx.__enter__()
        self._open = True
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def close(self) -> None:
        if self._open:
            self._open = False
            self._ctx.__exit__(None, None, None)


class CudaEventFlags(enum.IntEnum):
    """`Default` records timestamps (needed by `CudaEvent.elapsed_time`), `DisableTiming` is the
    cheaper synchronisation-only event (flodl/src/distributed/cuda_event.rs:32-37)."""
    Default = 0
    DisableTiming = 1


class CudaEvent:
    def __init__(self, timing=False):
        if isinstance(timing, CudaEventFlags):
            timing = timing == CudaEventFlags.Default
        self.e = torch.cuda.Event(enable_timing=bool(timing))

    @classmethod
    def new(cls, timing=False): return cls(timing)

    @staticmethod
    def elapsed_time(start: "CudaEvent", end: "CudaEvent") -> float:
        """Milliseconds between two recorded timing events."""
        return start.e.elapsed_time(end.e)

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


def nvls_wanted(world: Optional[int] = None) -> bool:
    """Whether symmetric buffers are bound to an NVLink multicast object. `FLODL_B200_NVLS=1|0` forces it on or
    off. By default it is used from four ranks up: the switch-side reduction moves 1 + 1/W of the payload per
    link direction against 2 (W - 1) / W for peer loads and stores, which pays from W = 4; measured at W = 2 the
    peer path reaches 678 GB/s bus against 400 GB/s through the switch (every operand, the local one included,
    crosses the link)."""
    e = os.environ.get("FLODL_B200_NVLS")
    if e is not None:
        return e not in ("0", "false", "off", "no")
    w = world if world is not None else world_size()
    return w >= int(os.environ.get("FLODL_B200_NVLS_MIN_WORLD", "4"))


def _exchange_fds(my_fds: Sequence[int], group=None) -> List[List[int]]:
    """Every rank hands the same file descriptors to every other rank of the node; returns, per
    rank, the descriptors received from it (this rank's own list at its own index). Descriptors
    travel as SCM_RIGHTS messages over abstract unix-domain sockets; the socket names are agreed
    through the process group."""
    r, w = rank(), world_size()
    token = _exchange(uuid.uuid4().hex if r == 0 else None, group)[0]
    name = lambda k: f"\0flodl_b200_{token}_{k}"  # noqa: E731
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name(r))
    srv.listen(w)
    srv.settimeout(120.0)
    counts = _exchange(len(my_fds), group)          # also: every server is listening from here on
    err: List[BaseException] = []

    def serve():
        try:
            for _ in range(w - 1):
                conn, _a = srv.accept()
                with conn:
                    if my_fds:
                        socket.send_fds(conn, [b"f"], list(my_fds))
                    else:
                        conn.sendall(b"n")
        except BaseException as e:  # noqa: BLE001
            err.append(e)

    th = threading.Thread(target=serve, daemon=True)
    th.start()
    out: List[List[int]] = [[] for _ in range(w)]
    out[r] = list(my_fds)
    try:
        for k in range(w):
            if k == r:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(120.0)
            with c:
                c.connect(name(k))
                if counts[k]:
                    _msg, fds, _flags, _addr = socket.recv_fds(c, 16, counts[k])
                    out[k] = list(fds)
                else:
                    c.recv(1)
    finally:
        th.join(timeout=130.0)
        srv.close()
    if err:
        raise TensorError(f"descriptor exchange failed: {err[0]}")
    return out


_LIVE_SYMM: "weakref.WeakSet[SymmetricBuffer]" = weakref.WeakSet()


def close_all_symmetric() -> None:
    for b in sorted(list(_LIVE_SYMM), key=lambda b: b._serial):
        b.close()


class SymmetricBuffer:
    """`nbytes` of device memory on every rank, each rank holding a pointer to every peer's block.

    `view(dtype, offset_bytes, numel)` gives a tensor over the LOCAL block. Collective calls take
    byte offsets and run on the current CUDA stream; they must be issued in the same order, with
    the same sizes and block counts, on every rank. Device-side waits are bounded
    (`timeout_s`); `check()` turns a recorded give-up into an exception and `abort()` makes every
    pending wait on this rank return at once (the role `NcclAbortHandle` plays in the reference,
    nccl.rs:384-417).

    `nvls=None` takes the switch-multicast path when the GPU reports support and
    `FLODL_B200_NVLS` does not say otherwise; `nvls=False` forces plain peer loads and stores
    (use that wherever a rank may leave or a wait is meant to run out)."""

    _count = 0

    def __init__(self, nbytes: int, device: Optional[int] = None, timeout_s: float = 2.0, group=None, nvls: Optional[bool] = None):
        C = _ext.require()
        self.C = C
        self.device = torch.cuda.current_device() if device is None else device
        self.nbytes = (nbytes + 255) // 256 * 256
        self.rank, self.world = rank(), world_size()
        self.group = group
        SymmetricBuffer._count += 1
        self._serial = SymmetricBuffer._count
        self._closed = False
        if self.world > C.MAX_RANKS:
            raise TensorError(f"world size {self.world} exceeds {C.MAX_RANKS}")
        want = nvls_wanted(self.world) if nvls is None else bool(nvls)
        want = want and self.world > 1 and C.multicast_supported(self.device)
        want = all(_exchange(bool(want), group))
        self.nvls = False
        self.data = None
        dptrs: List[int] = []
        self._opened: List[int] = []
        if want:
            dptrs = self._setup_vmm(group)
        if not dptrs:
            self.data = C.SymmAlloc(self.nbytes, self.device)
        self.sig = C.SymmAlloc(C.SIGNAL_PAD_BYTES, self.device)
        handles = _exchange((None if self.nvls else self.data.ipc_handle(), self.sig.ipc_handle()), group)
        sptrs = []
        ipc_d = []
        for r, (hd, hs) in enumerate(handles):
            if r == self.rank:
                ipc_d.append(self.data.address())
                sptrs.append(self.sig.address())
            else:
                ps = C.open_ipc(hs)
                self._opened.append(ps)
                sptrs.append(ps)
                if not self.nvls:
                    pd = C.open_ipc(hd)
                    self._opened.append(pd)
                    ipc_d.append(pd)
        if not self.nvls:
            dptrs = ipc_d
        self.peer_ptrs = dptrs
        self.comm = C.SymmComm(self.rank, self.world, dptrs, sptrs, self.device, int(timeout_s * 1e9))
        if self.nvls:
            self.comm.set_mc(self.data.mc_address())
        _LIVE_SYMM.add(self)
        barrier()

    def _setup_vmm(self, group) -> List[int]:
        """VMM allocation + peer mapping + multicast binding. Every step that can fail is followed by
        an agreement over the process group, so either all ranks end up on this path or none."""
        C = self.C

        def agree(ok: bool) -> bool:
            return all(_exchange(bool(ok), group))

        data, fds, err = None, [], None
        try:
            data = C.VmmAlloc(self.nbytes, self.device)
            fds = [data.export_fd()]
            if self.rank == 0:
                fds.append(data.mc_create(self.world))
        except Exception as e:  # noqa: BLE001
            err = e
        if not agree(err is None):
            for fd in fds:
                os.close(fd)
            if data is not None:
                data.release()
            if self.rank == 0 and err is not None:
                from .. import log
                log.verbose(f"NVLS set-up not available ({err}); using CUDA IPC peer memory")
            return []
        got = _exchange_fds(fds, group)
        ptrs: List[int] = []
        try:
            for r in range(self.world):
                ptrs.append(data.address() if r == self.rank else data.import_peer(got[r][0]))
            if self.rank != 0:
                data.mc_import(got[0][1])
            data.mc_add_device()
        except Exception as e:  # noqa: BLE001
            err = e
        finally:
            for r, lst in enumerate(got):
                for fd in lst:
                    try:
                        os.close(fd)
                    except OSError:
                        pass
        if not agree(err is None):           # all devices are in the team from here on (or nobody binds)
            data.release()
            return []
        try:
            data.mc_bind()
        except Exception as e:  # noqa: BLE001
            err = e
        if not agree(err is None):
            data.release()
            return []
        try:
            data.mc_map()
        except Exception as e:  # noqa: BLE001
            err = e
        if not agree(err is None):
            data.release()
            return []
        self.data = data
        self.nvls = True
        return ptrs

    def view(self, dtype: torch.dtype, offset_bytes: int = 0, numel: Optional[int] = None) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // esz if numel is None else numel
        return self.data.tensor(dtype, offset_bytes, n)

    # collectives (current stream)
    def all_reduce(self, offset_bytes: int, numel: int, dtype: torch.dtype, weights: Optional[Sequence[float]] = None,
                   blocks: int = 32) -> None:
        """In place over [offset, offset + numel): reduce-scatter + all-gather (through the switch
        when the buffer is multicast-bound and the weights are equal, peer loads and stores
        otherwise); the result is the weighted sum (default weights 1/world = average) on every rank."""
        self.comm.allreduce(offset_bytes, numel, dtype == torch.bfloat16, None if weights is None else list(weights), blocks)

    def all_reduce_into(self, offset_bytes: int, numel: int, dtype: torch.dtype, out: torch.Tensor,
                        weights: Optional[Sequence[float]] = None, blocks: int = 32) -> None:
        """One-shot: every rank reads all peers and writes `out` (fp32 or bf16, local)."""
        self.comm.allreduce_oneshot(offset_bytes, numel, dtype == torch.bfloat16, out, None if weights is None else list(weights), blocks)

    def broadcast(self, offset_bytes: int, nbytes: int, root: int = 0, blocks: int = 32) -> None:
        self.comm.broadcast(offset_bytes, nbytes, root, blocks)

    def barrier(self, blocks: int = 1) -> None:
        self.comm.barrier(blocks)

    # ---- failure handling -----------------------------------------------------------------------
    def status(self) -> int:
        """Waits for the device, then returns the status word (0 = every wait was answered)."""
        return self.comm.read_status()

    def poll(self) -> int:
        """The status word as it stands now, without waiting for the device (it is host-mapped)."""
        return self.comm.poll_status()

    def status_address(self) -> int:
        """Device address of the status word, for kernels that must not run after a give-up
        (the fused optimizers take it as their `skip` word)."""
        return self.comm.status_device_address()

    def _raise(self, st: int) -> None:
        what = {4: "gave up waiting for a peer", 7: "stopped because a peer had given up"}.get(st, f"reported status {st}")
        raise TensorError(f"symmetric collective {what} (status {st}); a rank is late, gone or aborted. "
                          "Gradients were not applied; call recover() on every rank before the next collective")

    def check(self) -> None:
        st = self.comm.read_status()
        if st != 0:
            self._raise(st)

    def check_async(self) -> None:
        """`check()` without a device sync: raises for a give-up that has already been reported."""
        st = self.comm.poll_status()
        if st != 0:
            self._raise(st)

    def recover(self) -> None:
        """Collective: after a give-up, every rank calls this to put flags, epochs and status back to
        their initial state (between two host barriers, with the device idle)."""
        torch.cuda.synchronize(self.device)
        barrier()
        self.sig.tensor(torch.int32, 0, self.C.SIGNAL_PAD_BYTES // 4).zero_()
        self.comm.reset_epochs()
        self.comm.clear_abort()
        torch.cuda.synchronize(self.device)
        self.comm.clear_status()
        barrier()

    def abort(self) -> None:
        self.comm.abort()

    def clear_abort(self) -> None:
        self.comm.clear_abort()

    def close(self) -> None:
        """Collective when multicast-bound: every rank unbinds before any rank frees its block."""
        if self._closed:
            return
        self._closed = True
        _LIVE_SYMM.discard(self)
        if torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
        if self.nvls and dist.is_initialized():
            try:
                barrier()
            except Exception:  # noqa: BLE001  (the group may be gone at interpreter exit)
                pass
        for p in self._opened:
            self.C.close_ipc(p)
        self._opened = []
        if self.nvls and self.data is not None:
            self.data.release()
            if dist.is_initialized():
                try:
                    barrier()
                except Exception:  # noqa: BLE001
                    pass


atexit.register(close_all_symmetric)


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
        self._aborted = False

    def is_aborted(self) -> bool:
        return self._aborted

    def register(self, buf: "SymmetricBuffer") -> None:
        self.buffers.append(buf)

    def abort(self) -> None:
        self._aborted = True
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
