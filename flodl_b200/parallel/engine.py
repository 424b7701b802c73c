"""`TrainEngine`: the fused single-process-per-GPU training step.

What one step does (eager or replayed from a CUDA graph):

    zero the flat gradient buffer -> bump the dropout seed -> forward -> backward
      (weight gradients are written by the backward GEMMs straight into the flat buffer; each
       ~25 MB bucket is all-reduced over NVLink on a side stream as soon as it is complete)
    -> global-norm clip coefficient on the device (optional) -> ONE fused optimizer kernel over
       the flat parameter buffer, which also refreshes the bf16 shadow the next forward reads.

This replaces the reference's step sequence `backward -> per-parameter ncclAllReduce ->
per-buffer broadcast -> optimizer -> zero_grad` (flodl/src/graph/distributed.rs:239-452).
With `capture()` the whole step becomes one CUDA graph launch (the reference exposes CUDA graphs
through `cuda_graph_capture`, flodl/src/nn/cuda_graph.rs:166-190); per-step scalars (learning
rate, Adam bias corrections, dropout seed, collective epochs) live in device memory so a replay
is a correct new step.
"""
from __future__ import annotations

import os

from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..ops import core as _core_ops

from .. import _ext, ops as _ops
from ..nn.module import Module, Parameter, walk_modules
from ..tensor import TensorError
from . import comm as _comm
from .flat import FlatParams
from .grad_sync import GradSync

SEED_STRIDE = 1_000_003


class TrainEngine:
    def __init__(self, model: Module, optimizer_factory: Callable[[List[Parameter]], object], *, max_grad_norm: Optional[float] = None,
                 bucket_mb: float = 25.0, overlap: bool = True, comm_backend: str = "symm", comm_blocks: int = 24,
                 comm_timeout_s: float = 10.0, sync_params: bool = True, grad_sync: bool = True, param_staging: bool = False):
        """`grad_sync=False`: replicas do not exchange gradients (Local SGD); with
        `param_staging=True` the parameters still live in peer-mapped memory, next to a staging
        buffer of the same size, so `average_params()` can run the fused averaging kernel."""
        self.model = model
        params = model.parameters()
        tensors = [p.t for p in params]
        if not tensors:
            raise TensorError("TrainEngine: the model has no parameters")
        self.device = tensors[0].device
        self.world, self.rank = _comm.world_size(), _comm.rank()
        groups = [[p.t for p in g] for m in walk_modules(model) for g in m.fuse_groups()]
        self.symm_grads = self.symm_params = None
        grad_alloc = param_alloc = None
        self.symm_stage = None
        self.grad_sync = bool(grad_sync)
        use_symm = self.world > 1 and self.device.type == "cuda" and comm_backend == "symm"
        if use_symm and self.grad_sync:
            def grad_alloc(n):
                self.symm_grads = _comm.SymmetricBuffer(n * 4, self.device.index, comm_timeout_s)
                return self.symm_grads.view(torch.float32, 0, n)
        if use_symm and (self.grad_sync or param_staging):
            def param_alloc(n):
                self.symm_params = _comm.SymmetricBuffer(n * 4, self.device.index, comm_timeout_s)
                return self.symm_params.view(torch.float32, 0, n)
        self.flat = FlatParams(tensors, shadow=self.device.type == "cuda", grad_alloc=grad_alloc, param_alloc=param_alloc, groups=groups)
        if self.world > 1 and (comm_backend != "symm" or self.symm_grads is None):
            comm_backend = "nccl"
        if use_symm and param_staging:
            self.symm_stage = _comm.SymmetricBuffer(self.flat.total * 4, self.device.index, comm_timeout_s)
        _core_ops.set_eager_min_numel(0)      # flat buffers and direct gradient slots: native kernels for every size
        # launch shape of the gradient exchange (tuning knobs; the defaults come from measurements on B200)
        comm_blocks = int(os.environ.get("FLODL_B200_COMM_BLOCKS", comm_blocks))
        bucket_mb = float(os.environ.get("FLODL_B200_BUCKET_MB", bucket_mb))
        tail_blocks = int(os.environ.get("FLODL_B200_COMM_TAIL_BLOCKS", 96))
        self.sync = GradSync(self.flat, self.symm_grads, int(bucket_mb * 1024 * 1024), overlap, comm_blocks, comm_backend,
                             world=None if self.grad_sync else 1, tail_blocks=tail_blocks)
        # Buffers (BatchNorm running statistics) follow rank 0 after every step, as in the reference
        # (one ncclBroadcast per buffer per step, flodl/src/distributed/ddp.rs:150-157). Here they are
        # re-homed into one peer-mapped block and refreshed by ONE pull-broadcast launch per step.
        self.symm_bufs = None
        self._buf_bytes = 0
        self._float_bufs = [b.get() for b in model.buffers() if b.get().is_floating_point() and b.get().numel() > 0]
        if use_symm and self.grad_sync and self._float_bufs:
            n = sum((t.numel() + 3) // 4 * 4 for t in self._float_bufs)
            self.symm_bufs = _comm.SymmetricBuffer(n * 4, self.device.index, comm_timeout_s)
            block = self.symm_bufs.view(torch.float32, 0, n)
            block.zero_()
            off = 0
            with torch.no_grad():
                for t in self._float_bufs:
                    v = block[off:off + t.numel()].view(t.shape)
                    v.copy_(t.float())
                    t.data = v
                    off += (t.numel() + 3) // 4 * 4
            self._buf_bytes = off * 4
        self.optimizer = optimizer_factory(params)
        self.sync.guard(self.optimizer)       # a gradient exchange that gave up must never be applied
        self.max_grad_norm = max_grad_norm
        self.scheduler = None
        self.lr_scale = 1.0
        self.steps = 0
        self._graph = None
        self._static_in: List[torch.Tensor] = []
        self._static_loss: Optional[torch.Tensor] = None
        self._step_fn = None
        self.norm_out: Optional[torch.Tensor] = None
        if sync_params and self.world > 1:
            self.broadcast_params(0)

    # ---- parameter sync -------------------------------------------------------------------------
    def broadcast_params(self, root: int = 0) -> None:
        """Initial parameter sync: one P2P broadcast kernel over the flat buffer instead of one
        `ncclBroadcast` per tensor (ddp.rs:160-167)."""
        if self.world <= 1:
            return
        if self.symm_params is not None:
            self.symm_params.broadcast(0, self.flat.total * 4, root, 96)
        else:
            torch.distributed.broadcast(self.flat.params, root)
        self.flat.refresh_shadow()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if self.symm_params is not None:
            self.symm_params.check()

    def average_params(self, weights: Optional[Sequence[float]] = None, alpha: float = 1.0, blocks: Optional[int] = None) -> torch.Tensor:
        """Periodic parameter averaging for Local SGD: p <- p + alpha * (sum_r w_r p_r - p) on every
        rank. Returns a device tensor `[sum (p_new - p_old)^2, sum p_new^2]` (this rank's distance
        from the consensus), without a host sync.

        With peer-mapped parameters this is ONE kernel: each rank reduces its slice of all peers'
        parameters over NVLink, scatters the result into every peer's staging buffer, then blends it
        into its own fp32 weights, refreshes the bf16 shadow and accumulates the two norms in the
        same pass. The reference copies every parameter to scratch, calls `ncclAllReduce(Avg)` over
        all of them and derives the norms with three `foreach` passes
        (flodl/src/distributed/ddp_run/worker.rs:515-584)."""
        if self.world <= 1:
            return torch.zeros(2, device=self.device)
        n = self.flat.total
        if blocks is None:
            # nothing else runs while parameters are averaged, so the kernel may take most of the GPU:
            # measured on 2 x B200, 128 blocks move 52 M parameters in 0.43 ms against 0.57 ms with 32
            blocks = 128 if n >= (4 << 20) else 32
        if self.symm_stage is not None and self.symm_params is not None:
            return self.symm_params.comm.param_average(self.symm_stage.comm, n, None if weights is None else [float(w) for w in weights],
                                                       float(alpha), self.flat.shadow, blocks)
        p = self.flat.params
        with torch.no_grad():
            pre = p.clone()
            try:
                if weights is not None:
                    p.mul_(float(weights[self.rank]))
                    torch.distributed.all_reduce(p, torch.distributed.ReduceOp.SUM)
                else:
                    torch.distributed.all_reduce(p, torch.distributed.ReduceOp.SUM)
                    p.div_(self.world)
            except RuntimeError:
                p.copy_(pre)            # a peer left in the middle: keep this rank's own weights, whole
                raise
            if alpha != 1.0:
                p.copy_(torch.lerp(pre, p, float(alpha)))
            out = torch.stack([(p - pre).pow(2).sum(), p.pow(2).sum()])
            self.flat.refresh_shadow()
        return out

    def sync_buffers(self, root: int = 0) -> None:
        """Broadcast module buffers (BatchNorm running statistics) from `root`, packed into one message."""
        if self.world <= 1:
            return
        bufs = [b.get() for b in self.model.buffers() if b.get().is_floating_point()]
        if not bufs:
            return
        flatb = torch.cat([b.reshape(-1).float() for b in bufs])
        torch.distributed.broadcast(flatb, root)
        off = 0
        for b in bufs:
            b.copy_(flatb[off:off + b.numel()].view(b.shape))
            off += b.numel()

    def set_scheduler(self, scheduler, lr_scale: float = 1.0) -> None:
        self.scheduler, self.lr_scale = scheduler, lr_scale

    # ---- one step -------------------------------------------------------------------------------
    def _pre(self) -> None:
        if self.scheduler is not None:
            self.optimizer.set_lr(self.scheduler.lr(self.steps) * self.lr_scale)
        if hasattr(self.optimizer, "advance"):
            self.optimizer.advance()

    def _body(self, loss_fn: Callable[[], object]) -> torch.Tensor:
        self.flat.zero_grad()
        if self.device.type == "cuda":
            _ops.seed_state(self.device).add_(SEED_STRIDE)
        self.sync.begin_step()
        loss = loss_fn()
        lt = loss.t if hasattr(loss, "t") else loss
        lt.backward()
        # Without clipping (which needs every gradient first) the optimizer can start on the buckets
        # that have arrived while the last one, complete only now, is still being exchanged.
        import inspect
        can_split = (self.max_grad_norm is None and hasattr(self.optimizer, "apply") and getattr(self.optimizer, "fused", False)
                     and "window" in inspect.signature(self.optimizer.apply).parameters and not getattr(self.optimizer, "groups", None))
        tail = self.sync.finish(defer_tail=can_split)
        if self.symm_bufs is not None:
            self.symm_bufs.broadcast(0, self._buf_bytes, 0, 1)
        elif self.world > 1 and self.grad_sync and self._float_bufs:
            self.sync_buffers(0)
        if self.max_grad_norm is not None and self.device.type == "cuda" and _ops.native_enabled():
            self.norm_out = _ext.require().grad_norm(self.flat.grads, float(self.max_grad_norm), 1.0)
            self.optimizer.set_grad_scale(self.norm_out[1:2])
        elif self.max_grad_norm is not None:
            from ..nn.clip import clip_grad_norm
            clip_grad_norm(self.flat.tensors, self.max_grad_norm)
        if tail is not None:
            self.optimizer.apply(window=(tail[1], self.flat.total))
            self.sync.wait_tail()
            self.optimizer.apply(window=(tail[0], tail[1]))
        elif hasattr(self.optimizer, "apply"):
            self.optimizer.apply()
        else:
            if self.sync.symm is not None and not torch.cuda.is_current_stream_capturing():
                self.sync.check()         # no fused path to predicate on the device: wait and look
            self.optimizer.step()
        return lt.detach()

    def step(self, loss_fn: Callable[[], object]) -> torch.Tensor:
        """Eager step; returns the (device) loss tensor."""
        self._pre()
        if not hasattr(self.optimizer, "advance"):
            loss = self._body(loss_fn)
        else:
            loss = self._body(loss_fn)
        self.steps += 1
        return loss

    # ---- CUDA graph -----------------------------------------------------------------------------
    def capture(self, step_fn: Callable[..., object], example_inputs: Sequence[torch.Tensor], warmup: int = 3) -> None:
        """Capture `loss = step_fn(*inputs)` + backward + gradient sync + optimizer as one CUDA graph.
        `example_inputs` fix shapes and dtypes; `replay(inputs)` copies new data into the static
        input buffers and launches the graph."""
        if self.device.type != "cuda":
            raise TensorError("capture() needs a CUDA device")
        self._static_in = [t.to(self.device).clone() for t in example_inputs]
        self._step_fn = step_fn
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):          # also learns the gradient-bucket readiness counts
                self._pre()
                self._body(lambda: step_fn(*self._static_in))
                self.steps += 1
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.sync.check()
        self._pre()
        g = torch.cuda.CUDAGraph()
        from ..ops import core as _core
        _core.reset_zero_arena()     # zeroed scratch used inside the graph must be allocated (and re-zeroed) by the graph itself
        with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
            self._static_loss = self._body(lambda: step_fn(*self._static_in))
        _core.reset_zero_arena()
        self.steps += 1
        self._graph = g

    def replay(self, inputs: Sequence[torch.Tensor]) -> torch.Tensor:
        """One training step through the captured graph. `inputs` may be pinned host tensors (copied
        asynchronously) or device tensors. Returns the static device loss tensor."""
        if self._graph is None:
            raise TensorError("replay() before capture()")
        if self.sync.symm is not None:
            self.sync.symm.check_async()
        for dst, src in zip(self._static_in, inputs):
            dst.copy_(src, non_blocking=True)
        self._pre()
        self._graph.replay()
        self.steps += 1
        return self._static_loss

    def recover(self) -> None:
        """Collective: re-arm every symmetric buffer after a reported give-up."""
        for b in (self.symm_grads, self.symm_params, self.symm_stage, self.symm_bufs):
            if b is not None:
                b.recover()
        self.sync.reset()

    def check(self) -> None:
        """Raise if a device-side wait of this rank's collectives or GEMMs gave up."""
        self.sync.check()
        for b in (self.symm_params, self.symm_stage, self.symm_bufs):
            if b is not None:
                b.check_async()
        if self.device.type == "cuda":
            st = _ext.require().read_status(self.device.index or 0)
            if st != 0:
                raise TensorError(f"a tensor-core kernel reported status {st} (bounded wait gave up)")
