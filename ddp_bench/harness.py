"""Run one (model, mode) pair and return what the report needs (ddp-bench/src/harness.rs:40-215).

`solo-N` trains on one device with a plain loop. `sync` distributes a graph model with `Trainer.setup`
and drives it with `model.step()`. The builder modes go through `Trainer.builder(...).run().join()`
with the mode's policy and averaging backend. Every path uses the same dataset (fixed seed), the same
initial weights (seeded factory) and the same optimizer settings, so final losses are comparable.
Multi-rank modes expect one process per rank (torch.distributed.run); a `Timeline` records epoch
boundaries and the averaging events, and a `Monitor` can serve the live dashboard."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import torch

from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.data import TensorDataSet
from flodl_b200.monitor import Monitor, Timeline
from flodl_b200.parallel import comm
from flodl_b200.parallel.ddp import Trainer

from .config import DdpMode, RunOptions
from .models import ModelDef


@dataclass
class RunResult:
    model: str
    mode: str
    world: int
    device: str
    epochs: int
    batches_per_epoch: int
    batch_size: int
    epoch_losses: List[float] = field(default_factory=list)
    epoch_ms: List[float] = field(default_factory=list)
    final_eval: Optional[float] = None
    total_ms: float = 0.0
    timeline_events: int = 0
    error: str = ""

    def json(self) -> str:
        return json.dumps(asdict(self))


_TIMELINES: dict = {}       # (model, mode) -> the finished run's timeline, until `run()` has written it next to the result


def _timeline(opts: RunOptions) -> Timeline:
    """Events always; the background sampler (CPU, RAM, GPU utilisation and memory every 100 ms) only for runs whose
    results are kept, since only those are analysed."""
    tl = Timeline.new(100)
    if opts.output_dir:
        tl.start()
    return tl


def _keep_timeline(res: "RunResult", tl: Timeline) -> None:
    tl.stop()
    res.timeline_events = len(tl.events())
    _TIMELINES[(res.model, res.mode)] = tl


def _device(opts: RunOptions, index: int) -> torch.device:
    if opts.device == "cpu" or (opts.device == "auto" and not torch.cuda.is_available()):
        return torch.device("cpu")
    return torch.device("cuda", index % max(1, torch.cuda.device_count()))


def _resolve(md: ModelDef, opts: RunOptions):
    d = md.defaults
    epochs = opts.epochs or (2 if opts.tiny else d.epochs)
    bpe = opts.batches_per_epoch or (6 if opts.tiny else d.batches_per_epoch)
    bs = opts.batch_size or (16 if opts.tiny else d.batch_size)
    return epochs, bpe, bs, (opts.lr or d.lr) * (opts.lr_scale or 1.0)


def _factory(md: ModelDef, opts: RunOptions):
    def make(device):
        torch.manual_seed(opts.seed)            # identical initial weights on every rank and in every mode
        m = md.build(device, opts.tiny)
        m.train()
        return m
    return make


def _evaluate(md: ModelDef, model, x, y, device) -> float:
    model.eval()
    n = min(512, x.shape[0])
    v = md.eval_fn(model, x[:n].to(device), y[:n].to(device))
    model.train()
    return v


def run_solo(md: ModelDef, mode: DdpMode, opts: RunOptions) -> RunResult:
    epochs, bpe, bs, lr = _resolve(md, opts)
    device = _device(opts, mode.solo_index)
    x, y = md.dataset(bpe * bs, opts.seed, opts.tiny)
    model = _factory(md, opts)(device)
    opt = md.optimizer(lr)(model.parameters())
    res = RunResult(md.name, mode.name(), 1, str(device), epochs, bpe, bs)
    tl = _timeline(opts)
    t_all = time.perf_counter()
    for e in range(epochs):
        t0 = time.perf_counter()
        tl.event("EpochStart", epoch=e)
        perm = torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(opts.seed + e))
        total = 0.0
        for b in range(bpe):
            idx = perm[b * bs:(b + 1) * bs]
            loss = md.train_fn(model, (x[idx].to(device), y[idx].to(device)))
            opt.zero_grad()
            loss.backward()
            opt.step()
            total += loss.item()
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        tl.event("EpochEnd", epoch=e, loss=total / bpe)
        res.epoch_losses.append(total / bpe)
        res.epoch_ms.append((time.perf_counter() - t0) * 1e3)
    res.total_ms = (time.perf_counter() - t_all) * 1e3
    res.final_eval = _evaluate(md, model, x, y, device)
    _keep_timeline(res, tl)
    return res


def run_sync(md: ModelDef, mode: DdpMode, opts: RunOptions) -> RunResult:
    """Graph DDP: every rank feeds the whole batch, `forward` keeps this rank's rows, `step()` all-reduces."""
    if not md.graph:
        raise ValueError(f"mode 'sync' needs a FlowBuilder graph; {md.name} is a hand-written module")
    epochs, bpe, bs, lr = _resolve(md, opts)
    rank, world = comm.rank(), comm.world_size()
    device = _device(opts, comm.local_rank())
    x, y = md.dataset(bpe * bs, opts.seed, opts.tiny)
    model = _factory(md, opts)(device)
    Trainer.setup(model, None, md.optimizer(lr))
    res = RunResult(md.name, mode.name(), world, str(device), epochs, bpe, bs)
    tl = _timeline(opts)
    t_all = time.perf_counter()
    for e in range(epochs):
        t0 = time.perf_counter()
        tl.event("EpochStart", epoch=e)
        perm = torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(opts.seed + e))
        total = 0.0
        for b in range(bpe):
            idx = perm[b * bs:(b + 1) * bs]
            xb, yb = x[idx].to(device), y[idx].to(device)
            out = model.forward(Variable.wrap(xb))
            n = out.t.shape[0]
            start = sum(model.shard_sizes(xb.shape[0])[:rank]) if world > 1 else 0
            tgt = yb[start:start + n]
            loss = (nn.cross_entropy_loss(out, Variable.wrap(tgt)) if tgt.dtype == torch.long else nn.mse_loss(out, Variable.wrap(tgt)))
            loss.backward()
            model.step()
            total += loss.item()
        tl.event("EpochEnd", epoch=e, loss=total / bpe)
        res.epoch_losses.append(total / bpe)
        res.epoch_ms.append((time.perf_counter() - t0) * 1e3)
    res.total_ms = (time.perf_counter() - t_all) * 1e3
    # evaluate on a plain copy: the distributed graph's forward keeps only this rank's rows
    plain = _factory(md, opts)(device)
    with torch.no_grad():
        for dst, src in zip(plain.parameters(), model.parameters()):
            dst.t.copy_(src.t)
        for dst, src in zip(plain.buffers(), model.buffers()):
            dst.get().copy_(src.get())
    res.final_eval = _evaluate(md, plain, x, y, device)
    _keep_timeline(res, tl)
    return res


def run_builder(md: ModelDef, mode: DdpMode, opts: RunOptions) -> RunResult:
    epochs, bpe, bs, lr = _resolve(md, opts)
    world = comm.world_size() if comm.is_initialized() else 1
    device = _device(opts, comm.local_rank() if comm.is_initialized() else 0)
    x, y = md.dataset(bpe * bs, opts.seed, opts.tiny)
    tl = _timeline(opts)
    b = (Trainer.builder(_factory(md, opts), md.optimizer(lr), md.train_fn).dataset(TensorDataSet(x, y)).batch_size(bs).num_epochs(epochs)
         .policy(mode.policy).backend(mode.backend).timeline(tl))
    res = RunResult(md.name, mode.name(), world, str(device), epochs, bpe, bs)
    t_all = time.perf_counter()
    handle = b.run()
    monitor = None
    if opts.monitor_port > 0 and comm.rank() == 0:
        monitor = Monitor(epochs)
        monitor.serve(opts.monitor_port)
        handle.setup_monitor(monitor)
    state = handle.join()
    res.total_ms = (time.perf_counter() - t_all) * 1e3
    for m in handle.poll_metrics():
        res.epoch_losses.append(m.avg_loss)
        res.epoch_ms.append(float(m.scalars.get("epoch_ms", 0.0)))
    if state is not None:
        model = _factory(md, opts)(torch.device("cpu"))
        with torch.no_grad():
            for p, s in zip(model.parameters(), state.params):
                p.t.copy_(s)
            for bf, s in zip(model.buffers(), state.buffers):
                bf.get().copy_(s)
        res.final_eval = _evaluate(md, model, x, y, torch.device("cpu"))
    errs = handle.errors()
    if errs:
        res.error = "; ".join(str(e) for e in errs)
    _keep_timeline(res, tl)
    if monitor is not None:
        monitor.finish()
    return res


def run(md: ModelDef, mode: DdpMode, opts: RunOptions) -> Optional[RunResult]:
    """Dispatch one run. Returns the result on rank 0 (and on the only process of a solo run), None elsewhere."""
    if mode.kind == "solo":
        if comm.is_initialized() and comm.rank() != 0:
            return None
        res = run_solo(md, mode, opts)
    elif mode.kind == "sync":
        res = run_sync(md, mode, opts)
    else:
        res = run_builder(md, mode, opts)
    if comm.is_initialized() and comm.rank() != 0:
        return None
    if opts.output_dir:
        os.makedirs(opts.output_dir, exist_ok=True)
        with open(os.path.join(opts.output_dir, f"{md.name}__{mode.name()}.json"), "w") as f:
            f.write(res.json() + "\n")
        tl = _TIMELINES.pop((res.model, res.mode), None)
        if tl is not None:
            tl.save_json(os.path.join(opts.output_dir, f"{md.name}__{mode.name()}.timeline.json"))
    _TIMELINES.pop((res.model, res.mode), None)
    return res
