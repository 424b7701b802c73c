"""Run the benchmark suite and print one JSON line per (model, implementation), then a comparison table.

    python -m benchmarks.run [--models mlp,convnet] [--impl flodl,torch] [--device cuda] [--rounds 1]
                             [--quick] [--out report.md]

`--rounds N` interleaves the implementations N times and keeps each one's best round (the reference's
run.sh does the same to cancel drift; it also locks the GPU clocks, which this runner never does: it
reads and reports them instead)."""
from __future__ import annotations

import argparse
import os
import json
import subprocess
import sys
from typing import Dict, List

import torch

from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.cli.args import answer_schema_probe

from .harness import BenchConfig, BenchResult, run_benchmark
from .models import MODELS, TIER1, TIER2


def run_model(name: str, impl: str, device: str, quick: bool, seed: int = 0, runs: int = 0, epochs: int = 0, warmup: int = -1,
              mode: str = "captured") -> BenchResult:
    """`mode` (flodl arm, CUDA only): "captured" runs the framework's standard training path, a
    `TrainEngine` whose whole step (forward, backward, fused optimizer over the flat parameter
    buffer) is one CUDA-graph launch; a model whose forward reads values on the host (data-dependent
    loops) cannot be captured and trains through the plain loop. "eager" is that plain op-by-op loop
    with a per-tensor optimizer for every model, the shape of the reference's benchmark loop."""
    build, cfg = MODELS[name]
    if quick:
        cfg = cfg.quick()
    if runs or epochs or warmup >= 0:
        cfg = BenchConfig(cfg.name, runs or cfg.runs, cfg.warmup_epochs if warmup < 0 else warmup, epochs or cfg.measured_epochs,
                          cfg.batches_per_epoch, cfg.batch_size)
    torch.manual_seed(seed)
    dev = torch.device(device)
    model, make_batch, loss_kind, lr = build(cfg, impl, dev, 8 if quick else 1)
    gen = torch.Generator().manual_seed(seed + 1)
    batches = [make_batch(dev, gen) for _ in range(cfg.batches_per_epoch)]
    impl_label = impl
    capturable = False
    if impl == "flodl" and mode == "captured" and dev.type == "cuda":
        model.train()

        def step_fn(x, y):
            pred = model.forward(Variable.wrap(x))
            if loss_kind == "ce":
                return nn.cross_entropy_loss(pred.reshape([-1, pred.t.shape[-1]]), Variable.wrap(y.reshape(-1)))
            return nn.mse_loss(pred, Variable.wrap(y))
        # A forward that reads device values on the host (a data-dependent loop count, an early exit)
        # cannot be recorded into a graph. Find out with one eager forward + backward under PyTorch's
        # sync detector rather than by letting a capture fail half-way. Such a model trains through the
        # plain op-by-op loop below (measured on B200, feedback_loop: 78 ms per epoch that way, 96 ms
        # stepping the flat-buffer engine without a capture, 94 ms PyTorch).
        capturable = True
        torch.cuda.synchronize()
        torch.cuda.set_sync_debug_mode("error")
        try:
            step_fn(*batches[0]).t.backward()
        except RuntimeError:
            capturable = False
        finally:
            torch.cuda.set_sync_debug_mode("default")
        torch.cuda.synchronize()
        for p in model.parameters():
            p.t.grad = None
    if capturable:
        from flodl_b200.parallel.engine import TrainEngine
        count = sum(p.t.numel() for p in model.parameters())
        eng = TrainEngine(model, lambda ps: nn.Adam(ps, lr))
        eng.capture(step_fn, list(batches[0]), warmup=2)
        impl_label = "flodl (one CUDA graph per step)"

        def epoch(_i, _warm):
            total = 0.0
            for x, y in batches:
                total += eng.replay([x, y]).item()
            return total / len(batches)
    elif impl == "flodl":
        if mode == "captured" and dev.type == "cuda":
            impl_label = "flodl (op by op: the forward reads device values on the host)"
        # an engine built for an earlier model of this process switched every size to the native kernels; the plain
        # loop wants the default again (small tensors through ATen: their cost is host time)
        from flodl_b200.ops import core as _core
        _core.set_eager_min_numel(int(os.environ.get("FLODL_B200_EAGER_MIN_NUMEL", str(1 << 20))))
        model.train()
        params = model.parameters()
        count = sum(p.t.numel() for p in params)
        opt = nn.Adam(params, lr)

        def epoch(_i, _warm):
            total = 0.0
            for x, y in batches:
                pred = model.forward(Variable.wrap(x))
                if loss_kind == "ce":
                    loss = nn.cross_entropy_loss(pred.reshape([-1, pred.t.shape[-1]]), Variable.wrap(y.reshape(-1)))
                else:
                    loss = nn.mse_loss(pred, Variable.wrap(y))
                opt.zero_grad()
                loss.backward()
                opt.step()
                total += loss.item()
            return total / len(batches)
    else:
        model.train()
        count = sum(p.numel() for p in model.parameters())
        opt = torch.optim.Adam(model.parameters(), lr=lr)

        def epoch(_i, _warm):
            total = 0.0
            for x, y in batches:
                pred = model(x)
                loss = (torch.nn.functional.cross_entropy(pred.reshape(-1, pred.shape[-1]), y.reshape(-1)) if loss_kind == "ce"
                        else torch.nn.functional.mse_loss(pred, y))
                opt.zero_grad(set_to_none=True)
                loss.backward()
                opt.step()
                total += loss.item()
            return total / len(batches)
    res = run_benchmark(cfg, impl, count, epoch, dev)
    res.impl = impl_label
    return res


def gpu_clocks() -> str:
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
        return out[0] if out else "n/a"
    except Exception:
        return "n/a"


def report(results: Dict[str, Dict[str, BenchResult]]) -> str:
    lines = ["| model | params | flodl_b200 ms/epoch | PyTorch ms/epoch | speed-up | flodl_b200 peak MB | PyTorch peak MB | flodl_b200 path |",
             "|---|---|---|---|---|---|---|---|"]
    for name, by in results.items():
        a, b = by.get("flodl"), by.get("torch")
        fmt = lambda r, f: "-" if r is None or f(r) is None else f"{f(r):.1f}"
        ratio = "-" if a is None or b is None else f"{b.median_epoch_ms / a.median_epoch_ms:.2f}x"
        lines.append(f"| {name} | {(a or b).param_count} | {fmt(a, lambda r: r.median_epoch_ms)} | {fmt(b, lambda r: r.median_epoch_ms)} | {ratio} | "
                     f"{fmt(a, lambda r: r.peak_vram_mb)} | {fmt(b, lambda r: r.peak_vram_mb)} | {a.impl if a is not None else '-'} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="benchmarks.run")
    ap.add_argument("--models", default="all", help="comma list, or all / tier1 / tier2")
    ap.add_argument("--impl", default="flodl,torch")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--rounds", type=int, default=1)
    ap.add_argument("--quick", action="store_true", help="tiny shapes and two epochs: a smoke test, not a measurement")
    ap.add_argument("--out", default="")
    ap.add_argument("--runs", type=int, default=0, help="passes per model (default 4, the first is discarded)")
    ap.add_argument("--epochs", type=int, default=0, help="measured epochs per pass (default 20)")
    ap.add_argument("--warmup", type=int, default=-1, help="warm-up epochs per pass (default 3)")
    ap.add_argument("--mode", default="captured", choices=["captured", "eager"],
                    help="flodl arm on CUDA: whole-step CUDA graph through TrainEngine (default) or the op-by-op loop")
    ap.add_argument("--warmup-secs", type=float, default=0.0, help="GPU warm-up before the first model (matrix products; 0 = none)")
    ap.add_argument("--lock-clocks", type=int, default=None, metavar="MHZ",
                    help="lock the SM clocks for the run and reset them afterwards (0 = the device's base clock). OFF unless given: "
                         "a GPU setting outlives the process, do not use it on a machine you share")
    answer_schema_probe(ap, argv)
    args = ap.parse_args(argv)
    if args.lock_clocks is not None and args.device.startswith("cuda"):
        from .clocks import ClockLock, NvmlBackend
        with ClockLock(NvmlBackend(), args.lock_clocks or None):
            return _run(args)
    return _run(args)


def _run(args) -> int:
    names = {"all": TIER1 + TIER2, "tier1": TIER1, "tier2": TIER2}.get(args.models) or [m for m in args.models.split(",") if m]
    impls = [i for i in args.impl.split(",") if i]
    for n in names:
        if n not in MODELS:
            print(f"unknown model {n!r}; known: {', '.join(MODELS)}", file=sys.stderr)
            return 2
    if args.warmup_secs > 0:
        from .clocks import gpu_warmup
        print(f"=== GPU warm-up: {gpu_warmup(args.warmup_secs, args.device)} products in {args.warmup_secs:.0f} s ===", flush=True)
    best: Dict[str, Dict[str, BenchResult]] = {n: {} for n in names}
    for _round in range(max(1, args.rounds)):
        for n in names:
            for impl in impls:           # interleaved: flodl, torch, flodl, torch, ...
                r = run_model(n, impl, args.device, args.quick, 0, args.runs, args.epochs, args.warmup, args.mode)
                print(r.json(), flush=True)
                if impl not in best[n] or r.median_epoch_ms < best[n][impl].median_epoch_ms:
                    best[n][impl] = r
    table = report(best)
    head = f"device {args.device}; clocks (sm, max, reasons): {gpu_clocks()}; rounds {args.rounds}{'; QUICK MODE' if args.quick else ''}"
    print(head)
    print(table)
    if args.out:
        with open(args.out, "w") as f:
            f.write(head + "\n\n" + table + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
