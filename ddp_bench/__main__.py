"""    python -m ddp_bench --list
    python -m ddp_bench --model mlp --mode solo-0 --output runs/
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m ddp_bench --model mlp --mode nccl-cadence --output runs/
    python -m ddp_bench --report runs/ [--report-out docs/ddp-benchmark.md]

`--model all` / `--mode all` sweep every model / every mode that the launch can run (solo modes in a
single process, the distributed modes under torch.distributed.run)."""
from __future__ import annotations

import argparse
import os
import sys

import torch

from flodl_b200.cli.args import answer_schema_probe
from flodl_b200.parallel import comm

from .config import ALL_MODES, DdpMode, RunOptions
from .harness import run
from .models import all_models, find_model
from .report import load_baselines, results_to_baselines, save_baselines, validate_results, write_report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ddp_bench")
    ap.add_argument("--list", action="store_true", help="show the models and modes, then exit")
    ap.add_argument("--model", "-m", default="mlp", choices=[m.name for m in all_models()] + ["all"], help="one model, or all")
    ap.add_argument("--mode", default="solo-0", choices=list(ALL_MODES) + ["all"], help="one DDP mode, or all")
    ap.add_argument("--epochs", type=int, help="epochs (default: the model's)")
    ap.add_argument("--batches", type=int, help="batches per epoch (default: the model's)")
    ap.add_argument("--batch-size", type=int, help="batch size per GPU")
    ap.add_argument("--lr", type=float, help="learning rate (default: the model's)")
    ap.add_argument("--seed", type=int, default=42, help="RNG seed")
    ap.add_argument("--device", default="auto", choices=["auto", "cpu", "cuda"], help="where to train")
    ap.add_argument("--output", default="", help="directory for results and timelines")
    ap.add_argument("--monitor", type=int, default=0, help="serve the live dashboard on this port (builder modes)")
    ap.add_argument("--tiny", action="store_true", help="smoke-test sizes")
    ap.add_argument("--report", default="", help="directory of results: print the report and exit")
    ap.add_argument("--report-out", default="")
    ap.add_argument("--lr-scale", type=float, help="multiply every model's default learning rate")
    ap.add_argument("--data-dir", default="data", help="dataset cache directory (the built-in tasks are synthetic and need none)")
    ap.add_argument("--validate", action="store_true", help="check the final losses against the baselines")
    ap.add_argument("--save-baseline", action="store_true", help="save this run's final losses as the new baselines")
    ap.add_argument("--baseline", default="baselines/baseline.json", help="baseline JSON file")
    ap.add_argument("--tolerance", type=float, default=0.15, help="relative loss tolerance of --validate")
    answer_schema_probe(ap, argv)
    args = ap.parse_args(argv)
    if args.list:
        for m in all_models():
            print(f"{m.name:14s} {m.description}")
        print("modes: " + ", ".join(ALL_MODES))
        return 0
    if args.report:
        print(write_report(args.report, args.report_out or None))
        return 0
    models = all_models() if args.model == "all" else [find_model(args.model)]
    if None in models:
        print(f"unknown model {args.model!r}", file=sys.stderr)
        return 2
    modes = [DdpMode.parse(m) for m in (ALL_MODES if args.mode == "all" else [args.mode])]
    if None in modes:
        print(f"unknown mode {args.mode!r}; known: {', '.join(ALL_MODES)}", file=sys.stderr)
        return 2
    distributed = int(os.environ.get("WORLD_SIZE", "1")) > 1
    if distributed and not comm.is_initialized():
        use_cuda = args.device != "cpu" and torch.cuda.is_available()
        comm.init_process_group("nccl" if use_cuda else "gloo")
    opts = RunOptions(args.epochs, args.batches, args.batch_size, args.lr, args.seed, args.device, args.output, args.monitor, args.tiny,
                      args.lr_scale)
    rc = 0
    finished = []
    for md in models:
        for mode in modes:
            if mode.requires_multi_gpu() and not distributed:
                if args.mode != "all":
                    print(f"mode {mode.name()} needs one process per rank (torch.distributed.run)", file=sys.stderr)
                    rc = 2
                continue
            if mode.kind == "solo" and mode.solo_index > 0 and args.device != "cpu" and torch.cuda.device_count() <= mode.solo_index and args.mode == "all":
                continue
            if mode.kind == "sync" and not md.graph:
                continue
            res = run(md, mode, opts)
            if res is not None:
                print(res.json(), flush=True)
                finished.append(res)
            if distributed:
                comm.barrier()
    if distributed:
        comm.destroy_process_group()
    if args.save_baseline and finished:
        save_baselines(args.baseline, results_to_baselines(finished))
        print(f"saved {len(finished)} baseline(s) to {args.baseline}", file=sys.stderr)
    if args.validate and finished:
        try:
            ok, bad, lines = validate_results(finished, load_baselines(args.baseline), args.tolerance)
        except ValueError as e:
            print(f"--validate: {e}", file=sys.stderr)
            return 2
        print("\n".join(lines), file=sys.stderr)
        print(f"validation: {ok} passed, {bad} failed", file=sys.stderr)
        rc = rc or (1 if bad else 0)
    return rc


if __name__ == "__main__":
    sys.exit(main())
