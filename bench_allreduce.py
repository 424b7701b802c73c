"""Gradient all-reduce sweep: this library's peer-memory kernels vs NCCL, 1 KB ... 1 GB, fp32 + bf16.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29520 bench_allreduce.py [--max-mb 1024] [--iters 20]

Values ~N(0, 1e-3), averaged across ranks (the fused scale). Device-timed with CUDA events, max over
ranks. Bus bandwidth = 2 (W-1)/W * bytes / time; roofline = the measured NVLink peer-copy rate
(770 GB/s per direction per GPU). The NCCL columns are the reference's path: `flat` = one
all-reduce over the same flat buffer, `per_tensor_25MB` = the same bytes as 25 MB chunks in one
group (flodl-sys/ops_cuda.cpp:496-537). Rank 0 prints one JSON line per size and a final summary line.

`--also param_average,broadcast` adds the two other collectives of the training loops:
  * parameter averaging of Local SGD over P fp32 parameters (52 M = the decoder LM, 110 M = BERT-base):
    the fused kernel (peer reduce + lerp + bf16 shadow + divergence sums, one launch) against the
    reference's sequence (copy to scratch, ncclAllReduce(Avg), three foreach norm passes;
    flodl/src/distributed/ddp_run/worker.rs:515-584);
  * parameter broadcast from rank 0 (time-to-sync at start-up) and the per-step buffer broadcast:
    one pull kernel over the flat buffer against one ncclBroadcast per tensor (flodl/src/distributed/ddp.rs:150-167).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from flodl_b200.parallel import comm  # noqa: E402

NVLINK_GBS = 770.0


def timed(fn, iters, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, dist.ReduceOp.MAX)
    return float(t.item())


def bench_param_average(buf, max_bytes, iters, dev, rank, world):
    """W = world ranks average P fp32 parameters in place (alpha = 1) and get the two divergence sums."""
    for name, P in (("decoder-lm", 52_000_000), ("bert-base", 110_000_000)):
        if P * 4 > max_bytes:
            continue
        stage = comm.SymmetricBuffer(P * 4, timeout_s=10.0)
        params = buf.view(torch.float32, 0, P)
        params.copy_(torch.randn(P, device=dev) * 0.02)
        shadow = torch.empty(P, device=dev, dtype=torch.bfloat16)
        per_blocks = {nb: timed(lambda: buf.comm.param_average(stage.comm, P, None, 1.0, shadow, nb), max(5, iters // 2), dev) for nb in (32, 64, 128)}
        ms_ours = min(per_blocks.values())
        buf.check()
        # the reference's sequence on a plain tensor of the same size
        p2 = torch.randn(P, device=dev) * 0.02
        chunks = list(p2.split(P // 200))          # ~200 parameter tensors

        def reference():
            pre = [c.clone() for c in chunks]
            with dist._coalescing_manager(device=dev):
                for c in chunks:
                    dist.all_reduce(c, dist.ReduceOp.AVG)
            diff = torch._foreach_sub(chunks, pre)
            d2 = torch.stack(torch._foreach_norm(diff)).pow(2).sum()
            n2 = torch.stack(torch._foreach_norm(chunks)).pow(2).sum()
            shadow.copy_(p2)
            return d2, n2
        ms_ref = timed(reference, max(5, iters // 2), dev)
        stage.close()
        if rank == 0:
            print(json.dumps({"collective": "param_average", "model": name, "params": P, "world": world, "ours_fused_us": round(ms_ours * 1e3, 1),
                              "ours_us_by_blocks": {str(k): round(v * 1e3, 1) for k, v in per_blocks.items()}, "reference_sequence_us": round(ms_ref * 1e3, 1), "speedup": round(ms_ref / ms_ours, 3),
                              "ours_bus_GBs": round(2 * (world - 1) / world * P * 4 / (ms_ours * 1e-3) / 1e9, 1)}), flush=True)


def bench_broadcast(buf, max_bytes, iters, dev, rank, world):
    """Rank 0's flat buffer to every rank: all parameters once (start-up), BatchNorm buffers every step."""
    for name, nbytes, ntensors in (("resnet20 BN buffers", 11_000, 42), ("decoder-lm params", 208_000_000, 80), ("bert-base params", 440_000_000, 200)):
        if nbytes > max_bytes:
            continue
        nbytes = nbytes // 16 * 16
        ms_ours = min(timed(lambda: buf.broadcast(0, nbytes, 0, nb), max(5, iters // 2), dev) for nb in ((32, 96) if nbytes > (1 << 20) else (1,)))
        buf.check()
        t = torch.randn(nbytes // 4, device=dev)
        parts = list(t.split(max(1, t.numel() // ntensors)))

        def reference():
            with dist._coalescing_manager(device=dev):
                for c in parts:
                    dist.broadcast(c, 0)
        try:
            ms_ref = timed(reference, max(5, iters // 2), dev)
        except Exception:       # coalesced broadcast is not available in every torch build
            ms_ref = timed(lambda: [dist.broadcast(c, 0) for c in parts], max(5, iters // 2), dev)
        if rank == 0:
            print(json.dumps({"collective": "broadcast", "what": name, "bytes": nbytes, "tensors": len(parts), "world": world,
                              "ours_pull_kernel_us": round(ms_ours * 1e3, 1), "nccl_per_tensor_us": round(ms_ref * 1e3, 1),
                              "speedup": round(ms_ref / ms_ours, 3), "ours_GBs_per_rank": round(nbytes / (ms_ours * 1e-3) / 1e9, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--also", default="", help="comma-separated extras: param_average, broadcast")
    ap.add_argument("--skip-sweep", action="store_true", help="only run the --also benchmarks")
    args = ap.parse_args()
    comm.init_process_group(timeout_s=180.0)
    rank, world = comm.rank(), comm.world_size()
    dev = torch.device("cuda", comm.local_rank())
    torch.cuda.set_device(dev)
    max_bytes = args.max_mb << 20
    buf = comm.SymmetricBuffer(max_bytes, timeout_s=10.0)
    results = []
    for dtype in (() if args.skip_sweep else (torch.float32, torch.bfloat16)):
        esz = 4 if dtype == torch.float32 else 2
        nbytes = 1024
        while nbytes <= max_bytes:
            numel = nbytes // esz
            v = buf.view(dtype, 0, numel)
            v.copy_((torch.randn(numel, device=dev) * 1e-3).to(dtype))
            iters = args.iters if nbytes <= (64 << 20) else max(5, args.iters // 4)
            blocks = args.blocks or (4 if nbytes <= (64 << 10) else 16 if nbytes <= (4 << 20) else 48)
            ms_two = timed(lambda: buf.all_reduce(0, numel, dtype, blocks=blocks), iters, dev)
            best_blocks = blocks
            if not args.blocks and nbytes >= (32 << 20):      # large messages: also try wider launches, keep the best
                for nb in (96, 192):
                    t = timed(lambda: buf.all_reduce(0, numel, dtype, blocks=nb), iters, dev)
                    if t < ms_two:
                        ms_two, best_blocks = t, nb
            buf.check()
            ms_one = None
            if nbytes <= (8 << 20):
                out = torch.empty(numel, device=dev, dtype=torch.float32)
                ms_one = timed(lambda: buf.all_reduce_into(0, numel, dtype, out, blocks=blocks), iters, dev)
            flat = torch.randn(numel, device=dev).to(dtype)
            ms_nccl = timed(lambda: dist.all_reduce(flat, dist.ReduceOp.AVG), iters, dev)
            chunk = (25 << 20) // esz
            parts = list(flat.split(chunk)) if numel > chunk else None
            ms_nccl_chunks = None
            if parts is not None:
                def grouped():
                    with dist._coalescing_manager(device=dev):
                        for p in parts:
                            dist.all_reduce(p, dist.ReduceOp.AVG)
                ms_nccl_chunks = timed(grouped, iters, dev)
            bus = lambda ms: None if ms is None else round(2 * (world - 1) / world * nbytes / (ms * 1e-3) / 1e9, 2)
            best = min(x for x in (ms_two, ms_one) if x is not None)
            row = {"dtype": str(dtype).split(".")[-1], "bytes": nbytes, "world": world, "path": "nvls" if buf.nvls else "p2p", "blocks": best_blocks,
                   "ours_two_shot_us": round(ms_two * 1e3, 2),
                   "ours_one_shot_us": None if ms_one is None else round(ms_one * 1e3, 2), "nccl_flat_us": round(ms_nccl * 1e3, 2),
                   "nccl_25MB_group_us": None if ms_nccl_chunks is None else round(ms_nccl_chunks * 1e3, 2),
                   "ours_bus_GBs": bus(best), "nccl_bus_GBs": bus(ms_nccl), "ours_frac_of_nvlink": round((bus(best) or 0) / NVLINK_GBS, 3),
                   "speedup_vs_nccl": round(ms_nccl / best, 3)}
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            nbytes *= 2
    extras = [e for e in args.also.split(",") if e]
    if "param_average" in extras:
        bench_param_average(buf, max_bytes, args.iters, dev, rank, world)
    if "broadcast" in extras:
        bench_broadcast(buf, max_bytes, args.iters, dev, rank, world)
    if rank == 0 and results:
        big = [r for r in results if r["bytes"] >= (64 << 20)]
        print(json.dumps({"summary": True, "world": world, "peak_ours_bus_GBs": max(r["ours_bus_GBs"] for r in results),
                          "peak_nccl_bus_GBs": max(r["nccl_bus_GBs"] for r in results),
                          "geomean_speedup_small(<=1MB)": round(float(torch.tensor([r["speedup_vs_nccl"] for r in results if r["bytes"] <= (1 << 20)]).log().mean().exp()), 3),
                          "geomean_speedup_large(>=64MB)": round(float(torch.tensor([r["speedup_vs_nccl"] for r in big]).log().mean().exp()), 3) if big else None}), flush=True)
    dist.barrier()
    comm.destroy_process_group()


if __name__ == "__main__":
    main()
