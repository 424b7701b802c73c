"""Gradient all-reduce sweep: this library's peer-memory kernels vs NCCL, 1 KB ... 1 GB, fp32 + bf16.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29520 bench_allreduce.py [--max-mb 1024] [--iters 20]

Values ~N(0, 1e-3), averaged across ranks (the fused scale). Device-timed with CUDA events, max over
ranks. Bus bandwidth = 2 (W-1)/W * bytes / time; roofline = the measured NVLink peer-copy rate
(770 GB/s per direction per GPU). The NCCL columns are the reference's path: `flat` = one
all-reduce over the same flat buffer, `per_tensor_25MB` = the same bytes as 25 MB chunks in one
group (flodl-sys/ops_cuda.cpp:496-537). Rank 0 prints one JSON line per size and a final summary line.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=0)
    args = ap.parse_args()
    comm.init_process_group()
    rank, world = comm.rank(), comm.world_size()
    dev = torch.device("cuda", comm.local_rank())
    torch.cuda.set_device(dev)
    max_bytes = args.max_mb << 20
    buf = comm.SymmetricBuffer(max_bytes, timeout_s=10.0)
    results = []
    for dtype in (torch.float32, torch.bfloat16):
        esz = 4 if dtype == torch.float32 else 2
        nbytes = 1024
        while nbytes <= max_bytes:
            numel = nbytes // esz
            v = buf.view(dtype, 0, numel)
            v.copy_((torch.randn(numel, device=dev) * 1e-3).to(dtype))
            iters = args.iters if nbytes <= (64 << 20) else max(5, args.iters // 4)
            blocks = args.blocks or (4 if nbytes <= (64 << 10) else 16 if nbytes <= (4 << 20) else 48)
            ms_two = timed(lambda: buf.all_reduce(0, numel, dtype, blocks=blocks), iters, dev)
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
            row = {"dtype": str(dtype).split(".")[-1], "bytes": nbytes, "world": world, "ours_two_shot_us": round(ms_two * 1e3, 2),
                   "ours_one_shot_us": None if ms_one is None else round(ms_one * 1e3, 2), "nccl_flat_us": round(ms_nccl * 1e3, 2),
                   "nccl_25MB_group_us": None if ms_nccl_chunks is None else round(ms_nccl_chunks * 1e3, 2),
                   "ours_bus_GBs": bus(best), "nccl_bus_GBs": bus(ms_nccl), "ours_frac_of_nvlink": round((bus(best) or 0) / NVLINK_GBS, 3),
                   "speedup_vs_nccl": round(ms_nccl / best, 3)}
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            nbytes *= 2
    if rank == 0:
        big = [r for r in results if r["bytes"] >= (64 << 20)]
        print(json.dumps({"summary": True, "world": world, "peak_ours_bus_GBs": max(r["ours_bus_GBs"] for r in results),
                          "peak_nccl_bus_GBs": max(r["nccl_bus_GBs"] for r in results),
                          "geomean_speedup_small(<=1MB)": round(float(torch.tensor([r["speedup_vs_nccl"] for r in results if r["bytes"] <= (1 << 20)]).log().mean().exp()), 3),
                          "geomean_speedup_large(>=64MB)": round(float(torch.tensor([r["speedup_vs_nccl"] for r in big]).log().mean().exp()), 3) if big else None}), flush=True)
    dist.barrier()
    comm.destroy_process_group()


if __name__ == "__main__":
    main()
