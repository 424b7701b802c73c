"""Times one round of the CPU averaging backend on the host: the single native pass (`average_and_divergence`) against
the same arithmetic with tensor operations (`average_params` + `divergence_of`).

    python -m flodl_b200.parallel.ddp_run.bench_cpu_avg [--params 110000000] [--ranks 2] [--tensors 200] [--repeat 3]
"""
from __future__ import annotations

import argparse
import time

import torch

from . import ParamSnapshot, average_and_divergence, average_params, divergence_of


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--params", type=int, default=110_000_000)
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--tensors", type=int, default=200)
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args(argv)
    shape = (max(1, a.params // a.tensors),)
    snaps = [ParamSnapshot(r, [torch.randn(shape) for _ in range(a.tensors)], [], 3 + r) for r in range(a.ranks)]

    def best(f):
        ts = []
        for _ in range(a.repeat):
            t = time.perf_counter()
            f()
            ts.append(time.perf_counter() - t)
        return min(ts) * 1e3

    def tensor_ops():
        divergence_of(snaps, average_params(snaps, 1))
    one = best(lambda: average_and_divergence(snaps, 1))
    ops = best(tensor_ops)
    gb = a.tensors * shape[0] * 4 * (a.ranks + 1) / 1e9
    print(f"params {a.tensors * shape[0]} ranks {a.ranks} threads {torch.get_num_threads()}: one pass {one:.0f} ms ({gb / one * 1e3:.1f} GB/s of "
          f"{gb:.2f} GB that must move), tensor operations {ops:.0f} ms, {ops / one:.1f}x")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
