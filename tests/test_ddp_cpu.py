"""Data-parallel logic on CPU: pure functions, then real multi-process runs over gloo."""
import os
import socket
import subprocess
import sys

import pytest

from flodl_b200.parallel.ddp import MIN_CHUNK_RATIO, rebalance_ratios, shard_sizes_from_ratios

HERE = os.path.dirname(os.path.abspath(__file__))


def test_rebalance_is_proportional_and_normalised():
    r = rebalance_ratios([300.0, 100.0])
    assert r == pytest.approx([0.75, 0.25])
    assert rebalance_ratios([0.0, 0.0]) is None


def test_rebalance_clamps_slow_ranks():
    r = rebalance_ratios([1000.0, 1.0, 1000.0])
    assert min(r) >= MIN_CHUNK_RATIO - 1e-9 and sum(r) == pytest.approx(1.0)
    assert r[0] == pytest.approx(r[2])


def test_shard_sizes_sum_to_batch():
    assert shard_sizes_from_ratios([0.5, 0.5], 9) == [4, 5]
    assert shard_sizes_from_ratios([0.7, 0.2, 0.1], 10) == [7, 2, 1]
    assert sum(shard_sizes_from_ratios([0.33, 0.33, 0.34], 128)) == 128


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(scenario: str, world: int = 2, timeout: int = 240):
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "_cpu_ddp_worker.py"), scenario], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=timeout)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"OK {scenario}" in out, f"rank {rank} failed:\n{out[-3000:]}"


@pytest.mark.parametrize("scenario", ["graph_ddp", "manual_ddp", "el_che_graph"])
def test_sync_ddp_over_gloo(scenario):
    run_ranks(scenario)


def test_sync_ddp_three_ranks():
    run_ranks("manual_ddp", world=3)
