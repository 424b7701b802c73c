"""The DDP validation bench in smoke mode: mode parsing, every model's solo run, the distributed modes under
gloo with two ranks, and the report."""
import json
import os
import subprocess
import sys

import pytest

from ddp_bench.config import ALL_MODES, DdpMode, RunOptions
from ddp_bench.harness import run
from ddp_bench.models import all_models, find_model
from ddp_bench.report import analyze, load_results, render
from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_modes_parse_and_round_trip():
    assert len(ALL_MODES) == 9
    for name in ALL_MODES:
        m = DdpMode.parse(name)
        assert m is not None and m.name() == name
    assert DdpMode.parse("solo-3").solo_index == 3 and not DdpMode.parse("solo-3").requires_multi_gpu()
    m = DdpMode.parse("cpu-cadence")
    assert m.policy == ApplyPolicy.Cadence and m.backend == AverageBackend.Cpu and m.requires_multi_gpu()
    assert DdpMode.parse("nccl-bogus") is None and DdpMode.parse("solo-x") is None


def test_eight_models_registered():
    names = [m.name for m in all_models()]
    assert names == ["logistic", "mlp", "lenet", "resnet", "resnet_graph", "char_rnn", "gpt_nano", "conv_ae"]
    assert find_model("nope") is None


@pytest.mark.parametrize("name", ["logistic", "lenet", "resnet_graph", "char_rnn", "gpt_nano", "conv_ae"])
def test_solo_run_trains(name, tmp_path):
    res = run(find_model(name), DdpMode.parse("solo-0"), RunOptions(tiny=True, device="cpu", output_dir=str(tmp_path)))
    assert len(res.epoch_losses) == 2 and res.final_eval is not None and res.timeline_events == 4
    assert (tmp_path / f"{name}__solo-0.json").exists()


def _launch(mode, out, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", str(port),
           "-m", "ddp_bench", "--model", "mlp", "--mode", mode, "--tiny", "--device", "cpu", "--output", out]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1            # rank 0 only
    return json.loads(lines[0])


def test_distributed_modes_and_report(tmp_path):
    out = str(tmp_path)
    run(find_model("mlp"), DdpMode.parse("solo-0"), RunOptions(tiny=True, device="cpu", output_dir=out))
    for i, mode in enumerate(["sync", "nccl-cadence", "cpu-sync"]):
        r = _launch(mode, out, 29721 + i)
        assert r["world"] == 2 and r["mode"] == mode and len(r["epoch_losses"]) == 2 and r["error"] == ""
    rows = analyze(load_results(out))
    assert [r["mode"] for r in rows] == ["solo-0", "sync", "nccl-cadence", "cpu-sync"]
    assert all("loss_delta" in r and "speedup_vs_solo" in r for r in rows)
    text = render(rows)
    assert "## mlp" in text and "| nccl-cadence | 2 |" in text and "reference" in text
