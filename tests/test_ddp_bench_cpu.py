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


# ---- baselines, validation, schema probe -------------------------------------------------------------------------
def test_baselines_round_trip_and_validation(tmp_path):
    from ddp_bench.harness import RunResult
    from ddp_bench.report import Baseline, load_baselines, results_to_baselines, save_baselines, validate_results
    runs = [RunResult("mlp", "solo-0", 1, "cpu", 2, 6, 16, [0.9, 0.5]), RunResult("lenet", "solo-0", 1, "cpu", 2, 6, 16, [1.2, 1.0]),
            RunResult("broken", "solo-0", 1, "cpu", 2, 6, 16, [], error="boom")]
    bs = results_to_baselines(runs)
    assert [(b.model, b.loss, b.epochs, b.batches, b.batch_size) for b in bs] == [("mlp", 0.5, 2, 6, 16), ("lenet", 1.0, 2, 6, 16)]
    path = str(tmp_path / "baselines" / "b.json")
    save_baselines(path, bs)
    back = load_baselines(path)
    assert back == bs and open(path).read().startswith('[\n  {"model":"mlp","mode":"solo-0","loss":0.500000,')
    later = [RunResult("mlp", "nccl-cadence", 2, "cpu", 2, 6, 16, [0.8, 0.55]), RunResult("lenet", "nccl-cadence", 2, "cpu", 2, 6, 16, [1.5, 1.4]),
             RunResult("gpt_nano", "solo-0", 1, "cpu", 2, 6, 16, [3.0]), RunResult("mlp", "cpu-async", 2, "cpu", 2, 6, 16, [float("nan")])]
    ok, bad, lines = validate_results(later, back, 0.15)
    assert (ok, bad) == (1, 2)
    assert lines[0].startswith("  PASS  mlp") and "diff=10.0%" in lines[0] and lines[1].startswith("  FAIL  lenet") and "SKIP  gpt_nano" in lines[2]
    assert lines[3].startswith("  FAIL  mlp")                                # a NaN loss never passes
    assert validate_results([RunResult("z", "solo-0", 1, "cpu", 1, 1, 1, [1e-12])], [Baseline("z", "solo-0", 0.0)], 0.15)[0] == 1
    (tmp_path / "bad.json").write_text('{"not": "a list"}')
    with pytest.raises(ValueError, match="expected a JSON array"):
        load_baselines(str(tmp_path / "bad.json"))
    with pytest.raises(ValueError, match="cannot read"):
        load_baselines(str(tmp_path / "missing.json"))


def test_cli_saves_and_validates_baselines_and_answers_the_schema_probe(tmp_path, capsys):
    from ddp_bench.__main__ import main
    base = str(tmp_path / "b.json")
    common = ["--model", "mlp", "--mode", "solo-0", "--tiny", "--device", "cpu", "--baseline", base]
    assert main(common + ["--save-baseline"]) == 0
    assert json.load(open(base))[0]["model"] == "mlp"
    capsys.readouterr()
    assert main(common + ["--validate"]) == 0                               # same seed, same sizes: the same loss
    assert "validation: 1 passed, 0 failed" in capsys.readouterr().err
    assert main(common + ["--validate", "--lr-scale", "0.001", "--tolerance", "0.0001"]) == 1
    assert "FAIL  mlp" in capsys.readouterr().err
    assert main(common[:-2] + ["--validate", "--baseline", str(tmp_path / "none.json")]) == 2
    capsys.readouterr()
    with pytest.raises(SystemExit) as e:
        main(["--fdl-schema"])
    assert e.value.code == 0
    schema = json.loads(capsys.readouterr().out)
    assert schema["options"]["model"]["short"] == "m" and "all" in schema["options"]["mode"]["choices"] and schema["options"]["validate"]["type"] == "bool"
    assert schema["options"]["tolerance"]["default"] == 0.15 and schema["strict"] is True


# ---- timelines: saved with the results, analysed into the report -------------------------------------------------------
def _fake_timeline():
    samples = []
    for t in range(0, 6000, 100):
        busy0 = not (2000 <= t <= 3000)                        # GPU 0 idles for a second around a sync
        busy1 = not (4500 <= t <= 5300)                        # GPU 1 idles with nothing nearby
        samples.append({"t_ms": t, "cpu_percent": 10.0, "ram_used_bytes": 1 << 30,
                        "gpus": [{"index": 0, "util": 90.0 if busy0 else 1.0, "vram_used": 2 << 30}, {"index": 1, "util": 80.0 if busy1 else 0.0, "vram_used": 1 << 30}]})
    events = [{"t_ms": 0, "kind": "EpochStart", "epoch": 0}, {"t_ms": 1000, "kind": "SyncStart"}, {"t_ms": 1010, "kind": "SyncEnd", "duration_ms": 10.0},
              {"t_ms": 2100, "kind": "SyncStart"}, {"t_ms": 2130, "kind": "SyncEnd", "duration_ms": 30.0}, {"t_ms": 2200, "kind": "AnchorChanged", "from": 10, "to": 14},
              {"t_ms": 3500, "kind": "SyncStart"}, {"t_ms": 3520, "kind": "SyncEnd", "duration_ms": 20.0}, {"t_ms": 3600, "kind": "Throttle", "rank": 1},
              {"t_ms": 3700, "kind": "CpuAvgStart"}, {"t_ms": 3750, "kind": "CpuAvgEnd", "duration_ms": 50.0}, {"t_ms": 5900, "kind": "EpochEnd", "epoch": 0, "loss": 0.25}]
    return {"samples": samples, "events": events}


def test_timeline_analysis_counts_syncs_anchor_moves_and_classifies_idle_gaps(tmp_path):
    from ddp_bench import analyze as A
    a = A.analyze("mlp", "nccl-cadence", _fake_timeline())
    assert (a.sync_count, a.cpu_avg_count, a.throttle_count) == (3, 1, 1) and abs(a.avg_sync_ms - 20.0) < 1e-9 and a.avg_cpu_avg_ms == 50.0
    assert a.anchor_changes == [(10, 14)] and a.final_anchor == 14 and a.epoch_losses == [0.25]
    assert a.sync_interval_p50_ms == 1250.0 and 1385 <= a.sync_interval_p95_ms <= 1400
    assert 70 < a.gpu_mean_util[0] < 80 and a.gpu_peak_vram_mb[0] == 2048.0 and a.gpu_mean_vram_mb[1] == 1024.0
    gaps = {(g.gpu, g.start_ms, g.duration_ms, g.cause) for g in a.idle_gaps}
    assert gaps == {(0, 2000, 1000, "sync"), (1, 4500, 800, "unexplained")}
    assert a.idle_ms() == 1800 and a.idle_ms(0) == 1000 and a.idle_by_cause(0)["sync"] == 1000
    assert A.classify_gap(5500, 6200, _fake_timeline()["events"]) == "epoch boundary"
    assert A.classify_gap(3300, 3400, [{"t_ms": 3700, "kind": "CpuAvgStart"}]) == "cpu avg"
    short = {"samples": [{"t_ms": t, "gpus": [{"index": 0, "util": 0.0}]} for t in range(0, 400, 100)], "events": []}
    assert A.analyze("m", "solo-0", short).idle_gaps == []                  # shorter than half a second: not reported
    (tmp_path / "bad.json").write_text("[1, 2]")
    with pytest.raises(ValueError, match="not a timeline"):
        A.load_timeline(str(tmp_path / "bad.json"))
    assert A.empty_analysis("m", "x").sync_count == 0


def test_runs_save_timelines_and_the_report_has_the_summary_sections(tmp_path):
    from ddp_bench import analyze as A
    from ddp_bench.report import write_report
    out = str(tmp_path / "runs")
    opts = RunOptions(epochs=2, device="cpu", output_dir=out, tiny=True)
    for name in ("mlp", "logistic"):
        assert run(find_model(name), DdpMode.parse("solo-0"), opts) is not None
    assert A.discover_runs(out) == [("logistic", "solo-0"), ("mlp", "solo-0")]
    tl = A.load_timeline(os.path.join(out, "mlp__solo-0.timeline.json"))
    kinds = [e["kind"] for e in tl["events"]]
    assert kinds.count("EpochStart") == 2 and kinds.count("EpochEnd") == 2 and "loss" in tl["events"][-1]
    analysis = A.analyze_dir(out)[("mlp", "solo-0")]
    assert len(analysis.epoch_losses) == 2
    json.dump(_fake_timeline(), open(os.path.join(out, "mlp__solo-0.timeline.json"), "w"))       # a multi-GPU run's timeline in its place
    text = write_report(out)
    for heading in ("## Best mode per model", "## Convergence quality (loss ratio vs solo-0)", "## Speed-up vs solo-0", "## Per-epoch loss trajectory",
                    "## Timeline", "## GPU idle analysis", "### Idle time by cause"):
        assert heading in text, heading
    assert "| mlp | solo-0 | 3 | 20.00 | 1250 / " in text and "10 -> 14 (1 changes)" in text and "| mlp | solo-0 | 0 | 2.0 | 1.0 | sync |" in text
    assert "| mlp | 1.00 |" in text and "| logistic | 1.00x |" in text
