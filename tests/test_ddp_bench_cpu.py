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
