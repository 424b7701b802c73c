"""Command line: typed argument parsing + schema, manifest commands, overlays, built-ins."""
import json
import os
from dataclasses import dataclass
from typing import List, Optional

import pytest

from flodl_b200.cli import REQUIRED, ArgError, FdlArgs, arg, deep_merge, load_manifest, main, resolve_command
from flodl_b200.cli.manifest import build_shell_line


@dataclass
class TrainArgs(FdlArgs):
    """Train a model."""
    data: str = arg(help="dataset directory", positional=True)
    epochs: int = arg(10, help="number of epochs", short="e")
    lr: float = arg(1e-3, help="learning rate")
    model: str = arg("mlp", help="model name", choices=["mlp", "resnet"])
    resume: bool = arg(False, help="resume from the last checkpoint")
    tags: List[str] = arg([], help="free-form tags")
    seed: Optional[int] = arg(None, help="random seed", env="TRAIN_SEED")


def test_typed_args_parse_and_defaults(monkeypatch):
    a = TrainArgs.parse(["/data", "-e", "3", "--lr=0.5", "--model", "resnet", "--resume", "--tags", "a", "--tags", "b"])
    assert (a.data, a.epochs, a.lr, a.model, a.resume, a.tags, a.seed) == ("/data", 3, 0.5, "resnet", True, ["a", "b"], None)
    b = TrainArgs.parse(["/d"])
    assert (b.epochs, b.lr, b.model, b.resume, b.tags) == (10, 1e-3, "mlp", False, [])
    monkeypatch.setenv("TRAIN_SEED", "7")
    assert TrainArgs.parse(["/d"]).seed == 7 and TrainArgs.parse(["/d", "--seed", "9"]).seed == 9
    assert TrainArgs.parse(["/d", "--no-resume"]).resume is False


@pytest.mark.parametrize("argv,needle", [([], "missing required"), (["/d", "--epochs", "x"], "invalid value"), (["/d", "--model", "gpt"], "not one of"),
                                         (["/d", "--nope"], "unknown option"), (["/d", "--epochs"], "needs a value"), (["/d", "extra"], "unexpected")])
def test_typed_args_errors(argv, needle):
    with pytest.raises(ArgError) as e:
        TrainArgs.parse(argv)
    assert needle in str(e.value)


def test_schema_and_help(capsys):
    sc = TrainArgs.schema()
    by = {a["name"]: a for a in sc["args"]}
    assert sc["description"] == "Train a model." and by["epochs"]["type"] == "integer" and by["epochs"]["short"] == "e"
    assert by["data"]["positional"] and by["data"]["required"] and by["tags"]["list"] and by["model"]["choices"] == ["mlp", "resnet"]
    assert TrainArgs.parse(["--fdl-schema"], exit_on_help=False) is None
    assert json.loads(capsys.readouterr().out)["command"] == "TrainArgs"
    text = TrainArgs.help_text("train")
    assert "usage: train [options] <data>" in text and "-e, --epochs <integer>" in text and "default 10" in text and "--fdl-schema" in text


def _project(tmp_path):
    (tmp_path / "fdl.yml").write_text("""
description: demo
commands:
  hello:
    description: say hello
    run: echo hello
    append: world
  sub:
  bench:
    path: ./benchmarks/
settings:
  device: cpu
  opts:
    a: 1
    b: 2
""")
    (tmp_path / "fdl.gpu.yml").write_text("settings:\n  device: cuda\n  opts:\n    b: 3\n")
    os.makedirs(tmp_path / "sub")
    (tmp_path / "sub" / "fdl.yml").write_text("commands:\n  inner:\n    run: echo inner\n")
    os.makedirs(tmp_path / "benchmarks")
    (tmp_path / "benchmarks" / "fdl.yml").write_text("commands:\n  quick:\n    run: echo quick\n")
    return str(tmp_path / "fdl.yml")


def test_manifest_commands_and_subcommands(tmp_path):
    m = _project(tmp_path)
    spec, rest, cwd = resolve_command(m, ["hello"])
    assert build_shell_line(spec, rest) == "echo hello world" and build_shell_line(spec, ["you", "two words"]) == "echo hello you 'two words'"
    spec, rest, cwd = resolve_command(m, ["sub", "inner", "x"])
    assert spec["run"] == "echo inner" and rest == ["x"] and cwd.endswith("sub")
    spec, _, cwd = resolve_command(m, ["bench", "quick"])
    assert spec["run"] == "echo quick" and cwd.endswith("benchmarks")
    with pytest.raises(Exception) as e:
        resolve_command(m, ["nope"])
    assert "available" in str(e.value)


def test_overlay_deep_merge_keeps_origins(tmp_path):
    m = _project(tmp_path)
    man, origin = load_manifest(m, "gpu")
    assert man["settings"] == {"device": "cuda", "opts": {"a": 1, "b": 3}}
    assert origin["settings.device"] == "fdl.gpu.yml" and origin["settings.opts.a"] == "fdl.yml" and origin["settings.opts.b"] == "fdl.gpu.yml"
    with pytest.raises(Exception):
        load_manifest(m, "missing")
    o = {}
    assert deep_merge({"a": {"x": 1}}, {"a": {"y": 2}, "b": 3}, o, "", "over") == {"a": {"x": 1, "y": 2}, "b": 3}


def test_main_dispatch(tmp_path, monkeypatch, capsys):
    _project(tmp_path)
    monkeypatch.chdir(tmp_path)
    assert main(["--dry-run", "hello", "there"]) == 0
    assert capsys.readouterr().out.strip() == "echo hello there"
    assert main(["hello"]) == 0
    assert main(["--env", "gpu", "config", "show"]) == 0
    out = capsys.readouterr().out
    assert "device: 'cuda'" in out and "# fdl.gpu.yml" in out
    assert main([]) == 0 and "say hello" in capsys.readouterr().out
    assert main(["completions", "bash"]) == 0 and "hello" in capsys.readouterr().out
    assert main(["schema", "bench"]) == 0 and json.loads(capsys.readouterr().out)["command"] == "BenchArgs"
    assert main(["definitely-not-a-command"]) == 2
    assert main(["diagnose", "--json"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert "python" in info and "native_library" in info
    assert main(["init", "proj"]) == 0 and os.path.isfile(tmp_path / "proj" / "train.py")
    assert main(["init", "proj"]) == 1


def test_api_ref_lists_public_names(capsys):
    assert main(["api-ref", "--json"]) == 0
    names = {r["name"] for r in json.loads(capsys.readouterr().out)}
    assert {"FlowBuilder", "Trainer", "Adam", "DataLoader", "CpuWorker", "record_scalar"} <= names


def test_setup_install_add_libtorch_skill(tmp_path, capsys):
    from flodl_b200.cli.main import main
    assert main(["add", str(tmp_path), "--playground"]) == 0
    for f in ("train.py", "fdl.yml", "playground.py"):
        assert (tmp_path / f).exists()
    (tmp_path / "train.py").write_text("# mine")
    assert main(["add", str(tmp_path)]) == 0                      # existing files are kept
    assert (tmp_path / "train.py").read_text() == "# mine"
    assert main(["skill", "install", str(tmp_path)]) == 0
    assert "Porting from floDl" in (tmp_path / ".fdl" / "skills" / "flodl_b200" / "SKILL.md").read_text()
    assert main(["libtorch", "info", "--json"]) == 0
    assert main(["libtorch", "path"]) == 0
    assert main(["install", "--check"]) == 0
    assert main(["setup"]) == 0
    out = capsys.readouterr().out
    assert "nvcc" in out and "ready:" in out and "lib_dir" in out
