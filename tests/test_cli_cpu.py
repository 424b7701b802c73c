"""Command line: typed argument parsing + schema, manifest commands, overlays, built-ins."""
import json
import os
import subprocess
import sys
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
    assert build_shell_line(spec, rest) == "echo hello world"
    assert build_shell_line(spec, ["you", "two words"]) == "echo hello you 'two words' world"      # run + forwarded + append
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
    assert main(["--dry-run", "hello", "--", "there"]) == 0
    assert capsys.readouterr().out.strip() == "echo hello there world"
    assert main(["--dry-run", "hello", "there"]) == 2                      # extra arguments only after `--`
    assert "fdl hello -- there" in capsys.readouterr().err
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
    assert "Porting from floDl" in (tmp_path / ".fdl" / "skills" / "guide" / "SKILL.md").read_text()
    assert main(["libtorch", "info", "--json"]) == 0
    assert main(["libtorch", "path"]) == 0
    assert main(["install", "--check"]) == 0
    assert main(["setup"]) == 0
    out = capsys.readouterr().out
    assert "nvcc" in out and "ready:" in out and "lib_dir" in out


# ---- the three command kinds, docker, presets, schema cache, first-word overlays ---------------------------------
def _bench_project(tmp_path):
    """A root manifest with a docker run command and a path-kind sub-command whose entry is a script that answers
    `--fdl-schema` (the shape of the reference's `ddp-bench/` and `benchmarks/`)."""
    from textwrap import dedent
    (tmp_path / "fdl.yml").write_text(dedent("""\
        description: demo
        commands:
          test:
            description: Run the tests
            run: pytest -q
            append: -- --nocapture
            docker: dev
          lint:
            run: ruff check .
          suite:
        """))
    (tmp_path / "fdl.ci.yml").write_text("commands:\n  test:\n    run: pytest -q -x\n")
    sub = tmp_path / "suite"
    sub.mkdir()
    (sub / "tool.py").write_text(dedent("""\
        import json, sys
        if "--fdl-schema" in sys.argv:
            print(json.dumps({"options": {"model": {"type": "string", "short": "m", "description": "which model", "default": "all",
                                                     "choices": ["mlp", "resnet", "all"]},
                                          "epochs": {"type": "int", "description": "epochs"},
                                          "validate": {"type": "bool", "description": "check baselines"}}, "strict": True}))
            sys.exit(0)
        print("ARGS", " ".join(sys.argv[1:]))
        """))
    (sub / "fdl.yml").write_text(dedent(f"""\
        description: the suite
        entry: {sys.executable} tool.py
        training:
          epochs: 5
          seed: 42
        ddp:
          policy: cadence
        commands:
          quick:
            description: Fast smoke test
            training: {{epochs: 1}}
            options: {{model: mlp, validate: true, batches: null}}
          full:
            options: {{model: all}}
          helper:
            run: echo helper
        """))
    return str(tmp_path / "fdl.yml")


def test_run_kind_docker_wrap_forwarding_and_overlay_by_first_word(tmp_path, monkeypatch, capsys):
    from flodl_b200.cli.manifest import compose, resolve
    m = _bench_project(tmp_path)
    assert compose(resolve(m, ["test"])) == "docker compose run --rm dev bash -c 'pytest -q -- --nocapture'"
    assert compose(resolve(m, ["test", "--", "-k", "two words"])) == "docker compose run --rm dev bash -c 'pytest -q -k '\"'\"'two words'\"'\"' -- --nocapture'"
    assert compose(resolve(m, ["lint"])) == "ruff check ."
    with pytest.raises(Exception, match="fdl test -- -k x"):
        compose(resolve(m, ["test", "-k", "x"]))
    monkeypatch.chdir(tmp_path)
    assert main(["--dry-run", "ci", "test"]) == 0                            # first word names fdl.ci.yml
    assert "pytest -q -x -- --nocapture" in capsys.readouterr().out
    assert main(["config", "show", "ci"]) == 0 and "# fdl.ci.yml" in capsys.readouterr().out
    monkeypatch.setenv("FDL_ENV", "ci")
    assert main(["--dry-run", "test"]) == 0 and "-x" in capsys.readouterr().out
    monkeypatch.delenv("FDL_ENV")
    (tmp_path / "fdl.lint.yml").write_text("description: clash\n")
    assert main(["--dry-run", "lint"]) == 2 and "both a command and the overlay" in capsys.readouterr().err


def test_presets_merge_sections_and_become_flags(tmp_path, monkeypatch, capsys):
    from flodl_b200.cli.manifest import compose, config_to_args, resolve
    m = _bench_project(tmp_path)
    r = resolve(m, ["suite", "quick", "--report", "out"])
    assert (r.kind, r.name, r.rest) == ("preset", "quick", ["--report", "out"])
    line = compose(r)
    assert line.endswith("tool.py --policy cadence --epochs 1 --seed 42 --model mlp --validate --report out")
    assert compose(resolve(m, ["suite", "--model", "resnet"])).endswith("tool.py --policy cadence --epochs 5 --seed 42 --model resnet")
    assert compose(resolve(m, ["suite", "helper"])) == "echo helper"
    monkeypatch.chdir(tmp_path)
    assert main(["suite", "full"]) == 0                                       # really runs the entry
    args = config_to_args({"ddp": {"mode": "sync", "speed_hint": {"slow_rank": 1, "ratio": 0.5}, "partition_ratios": [0.7, 0.3], "timeline": True,
                                   "progressive": False},
                           "training": {"batches_per_epoch": 10, "lr": 0.1}, "output": {"dir": "runs/", "monitor": 3000},
                           "options": {"data_dir": "d", "list": False, "tags": ["a", "b"]}})
    assert args == ["--mode", "sync", "--progressive", "false", "--speed-hint", "1:0.5", "--partition-ratios", "0.7,0.3", "--timeline", "--batches", "10",
                    "--lr", "0.1", "--output", "runs/", "--monitor", "3000", "--data-dir", "d", "--tags", "a,b"]


def test_schema_probe_cache_validation_and_help(tmp_path, monkeypatch, capsys):
    from flodl_b200.cli.manifest import cache_path, command_help, compose, discover_caches, resolve
    m = _bench_project(tmp_path)
    sub = str(tmp_path / "suite")
    text = command_help(resolve(m, ["suite"]))                                # probes the script and caches the answer
    assert os.path.isfile(cache_path(sub, "suite"))
    assert "the suite" in text and "quick" in text and "Fast smoke test" in text and "helper" in text
    assert "-m, --model <string>" in text and "one of: mlp, resnet, all" in text and "default: all" in text and "--validate" in text
    assert [c["status"] for c in discover_caches(m)] == ["fresh"]
    assert "--epochs 1" in command_help(resolve(m, ["suite", "quick"]))
    bad = (tmp_path / "suite" / "fdl.yml").read_text().replace("model: mlp", "model: lenet")
    (tmp_path / "suite" / "fdl.yml").write_text(bad)
    with pytest.raises(Exception, match="not one of mlp, resnet, all"):
        compose(resolve(m, ["suite", "quick"]))
    (tmp_path / "suite" / "fdl.yml").write_text(bad.replace("model: lenet", "modle: mlp"))
    with pytest.raises(Exception, match="does not declare"):
        compose(resolve(m, ["suite", "quick"]))                               # strict schema: unknown option
    monkeypatch.chdir(tmp_path)
    assert main(["suite", "--help"]) == 0 and "Options:" in capsys.readouterr().out
    assert main(["test", "--help"]) == 0 and "fdl test -- <args>" in capsys.readouterr().out
    assert main(["schema", "list", "--json"]) == 0 and json.loads(capsys.readouterr().out)[0]["command"] == "suite"
    assert main(["schema", "clear"]) == 0 and "removed 1" in capsys.readouterr().out and not os.path.isfile(cache_path(sub, "suite"))
    assert main(["schema", "refresh", "suite"]) == 0 and "refreshed: suite" in capsys.readouterr().out
    os.remove(tmp_path / "suite" / "fdl.yml")
    (tmp_path / "suite" / "fdl.yml").write_text("commands:\n  x:\n    run: echo x\n")
    assert discover_caches(m)[0]["status"] == "orphan"


def test_manifest_load_time_checks_json_and_templates(tmp_path, monkeypatch, capsys):
    from flodl_b200.cli.manifest import adopt_template, list_envs
    (tmp_path / "a").mkdir()
    (tmp_path / "a" / "fdl.json").write_text(json.dumps({"commands": {"hi": {"run": "echo hi"}}}))
    spec, _, _ = resolve_command(str(tmp_path / "a" / "fdl.json"), ["hi"])
    assert spec["run"] == "echo hi"
    for body, needle in (("commands:\n  p:\n    path: ./x/\n    docker: dev\n", "`docker:` on command `p` needs `run:`"),
                         ("commands:\n  p:\n    options: {a: 1}\n    append: x\n", "`append:` on command `p` needs `run:`"),
                         ("commands:\n  p:\n    options: {a: 1}\n", "presets need an `entry:`"),
                         ("commands:\n  p: echo\n", "must be a mapping"),
                         ("commands:\n  p:\n    run: [a]\n", "must be a string")):
        (tmp_path / "fdl.yml").write_text(body)
        with pytest.raises(Exception) as e:
            load_manifest(str(tmp_path / "fdl.yml"))
        assert needle in str(e.value), body
    os.remove(tmp_path / "fdl.yml")
    (tmp_path / "fdl.yml.example").write_text("commands:\n  hi:\n    run: echo template\n")
    (tmp_path / "fdl.dev.yml").write_text("{}\n")
    assert list_envs(str(tmp_path / "fdl.yml.example")) == ["dev"]
    monkeypatch.chdir(tmp_path)
    assert main(["--dry-run", "hi"]) == 0 and "echo template" in capsys.readouterr().out
    assert os.path.isfile(tmp_path / "fdl.yml")                               # the template was copied for local edits
    assert adopt_template(str(tmp_path / "fdl.yml")) == str(tmp_path / "fdl.yml")


def test_completion_scripts_know_nested_commands_and_choices(tmp_path, monkeypatch, capsys):
    m = _bench_project(tmp_path)
    monkeypatch.chdir(tmp_path)
    assert main(["completions", "bash"]) == 0
    out = capsys.readouterr().out
    assert '" suite") COMPREPLY=($(compgen -W "full helper quick --epochs --model --validate"' in out
    assert '" suite|--model") COMPREPLY=($(compgen -W "mlp resnet all"' in out and '" suite quick|--model")' in out
    assert "complete -F _fdl fdl" in out and '" libtorch")' in out
    assert subprocess.run(["bash", "-n"], input=out, text=True).returncode == 0        # the script parses
    assert main(["completions", "zsh"]) == 0 and capsys.readouterr().out.startswith("#compdef fdl")
    assert main(["completions", "fish"]) == 0 and "-l model -x -a 'mlp resnet all'" in capsys.readouterr().out
    assert main(["completions", "tcsh"]) == 2
    capsys.readouterr()
    monkeypatch.setenv("HOME", str(tmp_path / "home"))
    monkeypatch.setenv("SHELL", "/usr/bin/fish")
    assert main(["autocomplete"]) == 0 and os.path.isfile(tmp_path / "home" / ".config" / "fish" / "completions" / "fdl.fish")


# ---- libtorch variants -------------------------------------------------------------------------------------------
def _fake_variant(root, name, archs="9.0 10.0", cuda="12.8"):
    from flodl_b200.cli import libtorch as lt
    vdir = os.path.join(root, "libtorch", name)
    os.makedirs(os.path.join(vdir, "lib"))
    lt.write_arch(vdir, "2.10.0", cuda, archs, "compiled" if name.startswith("builds/") else "precompiled")
    return vdir


def test_libtorch_variants_list_activate_info_remove(tmp_path, monkeypatch, capsys):
    from flodl_b200.cli import libtorch as lt
    monkeypatch.setenv("FLODL_HOME", str(tmp_path / "home"))
    monkeypatch.chdir(tmp_path)                                    # no fdl.yml here: variants live under $FLODL_HOME
    root = lt.root_dir(".")
    assert root == str(tmp_path / "home")
    _fake_variant(root, "precompiled/cu128")
    _fake_variant(root, "builds/sm61-sm120", "6.1 12.0")
    os.makedirs(os.path.join(root, "libtorch", "precompiled", "broken"))      # no lib/: not a variant
    names = [v["name"] for v in lt.list_variants(root)]
    assert names[0].startswith("wheel/") and names[1:] == ["precompiled/cu128", "builds/sm61-sm120"]
    assert lt.active_variant(root)["name"].startswith("wheel/")              # nothing activated yet: the wheel's
    assert main(["libtorch", "activate", "builds/sm61-sm120"]) == 0
    assert lt.read_active(root) == "builds/sm61-sm120"
    capsys.readouterr()
    assert main(["libtorch", "info"]) == 0
    out = capsys.readouterr().out
    assert "Active:   builds/sm61-sm120" in out and "Archs:    6.1 12.0" in out and "Source:   compiled" in out
    assert main(["libtorch", "list"]) == 0 and "builds/sm61-sm120 (active)" in capsys.readouterr().out
    assert main(["libtorch", "list", "--json"]) == 0
    rows = json.loads(capsys.readouterr().out)
    assert [r["active"] for r in rows] == [False, False, True]
    assert main(["libtorch", "path"]) == 0 and capsys.readouterr().out.strip().endswith("builds/sm61-sm120/lib")
    assert main(["libtorch", "activate", "nope"]) == 1 and "no variant `nope`" in capsys.readouterr().err
    assert main(["libtorch", "remove", "builds/sm61-sm120"]) == 0
    assert lt.read_active(root) is None and not os.path.isdir(os.path.join(root, "libtorch", "builds", "sm61-sm120"))
    assert main(["libtorch", "remove", names[0]]) == 1 and "pip" in capsys.readouterr().err
    assert main(["libtorch", "activate"]) == 0 and "precompiled/cu128" in capsys.readouterr().out
    assert lt.arch_compatible(10, 0, "9.0 10.0") and lt.arch_compatible(6, 1, "6.1;12.0") and not lt.arch_compatible(7, 5, "9.0 10.0")
    assert main(["libtorch", "frobnicate"]) == 2


def test_libtorch_download_plan_archive_install_and_build_plan(tmp_path, monkeypatch, capsys):
    import zipfile
    from flodl_b200.cli import libtorch as lt
    monkeypatch.setenv("FLODL_HOME", str(tmp_path / "home"))
    monkeypatch.chdir(tmp_path)
    root = lt.root_dir(".")
    assert lt.pick_variant([]) == "cpu" and lt.pick_variant(["10.0"]) == "cu128" and lt.pick_variant(["6.1", "12.0"]) == "cu126"
    assert lt.download_url("cu128") == f"https://download.pytorch.org/libtorch/cu128/libtorch-shared-with-deps-{lt.LIBTORCH_VERSION}%2Bcu128.zip"
    assert main(["libtorch", "download", "--cuda", "12.8", "--dry-run"]) == 0
    out = capsys.readouterr().out
    assert "precompiled/cu128" in out and "dry run" in out and not os.path.isdir(os.path.join(root, "libtorch"))
    assert main(["libtorch", "download", "--cuda", "11.8"]) == 1 and "12.6 or 12.8" in capsys.readouterr().err
    z = tmp_path / "lt.zip"
    with zipfile.ZipFile(z, "w") as f:
        f.writestr("libtorch/lib/libtorch.so", b"x")
        f.writestr("libtorch/include/torch/torch.h", b"y")
    vdir = str(tmp_path / "home" / "libtorch" / "precompiled" / "cpu")
    os.makedirs(vdir)
    lt.install_archive(str(z), vdir)
    assert os.path.isfile(os.path.join(vdir, "lib", "libtorch.so")) and os.path.isfile(os.path.join(vdir, "include", "torch", "torch.h"))
    with zipfile.ZipFile(z, "w") as f:
        f.writestr("libtorch/../../escape.txt", b"x")
    with pytest.raises(lt.LibtorchError, match="escapes"):
        lt.install_archive(str(z), vdir)
    assert lt.arch_dir_name("6.1;12.0") == "sm61-sm120"
    monkeypatch.setattr(lt.shutil, "which", lambda t: "/usr/bin/" + t if t != "docker" else None)
    plan = lt.build_plan(root, "9.0;10.0", 8, None)
    assert plan["backend"] == "native" and plan["output"].endswith("builds/sm90-sm100") and 'TORCH_CUDA_ARCH_LIST="9.0;10.0" MAX_JOBS=8' in plan["commands"][2]
    with pytest.raises(lt.LibtorchError, match="docker is not installed"):
        lt.build_plan(root, "9.0", 6, "docker")
    assert main(["libtorch", "build", "--archs", "10.0", "--dry-run"]) == 0 and "nothing built" in capsys.readouterr().out
    monkeypatch.setattr(lt, "detect_gpu_archs", lambda: [])
    assert main(["libtorch", "build", "--dry-run"]) == 1 and "no GPU detected" in capsys.readouterr().err
    monkeypatch.setattr(lt.shutil, "which", lambda t: "/usr/bin/" + t)
    calls = []
    plan = lt.build_plan(root, "10.0", 4, "docker")
    lt.build_docker(plan, run=lambda cmd: calls.append(cmd) or 0, capture=lambda cmd, text=True: "abc123\n")
    assert calls[0][:2] == ["docker", "build"] and "TORCH_CUDA_ARCH_LIST=10.0" in calls[0] and calls[1][:2] == ["docker", "cp"]
    assert calls[1][2] == "abc123:/opt/libtorch/." and calls[2] == ["docker", "rm", "abc123"]


def test_the_repositorys_own_manifests_resolve(capsys):
    """`fdl.yml.example` at the root and the sub-command manifests of `ddp_bench/` and `benchmarks/` load, their presets pass
    the entries' own schemas, and the composed lines are what the docs promise."""
    from flodl_b200.cli.manifest import compose, load_manifest as load, resolve
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "fdl.yml.example")
    man, _ = load(root)
    assert {"build", "test", "test-gpu", "bench", "ddp-bench", "bench-models"} <= set(man["commands"])
    assert compose(resolve(root, ["test", "--", "-k", "ddp"])) == 'python -m pytest tests -q -m "not gpu" -k ddp -x'
    for sub in ("ddp-bench", "bench-models"):
        sub_man = resolve(root, [sub]).manifest
        for preset in sub_man["commands"]:
            line = compose(resolve(root, [sub, preset]))                     # raises if a preset sets an undeclared option
            assert line.startswith("PYTHONPATH=.. python -m ")
    assert compose(resolve(root, ["ddp-bench", "quick"])).endswith("--epochs 1 --seed 42 --output runs/ --model mlp --mode solo-0 --tiny")
    assert "--output" not in compose(resolve(root, ["ddp-bench", "report"]))
    assert compose(resolve(root, ["flodl-hf", "verify-export", "--", "out", "--no-hub-source"])).endswith("flodl_b200.hf.verify_export out --no-hub-source")
    assert compose(resolve(root, ["flodl-hf", "export", "--", "--hub", "bert-base-uncased", "--out", "x"])).endswith("export_tool --hub bert-base-uncased --out x")


def test_init_modes_and_add_flodl_hf(tmp_path, monkeypatch, capsys):
    from flodl_b200.cli.manifest import compose, resolve
    monkeypatch.chdir(tmp_path)
    assert main(["init", "dk", "--docker", "--with-hf"]) == 0
    files = {os.path.relpath(os.path.join(d, f), tmp_path / "dk") for d, _, fs in os.walk(tmp_path / "dk") for f in fs}
    assert {"train.py", "fdl.yml.example", ".gitignore", "README.md", "requirements.txt", "Dockerfile", "Dockerfile.cuda", "docker-compose.yml",
            "flodl-hf/classify.py", "flodl-hf/fill_mask.py", "flodl-hf/fdl.yml", "flodl-hf/README.md"} == files
    m = str(tmp_path / "dk" / "fdl.yml.example")
    assert compose(resolve(m, ["train"])) == "docker compose run --rm dev bash -c 'python train.py'"
    assert compose(resolve(m, ["cuda-train"])).startswith("docker compose run --rm cuda ")
    assert compose(resolve(m, ["flodl-hf", "classify"])) == "docker compose run --rm dev bash -c 'python classify.py'"
    import yaml
    assert set(yaml.safe_load(open(tmp_path / "dk" / "docker-compose.yml"))["services"]) == {"dev", "cuda"}
    for script in ("train.py", "flodl-hf/classify.py", "flodl-hf/fill_mask.py"):
        compile(open(tmp_path / "dk" / script).read(), script, "exec")
    assert main(["init", "nt", "--native"]) == 0
    files = set(os.listdir(tmp_path / "nt"))
    assert "Dockerfile" not in files and "docker-compose.yml" not in files and "flodl-hf" not in files
    m = str(tmp_path / "nt" / "fdl.yml.example")
    assert compose(resolve(m, ["train"])) == "python train.py" and "shell" not in open(m).read()
    assert main(["init", "x", "--docker", "--native"]) == 2
    capsys.readouterr()
    monkeypatch.chdir(tmp_path / "nt")
    assert main(["add", "hf"]) == 0 and "created flodl-hf/classify.py" in capsys.readouterr().out
    assert "docker:" not in open(tmp_path / "nt" / "flodl-hf" / "fdl.yml").read()         # native project: no docker lines
    assert main(["add", "flodl-hf"]) == 1 and "already exists" in capsys.readouterr().err
    (tmp_path / "bare").mkdir()
    monkeypatch.chdir(tmp_path / "bare")
    assert main(["add", "flodl-hf"]) == 1 and "initialised flodl project" in capsys.readouterr().err


def test_scaffolded_training_script_runs(tmp_path):
    from flodl_b200.cli.scaffold import TRAIN
    script = tmp_path / "train.py"
    script.write_text(TRAIN.replace("range(200)", "range(3)"))
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, str(script)], cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert os.path.isfile(tmp_path / "model.fdl") and out.stdout.startswith("0 ")


def test_api_ref_is_structured_by_section_with_constructors_and_builder_methods(capsys):
    from flodl_b200.cli.main import api_entries
    rows = {r["name"]: r for r in api_entries()}
    conv = rows["Conv2d"]
    assert conv["kind"] == "class" and conv["file"].endswith("nn/layers.py") and "Module" in conv["implements"]
    assert any(c.startswith("Conv2d.configure(") for c in conv["constructors"]) and conv["constructors"][0].startswith("Conv2d(in_channels")
    pool = rows["AvgPool2d"]
    assert {b.split("(")[0] for b in pool["builder"]} >= {".padding", ".ceil_mode", ".count_include_pad"} and ".name" not in {b.split("(")[0] for b in pool["builder"]}
    assert any(c.startswith("AvgPool2d.with_stride(") for c in pool["constructors"])
    fb = rows["FlowBuilder"]
    assert {".through", ".also", ".tag", ".using"} <= {b.split("(")[0] for b in fb["builder"]} and any(m.startswith(".build(") for m in fb["methods"])
    assert rows["gt_scalar"]["kind"] == "function" and rows["gt_scalar"]["section"] == "Tensor operations"
    assert rows["AutoModelForQuestionAnswering"]["section"] == "Hugging Face"
    assert main(["api-ref"]) == 0
    text = capsys.readouterr().out
    assert text.startswith("flodl_b200 API reference v") and "## Modules (nn)" in text and "### Linear" in text and "  constructors:" in text and "  builder:" in text


def test_skill_list_show_and_install_per_tool(tmp_path, monkeypatch, capsys):
    monkeypatch.chdir(tmp_path)
    assert main(["skill", "list"]) == 0
    out = capsys.readouterr().out
    assert "port" in out and "guide" in out and "tools detected here: none" in out
    assert main(["skill", "show", "port"]) == 0 and "FlowBuilder" in capsys.readouterr().out
    assert main(["skill", "show", "nope"]) == 2
    (tmp_path / ".claude").mkdir()
    (tmp_path / ".cursorrules").write_text("my own rule\n")
    capsys.readouterr()
    assert main(["skill", "install", "--skill", "port"]) == 0            # both tools detected: both get it
    assert "Port a PyTorch training script" in (tmp_path / ".claude" / "skills" / "port" / "SKILL.md").read_text()
    rules = (tmp_path / ".cursorrules").read_text()
    assert rules.startswith("my own rule") and rules.count("# --- flodl_b200 skill: port ---") == 1
    assert main(["skill", "install", "--tool", "cursor", "--skill", "port"]) == 0
    rules = (tmp_path / ".cursorrules").read_text()
    assert rules.count("# --- flodl_b200 skill: port ---") == 1 and rules.startswith("my own rule")      # replaced, not duplicated
    assert main(["skill", "install", "--tool", "generic"]) == 0
    assert (tmp_path / ".fdl" / "skills" / "port" / "SKILL.md").is_file() and (tmp_path / ".fdl" / "skills" / "guide" / "SKILL.md").is_file()
    assert main(["skill", "install", "--tool", "emacs"]) == 2 and main(["skill", "install", "--skill", "x"]) == 2
    assert main(["skill", "list"]) == 0 and "claude, cursor" in capsys.readouterr().out


# ---- update check: inert without a feed, daily, silent on failure ------------------------------------------------------
def test_update_check_switches_versions_and_daily_cache(tmp_path):
    from flodl_b200.cli import update_check as U
    cfgp = str(tmp_path / "flodl" / "config.json")
    feed = {"FLODL_B200_UPDATE_URL": "http://feed.invalid/latest.json"}
    calls = []

    def fetch(url):
        calls.append(url)
        return "0.3.0"
    none = str(tmp_path / "no-dockerenv")
    assert U.check("0.1.0", 1e9, cfgp, fetch, {}, none) == [] and calls == []                          # no feed configured: nothing fetched
    for env in ({**feed, "FDL_NO_UPDATE_CHECK": "1"}, {**feed, "CI": "true"}):
        assert U.check("0.1.0", 1e9, cfgp, fetch, env, none) == [] and calls == []
    (tmp_path / "dockerenv").write_text("")
    assert U.check("0.1.0", 1e9, cfgp, fetch, feed, str(tmp_path / "dockerenv")) == [] and calls == []
    lines = U.check("0.1.0", 1e9, cfgp, fetch, feed, none)
    assert len(calls) == 1 and "once a day" in lines[0] and "0.3.0 is available (this is 0.1.0)" in lines[1]
    lines = U.check("0.1.0", 1e9 + 3600, cfgp, fetch, feed, none)                                        # an hour later: remembered, no probe, no note
    assert len(calls) == 1 and len(lines) == 1 and "0.3.0" in lines[0]
    assert U.check("0.3.0", 1e9 + 7200, cfgp, fetch, feed, none) == []                                   # up to date: silent
    U.check("0.1.0", 1e9 + U.DAY_S + 1, cfgp, lambda url: calls.append(url), feed, none)                 # a day later: probes again; a failed probe is silent
    assert len(calls) == 2 and U.load_config(cfgp)["update_check"]["latest_known"]["flodl_b200"] == "0.3.0"
    cfg = U.load_config(cfgp)
    cfg["update_check"]["enabled"] = False
    U.save_config(cfg, cfgp)
    assert U.check("0.1.0", 1e9 + 3 * U.DAY_S, cfgp, fetch, feed, none) == [] and len(calls) == 2
    assert U.max_stable(["0.5.2", "0.6.0-rc1", "v0.5.10", "junk"]) == "0.5.10" and U.parse_version("1.2.0b1") is None and U.parse_version("1.2") == (1, 2, 0)


def test_update_check_reads_a_feed_and_never_disturbs_the_command(tmp_path, monkeypatch, capsys):
    import functools, http.server, threading
    from flodl_b200.cli import update_check as U
    (tmp_path / "www").mkdir()
    (tmp_path / "www" / "latest.json").write_text(json.dumps({"versions": ["9.0.0", "9.1.0-beta", "8.4.1"]}))

    class Quiet(http.server.SimpleHTTPRequestHandler):
        def log_message(self, *a): pass
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), functools.partial(Quiet, directory=str(tmp_path / "www")))
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        url = f"http://127.0.0.1:{srv.server_address[1]}/latest.json"
        assert U.fetch_latest(url) == "9.0.0" and U.fetch_latest(url.replace("latest", "missing")) is None
        monkeypatch.setenv("XDG_CONFIG_HOME", str(tmp_path / "cfg"))
        monkeypatch.setenv("FLODL_B200_UPDATE_URL", url)
        monkeypatch.delenv("CI", raising=False)
        monkeypatch.delenv("FDL_NO_UPDATE_CHECK", raising=False)
        monkeypatch.setattr(U.os.path, "exists", lambda p, _e=os.path.exists: False if p == "/.dockerenv" else _e(p))
        monkeypatch.chdir(tmp_path)
        assert main(["skill", "list"]) == 0
        err = capsys.readouterr().err
        assert "9.0.0 is available" in err and os.path.isfile(tmp_path / "cfg" / "flodl" / "config.json")
    finally:
        srv.shutdown()


def test_help_describes_a_sub_project_by_its_own_manifest(tmp_path, monkeypatch, capsys):
    (tmp_path / "fdl.yml").write_text("commands:\n  tools:\n  other:\n    path: elsewhere\n  hello:\n    run: echo hi\n    description: says hi\n")
    (tmp_path / "tools").mkdir()
    (tmp_path / "tools" / "fdl.yml").write_text("description: the tool box\nentry: python tool.py\n")
    (tmp_path / "elsewhere").mkdir()
    (tmp_path / "elsewhere" / "fdl.yml").write_text("description: lives elsewhere\nentry: python x.py\n")
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("FDL_NO_UPDATE_CHECK", "1")
    assert main(["--help"]) == 0
    out = capsys.readouterr().out
    assert "the tool box" in out and "lives elsewhere" in out and "says hi" in out
