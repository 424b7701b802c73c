from __future__ import annotations

import inspect
import re
import json
import os
import subprocess
import sys
from dataclasses import dataclass
from typing import List, Optional

from .args import ArgError, FdlArgs, arg
from .manifest import ManifestError, adopt_template, command_kind, env_from_first_word, find_manifest, load_manifest, manifest_in, run_command

BUILTINS = ["diagnose", "setup", "install", "libtorch", "build", "bench", "export-hf", "api-ref", "schema", "completions", "autocomplete", "config", "init",
            "add", "skill", "help"]


# ---- diagnose ---------------------------------------------------------------------------------------
def diagnose(as_json: bool = False) -> int:
    """Environment report: interpreter, torch, CUDA toolchain, GPUs, native library, NCCL."""
    import platform
    import shutil
    info = {"python": platform.python_version(), "platform": platform.platform()}
    try:
        import torch
        info["torch"] = torch.__version__
        info["torch_cuda"] = torch.version.cuda
        info["cuda_available"] = torch.cuda.is_available()
        info["gpus"] = []
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                p = torch.cuda.get_device_properties(i)
                info["gpus"].append({"index": i, "name": p.name, "sm": f"{p.major}{p.minor}", "memory_gib": round(p.total_memory / 2 ** 30, 1),
                                     "sms": p.multi_processor_count})
        try:
            info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
        except Exception:
            info["nccl"] = None
    except Exception as e:
        info["torch"] = f"unavailable: {e}"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    try:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
        info["nvcc"] = out.strip().splitlines()[-1] if out else None
    except Exception:
        info["nvcc"] = None
    try:
        from .. import _build, _ext
        info["native_library"] = {"path": str(_build.TARGET), "built": not _build.needs_build(), "loads": _ext.available()}
    except Exception as e:
        info["native_library"] = {"error": repr(e)}
    if as_json:
        print(json.dumps(info, indent=2))
    else:
        for k, v in info.items():
            if k == "gpus":
                for g in v:
                    print(f"  gpu {g['index']}: {g['name']} sm_{g['sm']} {g['memory_gib']} GiB {g['sms']} SMs")
            else:
                print(f"  {k}: {v}")
    return 0


# ---- api-ref ----------------------------------------------------------------------------------------
_API_SECTIONS = (("Tensors and devices", "flodl_b200.tensor"), ("Tensor operations", "flodl_b200.tensor_ops"), ("Tensor operations (nn, conversion, optimizer primitives)", "flodl_b200.tensor_nn_ops"),
                 ("Autograd", "flodl_b200.autograd"), ("Modules (nn)", "flodl_b200.nn"), ("Graph builder", "flodl_b200.graph"), ("Data", "flodl_b200.data"),
                 ("Monitor", "flodl_b200.monitor"), ("Synchronous DDP", "flodl_b200.parallel.ddp"), ("Training engine", "flodl_b200.parallel.engine"),
                 ("Collectives and streams", "flodl_b200.parallel.comm"), ("Asynchronous DDP", "flodl_b200.parallel.ddp_run"),
                 ("Hugging Face", "flodl_b200.hf"), ("Command line helpers", "flodl_b200.cli"), ("Other names of the package root", "flodl_b200"))
_CTOR_NAMES = ("new", "on_device", "configure", "builder", "with_groups", "no_bias", "from_shared_weight", "from_pretrained", "from_pretrained_on_device",
               "from_dataset", "from_batch_dataset", "from_json_str", "from_file", "from_config", "seed")


def _sig(obj) -> str:
    try:
        return str(inspect.signature(obj))
    except (TypeError, ValueError):
        return "(...)"


def _first_line(obj) -> str:
    doc = (getattr(obj, "__doc__", None) or "").strip().splitlines()          # the object's own text, not an inherited one
    return doc[0].strip() if doc else ""


def api_entries() -> List[dict]:
    """The public surface, section by section: every class with the file it lives in, its constructors (`X(...)` and the
    floDl spellings `new`, `on_device`, `configure`, ...), its builder-style methods (those that return the object they are
    called on) and its other public methods; every public function with its signature."""
    import importlib
    out, seen = [], set()
    for title, modname in _API_SECTIONS:
        mod = importlib.import_module(modname)
        names = sorted(n for n in dir(mod) if not n.startswith("_"))
        for name in names:
            obj = getattr(mod, name)
            if inspect.ismodule(obj) or id(obj) in seen or not callable(obj):
                continue
            if not str(getattr(obj, "__module__", "")).startswith("flodl_b200"):
                continue
            seen.add(id(obj))
            try:
                file = os.path.relpath(inspect.getsourcefile(obj), _repo_root())
            except (TypeError, ValueError):
                file = ""
            if not inspect.isclass(obj):
                out.append({"section": title, "kind": "function", "name": name, "signature": _sig(obj), "doc": _first_line(obj), "file": file})
                continue
            ctors, builders, methods = [f"{name}{_sig(obj)}"], [], []
            members = {}
            for klass in reversed([k for k in obj.__mro__ if k.__module__.startswith("flodl_b200") and k.__name__ != "Module"] or [obj]):
                members.update(vars(klass))                  # own definitions win over the intermediate bases'
            for m, fn in sorted(members.items()):
                if m.startswith("_"):
                    continue
                raw = fn.__func__ if isinstance(fn, (classmethod, staticmethod)) else fn
                if not callable(raw):
                    continue
                sig = _sig(getattr(obj, m))
                if isinstance(fn, (classmethod, staticmethod)) and (m in _CTOR_NAMES or m.startswith(("with_", "from_"))):
                    ctors.append(f"{name}.{m}{sig}")
                    continue
                try:
                    src = inspect.getsource(raw)
                except (OSError, TypeError):
                    src = ""
                returns = re.findall(r"\breturn\b[^\n]*", src)
                fluent = bool(returns) and all(re.fullmatch(r"return self\s*(#.*)?", r.strip()) for r in returns)
                (builders if fluent else methods).append(f".{m}{sig}")
            bases = [b.__name__ for b in obj.__mro__[1:] if b.__module__.startswith("flodl_b200")]
            out.append({"section": title, "kind": "class", "name": name, "doc": _first_line(obj), "file": file, "implements": bases,
                        "constructors": ctors, "builder": builders, "methods": methods})
    return out


def api_ref(as_json: bool = False) -> int:
    """`api-ref [--json]`: the structured API reference (for people and for porting tools)."""
    import flodl_b200 as pkg
    rows = api_entries()
    if as_json:
        print(json.dumps(rows, indent=1))
        return 0
    print(f"flodl_b200 API reference v{pkg.__version__}\n" + "=" * 40)
    section = None
    for r in rows:
        if r["section"] != section:
            section = r["section"]
            print(f"\n## {section}\n")
        if r["kind"] == "function":
            print(f"  {r['name']}{r['signature']}" + (f"    # {r['doc']}" if r["doc"] else ""))
            continue
        impl = f"  (implements: {', '.join(r['implements'])})" if r["implements"] else ""
        print(f"### {r['name']}{impl}")
        if r["doc"]:
            print(f"  {r['doc']}")
        print(f"  file: {r['file']}")
        print("  constructors:")
        for c in r["constructors"]:
            print(f"    {c}")
        if r["builder"]:
            print("  builder:\n    " + "  ".join(b.split("(")[0] + "()" for b in r["builder"]))
        if r["methods"]:
            print("  methods:")
            for m in r["methods"]:
                print(f"    {m}")
    return 0


# ---- typed commands -----------------------------------------------------------------------------------
@dataclass
class BenchArgs(FdlArgs):
    """Run the headline training benchmark (bench.py) on N GPUs of this node."""
    gpus: int = arg(1, help="number of GPUs", short="g")
    steps: int = arg(20, help="timed steps")
    warmup: int = arg(5, help="warm-up steps")
    model: str = arg("bert-base", help="which configuration", choices=["bert-base", "resnet20", "lm"])
    impl: str = arg("ours", help="implementation arm", choices=["ours", "twin", "reference"])


@dataclass
class ExportArgs(FdlArgs):
    """Export a `.fdl` checkpoint (with its config sidecar) as a HuggingFace model directory."""
    checkpoint: str = arg(help="path to the .fdl file", positional=True)
    out: str = arg("hf_export", help="output directory", short="o")


@dataclass
class InitArgs(FdlArgs):
    """Scaffold a small training project that uses this package."""
    name: str = arg(help="project directory to create", positional=True)
    docker: bool = arg(False, help="commands run inside docker compose services (Dockerfile, Dockerfile.cuda, docker-compose.yml)")
    native: bool = arg(False, help="no docker files; commands run on the host")
    with_hf: bool = arg(False, help="also scaffold the flodl-hf playground")


def _repo_root() -> str:
    return os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def bench(argv: List[str]) -> int:
    a = BenchArgs.parse(argv, "fdl bench")
    script = os.path.join(_repo_root(), "bench.py")
    tail = ["--gpus", str(a.gpus), "--steps", str(a.steps), "--warmup", str(a.warmup), "--model", a.model, "--impl", a.impl]
    if a.gpus > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", "29511", script] + tail
    else:
        cmd = [sys.executable, script] + tail
    return subprocess.call(cmd)


def export_hf(argv: List[str]) -> int:
    a = ExportArgs.parse(argv, "fdl export-hf")
    from ..hf import export_checkpoint
    export_checkpoint(a.checkpoint, a.out)
    print(f"wrote {a.out}/model.safetensors and {a.out}/config.json")
    return 0


def init(argv: List[str]) -> int:
    from .scaffold import project_files, write_files
    a = InitArgs.parse(argv, "fdl init")
    if a.docker and a.native:
        print("fdl init: --docker and --native exclude each other", file=sys.stderr)
        return 2
    if os.path.exists(a.name):
        print(f"fdl init: {a.name} already exists", file=sys.stderr)
        return 1
    import shutil
    mode = "docker" if a.docker else "native" if a.native else ("docker" if shutil.which("docker") else "native")
    written = write_files(a.name, project_files(os.path.basename(os.path.normpath(a.name)), mode, a.with_hf))
    print(f"created {a.name}/ ({mode} mode): " + ", ".join(sorted(written)))
    return 0


def completion_script(shell: str, manifest: Optional[str]) -> str:
    """A completion script that knows the built-in commands, the project's commands of all three kinds with their
    nested entries, and the values of options declared with `choices:`."""
    from .manifest import completion_tree, flatten_completions
    tree = completion_tree(manifest) if manifest else {"words": {}, "flags": {}}
    for b in BUILTINS:
        tree["words"].setdefault(b, {"words": {}, "flags": {}})
    tree["words"]["libtorch"]["words"] = {k: {"words": {}, "flags": {}} for k in ("info", "list", "path", "activate", "download", "build", "remove")}
    tree["words"]["schema"]["words"] = {k: {"words": {}, "flags": {}} for k in ("list", "clear", "refresh", "bench", "export-hf", "init")}
    tree["words"]["skill"]["words"] = {k: {"words": {}, "flags": {}} for k in ("list", "show", "install")}
    tree["words"]["completions"]["words"] = {k: {"words": {}, "flags": {}} for k in ("bash", "zsh", "fish")}
    tree["words"]["config"]["words"] = {"show": {"words": {}, "flags": {}}}
    rows = flatten_completions(tree)
    if shell == "fish":
        lines = []
        for path, words, choices in rows:
            parts = path.split()
            cond = "__fish_use_subcommand" if not parts else "__fish_seen_subcommand_from " + parts[-1]
            for w in words:
                if w.startswith("--"):
                    vals = choices.get(w)
                    lines.append(f"complete -c fdl -f -n '{cond}' -l {w[2:]}" + (f" -x -a '{' '.join(vals)}'" if vals else ""))
                else:
                    lines.append(f"complete -c fdl -f -n '{cond}' -a {w}")
        return "\n".join(lines)
    cases, value_cases = [], []
    for path, words, choices in rows:
        cases.append(f'    "{path}") COMPREPLY=($(compgen -W "{" ".join(words)}" -- "$cur"));;')
        for flag, vals in choices.items():
            value_cases.append(f'    "{path}|{flag}") COMPREPLY=($(compgen -W "{" ".join(vals)}" -- "$cur")); return;;')
    body = "\n".join([
        "_fdl() {",
        "  local cur prev path i w",
        '  cur="${COMP_WORDS[COMP_CWORD]}"; prev="${COMP_WORDS[COMP_CWORD-1]}"; path=""',
        "  for ((i=1; i<COMP_CWORD; i++)); do",
        '    w="${COMP_WORDS[i]}"',
        '    case "$w" in -*) ;; *) case "${COMP_WORDS[i-1]}" in --*) ;; *) path="$path $w";; esac;; esac',
        "  done",
        '  case "$path|$prev" in'] + value_cases + ["  esac", '  case "$path" in'] + cases + ["  esac", "}"])
    if shell == "zsh":
        return "#compdef fdl\nautoload -U +X bashcompinit && bashcompinit\n" + body + "\ncomplete -F _fdl fdl"
    return body + "\ncomplete -F _fdl fdl"


def completions(shell: str, manifest: Optional[str]) -> int:
    if shell not in ("bash", "zsh", "fish"):
        print(f"fdl completions: unknown shell {shell!r} (bash, zsh, fish)", file=sys.stderr)
        return 2
    print(completion_script(shell, manifest))
    return 0


def autocomplete(manifest: Optional[str]) -> int:
    """Detect the login shell and install the completion script where that shell looks for it."""
    shell = os.path.basename(os.environ.get("SHELL", "bash"))
    shell = shell if shell in ("bash", "zsh", "fish") else "bash"
    home = os.path.expanduser("~")
    dst = {"bash": os.path.join(home, ".local", "share", "bash-completion", "completions", "fdl"),
           "zsh": os.path.join(home, ".zfunc", "_fdl"),
           "fish": os.path.join(home, ".config", "fish", "completions", "fdl.fish")}[shell]
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    with open(dst, "w") as f:
        f.write(completion_script(shell, manifest) + "\n")
    print(f"installed {shell} completions to {dst}" + ("; add `fpath+=~/.zfunc` before compinit in ~/.zshrc" if shell == "zsh" else ""))
    return 0


def schema(argv: List[str], manifest: Optional[str] = None, env: Optional[str] = None) -> int:
    """`schema [bench|export-hf|init]`: the built-in commands' argument schemas. `schema list [--json] | clear [cmd] |
    refresh [cmd]`: the cached `--fdl-schema` answers of the project's sub-commands."""
    from .manifest import clear_caches, discover_caches, refresh_caches
    table = {"bench": BenchArgs, "export-hf": ExportArgs, "init": InitArgs}
    if argv and argv[0] in ("list", "clear", "refresh"):
        if manifest is None:
            print("fdl schema: no fdl.yml found", file=sys.stderr)
            return 1
        only = next((a for a in argv[1:] if not a.startswith("-")), None)
        if argv[0] == "list":
            rows = discover_caches(manifest)
            if "--json" in argv:
                print(json.dumps(rows, indent=2))
            else:
                for r in rows:
                    print(f"{r['command']:<20} {r['status']:<7} {r['path']}")
                if not rows:
                    print("no cached schemas")
        elif argv[0] == "clear":
            print(f"removed {clear_caches(manifest, only)} cached schema(s)")
        else:
            done = refresh_caches(manifest, only, env)
            print("refreshed: " + (", ".join(done) if done else "nothing (no sub-command with an entry answered --fdl-schema)"))
        return 0
    if not argv or argv[0] not in table:
        print(json.dumps({k: v.schema() for k, v in table.items()}, indent=2))
    else:
        print(json.dumps(table[argv[0]].schema(), indent=2))
    return 0


def config_show(manifest: Optional[str], env: Optional[str]) -> int:
    if manifest is None:
        print("no fdl.yml found", file=sys.stderr)
        return 1
    man, origin = load_manifest(manifest, env)

    def walk(node, path, depth):
        for k, v in node.items():
            sub = f"{path}.{k}" if path else str(k)
            if isinstance(v, dict):
                print("  " * depth + f"{k}:")
                walk(v, sub, depth + 1)
            else:
                print("  " * depth + f"{k}: {v!r}    # {origin.get(sub, '?')}")
    walk(man, "", 0)
    return 0


def usage(manifest: Optional[str]) -> str:
    lines = ["usage: python -m flodl_b200.cli [--env NAME] [--dry-run] <command> [args]", "", "built-in commands:",
             "  diagnose [--json]       report interpreter, torch, CUDA, GPUs and the native library",
             "  build                   compile the native library for sm_100a",
             "  bench [options]         run the training benchmark",
             "  export-hf <ckpt>        .fdl checkpoint -> HuggingFace directory",
             "  api-ref [--json]        list the public API",
             "  schema [command]        argument schemas as JSON",
             "  schema list|clear|refresh  cached --fdl-schema answers of the project's sub-commands",
             "  completions <shell>     shell completion script (bash, zsh, fish), aware of the project and of option values",
             "  autocomplete            install the completion script for the login shell",
             "  config show [env]       the merged manifest with the origin of every value",
             "  init <name>             scaffold a project",
             "  add [dir]               add a training scaffold to an existing directory",
             "  setup [--force]         check the machine and build the native library",
             "  install [--check|--dev] build and verify the native library",
             "  libtorch <verb>         info | list | path | activate | download | build | remove: the libtorch variants under libtorch/",
             "  skill show|install      the assistant guide (condensed API and porting reference)"]
    if manifest:
        try:
            cmds = load_manifest(manifest)[0].get("commands") or {}
            if cmds:
                lines += ["", f"commands from {manifest}:"]
                here = os.path.dirname(os.path.abspath(manifest))
                for k, v in cmds.items():
                    desc = (v or {}).get("description", "") if isinstance(v, dict) or v is None else ""
                    if not desc and command_kind(k, v, here) == "path":       # a sub-project: its own manifest describes it
                        child = manifest_in(os.path.join(here, (v or {}).get("path", k)))
                        try:
                            desc = (load_manifest(child)[0].get("description") or "") if child else ""
                        except ManifestError:
                            desc = ""
                    lines.append(f"  {k:<23} {desc}")
        except ManifestError as e:
            lines += ["", f"(manifest error: {e})"]
    return "\n".join(lines)


def main(argv: Optional[List[str]] = None) -> int:
    rc = _main(argv)
    try:                                              # after the command's own output; never in its way
        import flodl_b200
        from .update_check import check
        for line in check(flodl_b200.__version__):
            print(line, file=sys.stderr)
    except Exception:  # noqa: BLE001
        pass
    return rc


def _main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    env = None
    dry = False
    while argv and argv[0] in ("--env", "--dry-run"):
        if argv[0] == "--env":
            if len(argv) < 2:
                print("--env needs a name", file=sys.stderr)
                return 2
            env, argv = argv[1], argv[2:]
        else:
            dry, argv = True, argv[1:]
    manifest = find_manifest(os.getcwd())
    if manifest is not None and manifest.endswith((".example", ".dist")):
        manifest = adopt_template(manifest)              # a checkout ships the template; the copy is the user's to edit
    if manifest is not None and env is None and argv and not os.environ.get("FDL_ENV") and argv[0] not in BUILTINS:
        try:
            env, argv = env_from_first_word(manifest, argv)      # `fdl ci test` = `fdl --env ci test`
        except ManifestError as e:
            print(f"fdl: {e}", file=sys.stderr)
            return 2
    if not argv or argv[0] in ("help", "-h", "--help"):
        print(usage(manifest))
        return 0
    cmd, rest = argv[0], argv[1:]
    try:
        if cmd == "diagnose":
            return diagnose("--json" in rest)
        if cmd == "build":
            from .. import _build
            _build.build()
            return 0
        if cmd == "bench":
            return bench(rest)
        if cmd == "export-hf":
            return export_hf(rest)
        if cmd == "api-ref":
            return api_ref("--json" in rest)
        if cmd == "schema":
            return schema(rest, manifest, env)
        if cmd == "completions":
            return completions(rest[0] if rest else "bash", manifest)
        if cmd == "autocomplete":
            return autocomplete(manifest)
        if cmd == "config":
            if rest[:1] == ["show"]:
                return config_show(manifest, rest[1] if len(rest) > 1 else env)
            print("usage: config show [env]", file=sys.stderr)
            return 2
        if cmd == "init":
            return init(rest)
        if cmd in ("setup", "install", "libtorch", "add", "skill"):
            from . import setup_cmds
            return getattr(setup_cmds, cmd)(rest)
        if manifest is None:
            print(f"unknown command {cmd!r} and no fdl.yml found", file=sys.stderr)
            return 2
        return run_command(manifest, argv, env, dry)
    except (ArgError, ManifestError) as e:
        print(f"fdl: {e}", file=sys.stderr)
        return 2
