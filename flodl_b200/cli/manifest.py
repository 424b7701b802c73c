"""`fdl.yml` manifests: a project's commands, run through `python -m flodl_b200.cli <name>`
(flodl-cli/src/{config,overlay,run,dispatch,schema_cache}.rs).

A manifest (`fdl.yml`, `fdl.yaml` or `fdl.json`; `fdl.yml.example` / `.dist` when no real one exists) has a
`commands:` map. Every entry is one of three kinds, decided by the fields it sets:

* **run**: `run:` is a shell line. `docker: <service>` wraps it in `docker compose run --rm <service> bash -c ..`.
  Arguments typed after an explicit `--` are quoted and spliced in between `run:` and the optional `append:` tail;
  arguments before `--` are refused with the right form in the message.
* **path**: `path: ./dir/` (or an empty entry, meaning `./<name>/`) loads that directory's manifest and goes on there.
  A sub-manifest may declare `entry:` (the program behind the sub-command): every further word is handed to it.
* **preset**: neither `run:` nor `path:`, only inside a sub-manifest with an `entry:`: its `ddp:` / `training:` /
  `output:` / `options:` blocks are merged over the sub-manifest's own and turned into flags of the entry.

`fdl.<env>.yml` overlays are deep-merged over the base (`--env`, `FDL_ENV`, or the overlay's name as first word),
keeping, for `config show`, which file set every value. An entry that answers `--fdl-schema` with a JSON description of
its options is probed once, the answer cached in `<dir>/.fdl/schema-cache/<cmd>.json`, and used for `--help` and to
check preset values.
"""
from __future__ import annotations

import json
import os
import shlex
import shutil
import subprocess
from typing import Any, Dict, List, Optional, Tuple

import yaml

MANIFEST_NAMES = ("fdl.yml", "fdl.yaml", "fdl.json")
TEMPLATE_NAMES = ("fdl.yml.example", "fdl.yaml.example", "fdl.yml.dist", "fdl.yaml.dist")
SECTIONS = ("ddp", "training", "output", "options")


class ManifestError(Exception):
    pass


# ---- files ---------------------------------------------------------------------------------------------------
def manifest_in(directory: str) -> Optional[str]:
    """The manifest of one directory: a real one first, a template (`.example`, `.dist`) otherwise."""
    for n in MANIFEST_NAMES + TEMPLATE_NAMES:
        p = os.path.join(directory, n)
        if os.path.isfile(p):
            return p
    return None


def find_manifest(start: str = ".") -> Optional[str]:
    d = os.path.abspath(start)
    while True:
        p = manifest_in(d)
        if p is not None:
            return p
        parent = os.path.dirname(d)
        if parent == d:
            return None
        d = parent


def adopt_template(path: str) -> str:
    """Copy `fdl.yml.example` to the (git-ignored) `fdl.yml` beside it so it can be edited locally; returns the copy."""
    base = os.path.basename(path)
    for suffix in (".example", ".dist"):
        if base.endswith(suffix):
            real = os.path.join(os.path.dirname(path), base[: -len(suffix)])
            if not os.path.exists(real):
                shutil.copyfile(path, real)
            return real
    return path


def _read(path: str) -> Dict[str, Any]:
    with open(path) as f:
        data = json.load(f) if path.endswith(".json") else yaml.safe_load(f)
    data = data or {}
    if not isinstance(data, dict):
        raise ManifestError(f"{path}: top level must be a mapping")
    return data


# ---- overlays ------------------------------------------------------------------------------------------------
def deep_merge(base: Any, over: Any, origin: Dict[str, str], path: str, label: str) -> Any:
    """Dicts merge key by key, everything else is replaced; `origin[path]` records who set a leaf."""
    if isinstance(base, dict) and isinstance(over, dict):
        out = dict(base)
        for k, v in over.items():
            sub = f"{path}.{k}" if path else str(k)
            out[k] = deep_merge(base.get(k), v, origin, sub, label) if k in base else _mark(v, origin, sub, label)
        return out
    return _mark(over, origin, path, label)


def _mark(v: Any, origin: Dict[str, str], path: str, label: str) -> Any:
    if isinstance(v, dict):
        for k, x in v.items():
            _mark(x, origin, f"{path}.{k}" if path else str(k), label)
    else:
        origin[path] = label
    return v


def overlay_path(manifest_path: str, env: str) -> Optional[str]:
    stem = os.path.join(os.path.dirname(os.path.abspath(manifest_path)), "fdl")
    return next((p for p in (f"{stem}.{env}.yml", f"{stem}.{env}.yaml", f"{stem}.{env}.json") if os.path.isfile(p)), None)


def list_envs(manifest_path: str) -> List[str]:
    """Names of the overlays that sit beside the manifest (`fdl.ci.yml` -> `ci`)."""
    d = os.path.dirname(os.path.abspath(manifest_path))
    out = set()
    for n in os.listdir(d):
        parts = n.split(".")
        if len(parts) == 3 and parts[0] == "fdl" and parts[2] in ("yml", "yaml", "json") and parts[1] not in ("yml", "yaml"):
            out.add(parts[1])
    return sorted(out)


def load_manifest(path: str, env: Optional[str] = None) -> Tuple[Dict[str, Any], Dict[str, str]]:
    base = _read(path)
    origin: Dict[str, str] = {}
    _mark(base, origin, "", os.path.basename(path))
    env = env or os.environ.get("FDL_ENV")
    if env:
        over_path = overlay_path(path, env)
        if over_path is None:
            raise ManifestError(f"no overlay fdl.{env}.yml next to {path}")
        base = deep_merge(base, _read(over_path), origin, "", os.path.basename(over_path))
    validate_manifest(base, path)
    return base, origin


def env_from_first_word(manifest_path: str, words: List[str]) -> Tuple[Optional[str], List[str]]:
    """`fdl ci test` selects `fdl.ci.yml` when that file exists. A name that is both an overlay and a command is
    refused as ambiguous; a word that is no overlay falls through to ordinary dispatch."""
    if not words or overlay_path(manifest_path, words[0]) is None:
        return None, words
    cmds = _read(manifest_path).get("commands") or {}
    if words[0] in cmds:
        raise ManifestError(f"`{words[0]}` names both a command and the overlay fdl.{words[0]}.yml; use --env {words[0]} for the overlay")
    return words[0], words[1:]


# ---- command kinds and load-time checks ------------------------------------------------------------------------
def command_kind(name: str, spec: Any, here: str) -> str:
    """"run", "path" or "preset" (see the module docstring)."""
    if isinstance(spec, dict) and "run" in spec:
        return "run"
    if isinstance(spec, dict) and "path" in spec:
        return "path"
    if spec is None or spec == {} or (isinstance(spec, dict) and set(spec) <= {"description"}):
        return "path" if os.path.isdir(os.path.join(here, name)) or spec is None else "preset"
    return "preset"


def validate_manifest(man: Dict[str, Any], path: str) -> None:
    """What can be refused before anything runs: `docker:` or `append:` on an entry that is not a run command, a
    preset in a manifest without an `entry:`, a non-mapping entry."""
    cmds = man.get("commands") or {}
    if not isinstance(cmds, dict):
        raise ManifestError(f"{path}: `commands:` must be a mapping")
    here = os.path.dirname(os.path.abspath(path))
    for name, spec in cmds.items():
        if spec is not None and not isinstance(spec, dict):
            raise ManifestError(f"{path}: command `{name}` must be a mapping (or empty for ./{name}/)")
        kind = command_kind(name, spec, here)
        spec = spec or {}
        if kind != "run":
            for field in ("docker", "append"):
                if field in spec:
                    raise ManifestError(f"{path}: `{field}:` on command `{name}` needs `run:` (it is a {kind} entry)")
        if kind == "preset" and "entry" not in man:
            raise ManifestError(f"{path}: command `{name}` has neither `run:` nor `path:`; presets need an `entry:` in this manifest")
        if kind == "run" and not isinstance(spec.get("run"), str):
            raise ManifestError(f"{path}: `run:` of command `{name}` must be a string")


def _sub_manifest(here: str, name: str, spec: Any) -> str:
    sub_dir = os.path.normpath(os.path.join(here, (spec or {}).get("path", f"./{name}/")))
    sub = manifest_in(sub_dir)
    if sub is None:
        raise ManifestError(f"command {name!r} points at {sub_dir}, which has no fdl.yml")
    return sub


class Resolved:
    """Where dispatch ended: the manifest it is in, the kind, the command's own mapping (None when a sub-manifest's
    `entry:` is addressed directly), the words still left, and the directory to run in."""

    def __init__(self, manifest: Dict[str, Any], manifest_path: str, kind: str, name: str, spec: Optional[Dict[str, Any]], rest: List[str]):
        self.manifest, self.manifest_path, self.kind, self.name, self.spec, self.rest = manifest, manifest_path, kind, name, spec, rest
        self.cwd = os.path.dirname(os.path.abspath(manifest_path))


def resolve(manifest_path: str, words: List[str], env: Optional[str] = None, _name: str = "") -> Resolved:
    man, _ = load_manifest(manifest_path, env)
    cmds = man.get("commands") or {}
    here = os.path.dirname(os.path.abspath(manifest_path))
    if words and words[0] in cmds:
        name, rest = words[0], words[1:]
        spec = cmds[name]
        kind = command_kind(name, spec, here)
        if kind == "path":
            return resolve(_sub_manifest(here, name, spec), rest, env, name)
        return Resolved(man, manifest_path, kind, name, spec or {}, rest)
    if "entry" in man:                      # `fdl ddp-bench --model mlp`: straight to the entry with the manifest's defaults
        return Resolved(man, manifest_path, "entry", _name or os.path.basename(here), None, list(words))
    if not words:
        raise ManifestError("no command given; available: " + ", ".join(sorted(cmds)))
    raise ManifestError(f"unknown command {words[0]!r}; available: " + ", ".join(sorted(cmds)))


def resolve_command(manifest_path: str, words: List[str], env: Optional[str] = None):
    """(command mapping, remaining words, directory) of a run command, following `path:` entries."""
    r = resolve(manifest_path, words, env)
    if r.kind != "run":
        raise ManifestError(f"command {r.name!r} needs `run:` or `path:`")
    return r.spec, r.rest, r.cwd


# ---- composing the shell line ----------------------------------------------------------------------------------
def split_forwarded(name: str, rest: List[str]) -> List[str]:
    """The words after `--`. Words in front of it are refused: a run command takes extra arguments only this way."""
    if not rest:
        return []
    if rest[0] != "--":
        tail = " ".join(shlex.quote(a) for a in (rest if "--" not in rest else [a for a in rest if a != "--"]))
        raise ManifestError(f"`{name}` is a run command: pass extra arguments after `--` (use `fdl {name} -- {tail}`)")
    return rest[1:]


def build_shell_line(spec: Dict[str, Any], extra: List[str]) -> str:
    """`run:` + the forwarded arguments (quoted) + `append:`."""
    parts = [str(spec["run"])]
    if extra:
        parts.append(" ".join(shlex.quote(a) for a in extra))
    if spec.get("append"):
        parts.append(str(spec["append"]))
    return " ".join(parts).strip()


def docker_wrap(line: str, service: Optional[str]) -> str:
    return line if not service else f"docker compose run --rm {shlex.quote(str(service))} bash -c {shlex.quote(line)}"


_DDP_FLAGS = (("mode", "--mode"), ("policy", "--policy"), ("backend", "--backend"), ("anchor", "--anchor"), ("max_anchor", "--max-anchor"),
              ("overhead_target", "--overhead-target"), ("divergence_threshold", "--divergence-threshold"), ("max_batch_diff", "--max-batch-diff"),
              ("max_grad_norm", "--max-grad-norm"), ("snapshot_timeout", "--snapshot-timeout"), ("checkpoint_every", "--checkpoint-every"),
              ("progressive", "--progressive"), ("lr_scale_ratio", "--lr-scale-ratio"))
_TRAIN_FLAGS = (("epochs", "--epochs"), ("batch_size", "--batch-size"), ("batches_per_epoch", "--batches"), ("lr", "--lr"), ("seed", "--seed"))
_OUTPUT_FLAGS = (("dir", "--output"), ("monitor", "--monitor"))


def _scalar(v: Any) -> str:
    return ("true" if v else "false") if isinstance(v, bool) else str(v)


def config_to_args(cfg: Dict[str, Any]) -> List[str]:
    """Flags of the entry for a resolved configuration: the `ddp:`, `training:` and `output:` blocks by their fixed
    names, then every `options:` key as `--key value` (`true` gives the bare flag, `false` / null nothing)."""
    args: List[str] = []
    for block, table in (("ddp", _DDP_FLAGS), ("training", _TRAIN_FLAGS), ("output", _OUTPUT_FLAGS)):
        sec = cfg.get(block) or {}
        for key, flag in table:
            if sec.get(key) is not None:
                args += [flag, _scalar(sec[key])]
        if block == "ddp":
            hint = sec.get("speed_hint")
            if isinstance(hint, dict):
                args += ["--speed-hint", f"{hint.get('slow_rank')}:{hint.get('ratio')}"]
            if sec.get("partition_ratios"):
                args += ["--partition-ratios", ",".join(str(r) for r in sec["partition_ratios"])]
            if sec.get("timeline") is True:
                args.append("--timeline")
    for key, val in (cfg.get("options") or {}).items():
        flag = "--" + str(key).replace("_", "-")
        if val is True:
            args.append(flag)
        elif val is not None and val is not False:
            args += [flag, ",".join(str(x) for x in val) if isinstance(val, list) else str(val)]
    return args


def resolved_config(man: Dict[str, Any], preset: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    """The sub-manifest's own `ddp / training / output / options` with the preset's laid over them."""
    out: Dict[str, Any] = {}
    for sec in SECTIONS:
        merged = dict(man.get(sec) or {})
        merged.update((preset or {}).get(sec) or {})
        if merged:
            out[sec] = merged
    return out


def compose(r: Resolved) -> str:
    """The shell line a resolved command stands for."""
    if r.kind == "run":
        line = build_shell_line(r.spec, split_forwarded(r.name, r.rest))
        return docker_wrap(line, r.spec.get("docker"))
    cfg = resolved_config(r.manifest, r.spec)
    if r.kind == "preset":
        check_against_schema(r, cfg)
    extra = [a for a in r.rest if a != "--refresh-schema"]
    line = " ".join([str(r.manifest["entry"]).strip()] + [shlex.quote(a) for a in config_to_args(cfg) + extra])
    return docker_wrap(line, r.manifest.get("docker"))


# ---- `--fdl-schema`: probing, the cache, checks, help ------------------------------------------------------------
def cache_path(cmd_dir: str, cmd: str) -> str:
    return os.path.join(cmd_dir, ".fdl", "schema-cache", f"{cmd}.json")


def is_cargo_entry(entry: str) -> bool:
    """Entries that compile before they answer are never probed on their own (a `--help` must not start a build)."""
    first = shlex.split(entry)[:1]
    return bool(first) and first[0] == "cargo"


def probe(entry: str, cwd: str, timeout_s: float = 20.0) -> Optional[Dict[str, Any]]:
    """Run the entry with `--fdl-schema` and parse what it prints; None when it does not answer with a JSON object."""
    try:
        out = subprocess.run(f"{entry.strip()} --fdl-schema", shell=True, cwd=cwd, capture_output=True, text=True, timeout=timeout_s)
    except (subprocess.TimeoutExpired, OSError):
        return None
    if out.returncode != 0:
        return None
    try:
        data = json.loads(out.stdout)
    except ValueError:
        return None
    return data if isinstance(data, dict) and ("options" in data or "args" in data) else None


def read_cache(cmd_dir: str, cmd: str) -> Optional[Dict[str, Any]]:
    try:
        with open(cache_path(cmd_dir, cmd)) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def write_cache(cmd_dir: str, cmd: str, schema: Dict[str, Any]) -> str:
    p = cache_path(cmd_dir, cmd)
    os.makedirs(os.path.dirname(p), exist_ok=True)
    with open(p, "w") as f:
        json.dump(schema, f, indent=2)
    return p


def is_stale(cmd_dir: str, cmd: str, manifest_path: str) -> bool:
    """A cached schema older than the manifest it belongs to is probed again."""
    try:
        return os.path.getmtime(cache_path(cmd_dir, cmd)) < os.path.getmtime(manifest_path)
    except OSError:
        return True


def schema_for(r: Resolved, refresh: bool = False) -> Optional[Dict[str, Any]]:
    """The option schema of a sub-command with an `entry:`: an inline `schema:` block of the manifest wins; else the
    cache; else (for entries that do not compile first) a fresh probe that is then cached."""
    man = r.manifest
    if "entry" not in man:
        return None
    if isinstance(man.get("schema"), dict) and not refresh:
        return man["schema"]
    cmd = os.path.basename(r.cwd)
    cached = None if refresh else read_cache(r.cwd, cmd)
    if cached is not None and not is_stale(r.cwd, cmd, r.manifest_path):
        return cached
    if is_cargo_entry(str(man["entry"])) and not refresh:
        return cached
    fresh = probe(str(man["entry"]), r.cwd)
    if fresh is not None:
        write_cache(r.cwd, cmd, fresh)
        return fresh
    return cached


def check_against_schema(r: Resolved, cfg: Dict[str, Any]) -> None:
    """A preset may only set options the entry declares, with values among the declared `choices`."""
    schema = schema_for(r)
    if not schema or not isinstance(schema.get("options"), dict):
        return
    opts = schema["options"]
    strict = bool(schema.get("strict", False))
    for key, val in (cfg.get("options") or {}).items():
        name = str(key).replace("_", "-")
        decl = opts.get(name, opts.get(str(key)))
        if val is None:                     # null un-sets an inherited option: nothing reaches the entry
            continue
        if decl is None:
            if strict:
                raise ManifestError(f"preset `{r.name}` sets option `{name}`, which `{os.path.basename(r.cwd)}` does not declare")
            continue
        choices = decl.get("choices")
        if choices and not isinstance(val, bool) and str(val) not in [str(c) for c in choices]:
            raise ManifestError(f"preset `{r.name}`: `{name}: {val}` is not one of {', '.join(str(c) for c in choices)}")


def discover_caches(root_manifest: str) -> List[Dict[str, Any]]:
    """Every cached schema below the project root with its state: fresh, stale (older than its manifest) or orphan
    (no manifest with an `entry:` beside it any more)."""
    root = os.path.dirname(os.path.abspath(root_manifest))
    out = []
    for d, dirs, _files in os.walk(root):
        dirs[:] = [x for x in dirs if x not in (".git", "node_modules", "__pycache__", "build")]
        cdir = os.path.join(d, ".fdl", "schema-cache")
        if not os.path.isdir(cdir):
            continue
        man_path = manifest_in(d)
        for n in sorted(os.listdir(cdir)):
            if n.endswith(".json"):
                cmd = n[:-5]
                has_entry = man_path is not None and "entry" in _read(man_path)
                state = "orphan" if not has_entry else ("stale" if is_stale(d, cmd, man_path) else "fresh")
                out.append({"command": cmd, "dir": d, "path": os.path.join(cdir, n), "status": state})
    return out


def clear_caches(root_manifest: str, only: Optional[str] = None) -> int:
    n = 0
    for c in discover_caches(root_manifest):
        if only is None or c["command"] == only:
            os.remove(c["path"])
            n += 1
    return n


def refresh_caches(root_manifest: str, only: Optional[str] = None, env: Optional[str] = None) -> List[str]:
    """Probe every path-kind sub-command that has an `entry:` (or just `only`) and rewrite its cache."""
    man, _ = load_manifest(root_manifest, env)
    here = os.path.dirname(os.path.abspath(root_manifest))
    done = []
    for name, spec in (man.get("commands") or {}).items():
        if command_kind(name, spec, here) != "path" or (only is not None and name != only):
            continue
        try:
            r = resolve(root_manifest, [name], env)
        except ManifestError:
            continue
        if r.kind == "entry" and schema_for(r, refresh=True) is not None:
            done.append(name)
    return done


def command_help(r: Resolved) -> str:
    """`fdl <cmd> --help`: the description, the presets and other sub-commands, the resolved defaults and the
    entry's options as its schema describes them."""
    man = r.manifest
    lines = []
    if r.kind == "run":
        lines.append(f"{r.name}: {r.spec.get('description', '')}".rstrip(": "))
        lines.append(f"  runs: {docker_wrap(build_shell_line(r.spec, []), r.spec.get('docker'))}")
        lines.append(f"  extra arguments: fdl {r.name} -- <args>")
        return "\n".join(lines)
    lines.append(f"{os.path.basename(r.cwd)}: {man.get('description', '')}".rstrip(": "))
    presets = {k: v or {} for k, v in (man.get("commands") or {}).items() if command_kind(k, v, r.cwd) == "preset"}
    others = {k: v or {} for k, v in (man.get("commands") or {}).items() if k not in presets}
    if presets:
        lines += ["", f"Arguments:", f"  [{man.get('arg-name', 'preset')}]"]
        lines += [f"    {k:<18} {v.get('description', '')}".rstrip() for k, v in presets.items()]
    if others:
        lines += ["", "Commands:"] + [f"  {k:<20} {v.get('description', '')}".rstrip() for k, v in others.items()]
    cfg = resolved_config(man, r.spec if r.kind == "preset" else None)
    if cfg:
        lines += ["", "Resolved defaults:" if r.kind != "preset" else f"Resolved options of `{r.name}`:"]
        lines += ["  " + " ".join(shlex.quote(a) for a in config_to_args(cfg))]
    schema = schema_for(r)
    if schema and isinstance(schema.get("options"), dict):
        lines += ["", "Options:"]
        for name, decl in schema["options"].items():
            short = f"-{decl['short']}, " if decl.get("short") else "    "
            meta = "" if decl.get("type") == "bool" else f" <{decl.get('type', 'value')}>"
            extra = []
            if decl.get("default") is not None:
                extra.append(f"default: {decl['default']}")
            if decl.get("choices"):
                extra.append("one of: " + ", ".join(str(c) for c in decl["choices"]))
            if decl.get("env"):
                extra.append(f"env: {decl['env']}")
            lines.append(f"  {short}--{name}{meta}".ljust(34) + f" {decl.get('description', '')}" + (f" [{'; '.join(extra)}]" if extra else ""))
    for a in (schema or {}).get("args", []) or []:
        lines.append(f"  <{a.get('name', 'arg')}>".ljust(34) + f" {a.get('description', '')}")
    return "\n".join(lines)


# ---- running ---------------------------------------------------------------------------------------------------
def run_command(manifest_path: str, words: List[str], env: Optional[str] = None, dry_run: bool = False) -> int:
    if env is None and not os.environ.get("FDL_ENV"):
        env, words = env_from_first_word(manifest_path, words)
    r = resolve(manifest_path, words, env)
    if any(a in ("--help", "-h") for a in r.rest) and not (r.kind == "run" and "--" in r.rest and r.rest.index("--") < min(
            r.rest.index(a) for a in ("--help", "-h") if a in r.rest)):
        print(command_help(r))
        return 0
    if "--refresh-schema" in r.rest and r.kind in ("entry", "preset"):
        schema_for(r, refresh=True)
    line = compose(r)
    if dry_run:
        print(line)
        return 0
    return subprocess.call(line, shell=True, cwd=r.cwd)


# ---- completion data ---------------------------------------------------------------------------------------------
def completion_tree(manifest_path: str, env: Optional[str] = None, _depth: int = 0) -> Dict[str, Any]:
    """What can follow what, for the completion scripts: `{"words": {name: subtree}, "flags": {"--flag": [choices]}}`
    per level, following path-kind commands into their manifests and reading option names / choices from schemas."""
    try:
        man, _ = load_manifest(manifest_path, env)
    except ManifestError:
        return {"words": {}, "flags": {}}
    here = os.path.dirname(os.path.abspath(manifest_path))
    node: Dict[str, Any] = {"words": {}, "flags": {}}
    for name, spec in (man.get("commands") or {}).items():
        kind = command_kind(name, spec, here)
        sub: Dict[str, Any] = {"words": {}, "flags": {}}
        if kind == "path" and _depth < 4:
            try:
                sub = completion_tree(_sub_manifest(here, name, spec), env, _depth + 1)
            except ManifestError:
                pass
        node["words"][name] = sub
    if "entry" in man:
        r = Resolved(man, manifest_path, "entry", os.path.basename(here), None, [])
        schema = man.get("schema") if isinstance(man.get("schema"), dict) else read_cache(here, os.path.basename(here))
        if schema is None and not is_cargo_entry(str(man["entry"])):
            schema = schema_for(r)
        for opt, decl in ((schema or {}).get("options") or {}).items():
            node["flags"]["--" + opt] = [str(c) for c in (decl.get("choices") or [])]
        for name in node["words"]:                      # a preset takes the entry's flags too
            if not node["words"][name]["words"] and not node["words"][name]["flags"]:
                node["words"][name] = {"words": {}, "flags": dict(node["flags"])}
    return node


def flatten_completions(tree: Dict[str, Any], prefix: str = "") -> List[Tuple[str, List[str], Dict[str, List[str]]]]:
    """[(command path, words that may follow, {flag: choices})], root first."""
    out = [(prefix, sorted(tree["words"]) + sorted(tree["flags"]), {f: c for f, c in tree["flags"].items() if c})]
    for name, sub in tree["words"].items():
        out += flatten_completions(sub, f"{prefix} {name}")
    return out
