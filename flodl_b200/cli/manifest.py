"""`fdl.yml` manifests: named commands (`run:` shell line, `path:` sub-manifest, or a bare name =
`./<name>/fdl.yml`), `append:` default arguments, and `fdl.<env>.yml` overlays deep-merged over the
base with the origin of every value kept for `config show` (flodl-cli/src/{config,overlay,run}.rs)."""
from __future__ import annotations

import os
import shlex
import subprocess
from typing import Any, Dict, List, Optional, Tuple

import yaml

MANIFEST_NAMES = ("fdl.yml", "fdl.yaml", "fdl.yml.example")


class ManifestError(Exception):
    pass


def find_manifest(start: str = ".") -> Optional[str]:
    d = os.path.abspath(start)
    while True:
        for n in MANIFEST_NAMES:
            p = os.path.join(d, n)
            if os.path.isfile(p):
                return p
        parent = os.path.dirname(d)
        if parent == d:
            return None
        d = parent


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


def load_manifest(path: str, env: Optional[str] = None) -> Tuple[Dict[str, Any], Dict[str, str]]:
    with open(path) as f:
        base = yaml.safe_load(f) or {}
    if not isinstance(base, dict):
        raise ManifestError(f"{path}: top level must be a mapping")
    origin: Dict[str, str] = {}
    _mark(base, origin, "", os.path.basename(path))
    env = env or os.environ.get("FDL_ENV")
    if env:
        stem = os.path.join(os.path.dirname(path), "fdl")
        over_path = next((p for p in (f"{stem}.{env}.yml", f"{stem}.{env}.yaml") if os.path.isfile(p)), None)
        if over_path is None:
            raise ManifestError(f"no overlay fdl.{env}.yml next to {path}")
        with open(over_path) as f:
            over = yaml.safe_load(f) or {}
        base = deep_merge(base, over, origin, "", os.path.basename(over_path))
    return base, origin


def resolve_command(manifest_path: str, words: List[str], env: Optional[str] = None):
    """Follow `path:` / bare sub-commands; returns (command dict, remaining words, directory)."""
    man, _ = load_manifest(manifest_path, env)
    cmds = man.get("commands") or {}
    if not words:
        raise ManifestError("no command given; available: " + ", ".join(sorted(cmds)))
    name, rest = words[0], words[1:]
    if name not in cmds:
        raise ManifestError(f"unknown command {name!r}; available: " + ", ".join(sorted(cmds)))
    spec = cmds[name]
    here = os.path.dirname(os.path.abspath(manifest_path))
    if spec is None or (isinstance(spec, dict) and "path" in spec and "run" not in spec):
        sub_dir = os.path.join(here, (spec or {}).get("path", f"./{name}/"))
        sub = next((os.path.join(sub_dir, n) for n in MANIFEST_NAMES if os.path.isfile(os.path.join(sub_dir, n))), None)
        if sub is None:
            raise ManifestError(f"command {name!r} points at {sub_dir}, which has no fdl.yml")
        return resolve_command(sub, rest, env)
    if not isinstance(spec, dict) or "run" not in spec:
        raise ManifestError(f"command {name!r} needs `run:` or `path:`")
    return spec, rest, here


def build_shell_line(spec: Dict[str, Any], extra: List[str]) -> str:
    line = str(spec["run"])
    tail = " ".join(shlex.quote(a) for a in extra) if extra else str(spec.get("append", "") or "")
    return f"{line} {tail}".strip()


def run_command(manifest_path: str, words: List[str], env: Optional[str] = None, dry_run: bool = False) -> int:
    spec, rest, cwd = resolve_command(manifest_path, words, env)
    line = build_shell_line(spec, rest)
    if dry_run:
        print(line)
        return 0
    return subprocess.call(line, shell=True, cwd=cwd)
