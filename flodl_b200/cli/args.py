"""Typed command-line arguments from a dataclass: parser, `--help` text and a JSON schema
(`--fdl-schema`), the role `#[derive(FdlArgs)]` plays in the reference (flodl-cli-macros/src/lib.rs).

    @dataclass
    class TrainArgs(FdlArgs):
        '''Train a model.'''
        epochs: int = arg(10, help="number of epochs", short="e")
        lr: float = arg(1e-3, help="learning rate")
        model: str = arg("mlp", help="model name", choices=["mlp", "resnet"])
        resume: bool = arg(False, help="resume from the last checkpoint")
        data: str = arg(REQUIRED, help="dataset directory", positional=True)

    args = TrainArgs.parse(argv)          # exits with the help text on --help, prints the schema on --fdl-schema
"""
from __future__ import annotations

import dataclasses
import json
import sys
from typing import Any, Dict, List, Optional, Sequence, get_args, get_origin, get_type_hints

REQUIRED = object()


def arg(default: Any = REQUIRED, *, help: str = "", short: Optional[str] = None, choices: Optional[Sequence] = None,
        positional: bool = False, env: Optional[str] = None):
    meta = {"help": help, "short": short, "choices": list(choices) if choices else None, "positional": positional, "env": env}
    if default is REQUIRED:
        return dataclasses.field(default=None, metadata={**meta, "required": True})
    if isinstance(default, (list, dict)):
        return dataclasses.field(default_factory=lambda: type(default)(default), metadata={**meta, "required": False})
    return dataclasses.field(default=default, metadata={**meta, "required": False})


class ArgError(Exception):
    pass


def _kind(tp) -> tuple:
    """(base type, is_list, is_optional)"""
    origin = get_origin(tp)
    if origin in (list, List):
        return get_args(tp)[0], True, False
    if origin is not None and type(None) in get_args(tp):
        inner = [a for a in get_args(tp) if a is not type(None)][0]
        base, is_list, _ = _kind(inner)
        return base, is_list, True
    return tp, False, False


def _convert(base, text: str, name: str):
    try:
        if base is bool:
            if text.lower() in ("1", "true", "yes", "on"):
                return True
            if text.lower() in ("0", "false", "no", "off"):
                return False
            raise ValueError(text)
        return base(text)
    except (ValueError, TypeError):
        raise ArgError(f"invalid value {text!r} for --{name} (expected {getattr(base, '__name__', base)})")


class FdlArgs:
    """Mix into a dataclass."""

    @classmethod
    def _fields(cls):
        hints = get_type_hints(cls)
        out = []
        for f in dataclasses.fields(cls):
            base, is_list, optional = _kind(hints[f.name])
            out.append((f, base, is_list, optional))
        return out

    @classmethod
    def schema(cls) -> Dict[str, Any]:
        names = {int: "integer", float: "number", str: "string", bool: "boolean"}
        args = []
        for f, base, is_list, optional in cls._fields():
            m = f.metadata
            default = None if m.get("required") else (f.default if f.default is not dataclasses.MISSING else f.default_factory())
            args.append({"name": f.name.replace("_", "-"), "type": names.get(base, "string"), "list": is_list,
                         "required": bool(m.get("required")), "default": default, "help": m.get("help", ""),
                         "short": m.get("short"), "choices": m.get("choices"), "positional": bool(m.get("positional")), "env": m.get("env")})
        return {"command": cls.__name__, "description": (cls.__doc__ or "").strip(), "args": args}

    @classmethod
    def help_text(cls, prog: str = "") -> str:
        sc = cls.schema()
        pos = [a for a in sc["args"] if a["positional"]]
        opt = [a for a in sc["args"] if not a["positional"]]
        usage = f"usage: {prog or sc['command']} [options]" + "".join(f" <{a['name']}>" for a in pos)
        lines = [usage]
        if sc["description"]:
            lines += ["", sc["description"]]
        if pos:
            lines += ["", "arguments:"] + [f"  {a['name']:<22} {a['help']}" for a in pos]
        lines += ["", "options:"]
        for a in opt:
            flag = (f"-{a['short']}, " if a["short"] else "    ") + f"--{a['name']}"
            if a["type"] != "boolean":
                flag += f" <{a['type']}>"
            extra = []
            if a["choices"]:
                extra.append("one of " + ", ".join(map(str, a["choices"])))
            if not a["required"] and a["default"] not in (None, False, [], ""):
                extra.append(f"default {a['default']}")
            if a["required"]:
                extra.append("required")
            if a["env"]:
                extra.append(f"env {a['env']}")
            lines.append(f"  {flag:<30} {a['help']}" + (f" [{'; '.join(extra)}]" if extra else ""))
        lines.append(f"  {'    --fdl-schema':<30} print this command's argument schema as JSON")
        lines.append(f"  {'-h, --help':<30} show this help")
        return "\n".join(lines)

    @classmethod
    def parse(cls, argv: Optional[Sequence[str]] = None, prog: str = "", exit_on_help: bool = True):
        import os
        argv = list(sys.argv[1:] if argv is None else argv)
        if "--fdl-schema" in argv:
            print(json.dumps(cls.schema(), indent=2))
            if exit_on_help:
                sys.exit(0)
            return None
        if "-h" in argv or "--help" in argv:
            print(cls.help_text(prog))
            if exit_on_help:
                sys.exit(0)
            return None
        fields = cls._fields()
        by_flag = {}
        positional = []
        for item in fields:
            f = item[0]
            if f.metadata.get("positional"):
                positional.append(item)
            else:
                by_flag["--" + f.name.replace("_", "-")] = item
                if f.metadata.get("short"):
                    by_flag["-" + f.metadata["short"]] = item
        values: Dict[str, Any] = {}
        pos_vals: List[str] = []
        i = 0
        while i < len(argv):
            tok = argv[i]
            if tok == "--":
                pos_vals += argv[i + 1:]
                break
            if tok.startswith("-") and tok != "-" and not _is_number(tok):
                key, eq, inline = tok.partition("=")
                negate = False
                if key not in by_flag and key.startswith("--no-") and ("--" + key[5:]) in by_flag:
                    key, negate = "--" + key[5:], True
                if key not in by_flag:
                    raise ArgError(f"unknown option {tok!r}")
                f, base, is_list, _ = by_flag[key]
                name = f.name.replace("_", "-")
                if base is bool and not is_list:
                    values[f.name] = (not negate) if not eq else _convert(bool, inline, name)
                else:
                    if eq:
                        text = inline
                    else:
                        i += 1
                        if i >= len(argv):
                            raise ArgError(f"option --{name} needs a value")
                        text = argv[i]
                    v = _convert(base, text, name)
                    if f.metadata.get("choices") and v not in f.metadata["choices"]:
                        raise ArgError(f"--{name}: {v!r} is not one of {f.metadata['choices']}")
                    if is_list:
                        values.setdefault(f.name, []).append(v)
                    else:
                        values[f.name] = v
            else:
                pos_vals.append(tok)
            i += 1
        for (f, base, is_list, _), text in zip(positional, pos_vals):
            values[f.name] = [_convert(base, t, f.name) for t in pos_vals[positional.index((f, base, is_list, _)):]] if is_list else _convert(base, text, f.name)
        if len(pos_vals) > len(positional) and not (positional and positional[-1][2]):
            raise ArgError(f"unexpected argument {pos_vals[len(positional)]!r}")
        for f, base, is_list, _ in fields:
            if f.name not in values and f.metadata.get("env") and os.environ.get(f.metadata["env"]) is not None:
                values[f.name] = _convert(base, os.environ[f.metadata["env"]], f.name)
            if f.name not in values and f.metadata.get("required"):
                raise ArgError(f"missing required {'argument' if f.metadata.get('positional') else 'option --'}{f.name.replace('_', '-')}")
        return cls(**values)


def _is_number(tok: str) -> bool:
    try:
        float(tok)
        return True
    except ValueError:
        return False


def argparse_schema(parser, strict: bool = True) -> Dict[str, Any]:
    """The `--fdl-schema` description of an `argparse.ArgumentParser`: `{"options": {name: {type, short, description,
    default, choices}}, "args": [{name, description, ...}], "strict": bool}`. A program that already parses with argparse
    answers the probe with `answer_schema_probe(parser)` as its first line."""
    import argparse
    options: Dict[str, Any] = {}
    args: List[Dict[str, Any]] = []
    for a in parser._actions:
        if isinstance(a, argparse._HelpAction):
            continue
        kind = ("bool" if isinstance(a, (argparse._StoreTrueAction, argparse._StoreFalseAction)) else
                {int: "int", float: "float"}.get(a.type, "string"))
        decl: Dict[str, Any] = {"type": kind, "description": a.help or ""}
        if a.default not in (None, False, "", argparse.SUPPRESS) and kind != "bool":
            decl["default"] = a.default
        if a.choices:
            decl["choices"] = list(a.choices)
        longs = [o for o in a.option_strings if o.startswith("--")]
        shorts = [o for o in a.option_strings if o.startswith("-") and not o.startswith("--")]
        if not a.option_strings:
            args.append({"name": a.dest, **decl, "variadic": a.nargs in ("*", "+")})
            continue
        if shorts:
            decl["short"] = shorts[0][1:]
        options[(longs[0] if longs else shorts[0]).lstrip("-")] = decl
    return {"options": options, "args": args, "strict": strict}


def answer_schema_probe(parser, argv: Optional[Sequence[str]] = None) -> None:
    """Print the schema and exit 0 when the program was started with `--fdl-schema` (before any real work)."""
    argv = sys.argv[1:] if argv is None else argv
    if "--fdl-schema" in argv:
        print(json.dumps(argparse_schema(parser), indent=2))
        raise SystemExit(0)
