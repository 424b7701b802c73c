"""Tolerant `config.json` field parsers shared by the model families (flodl-hf/src/config_json.rs)."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

from ..nn.activation import GeluApprox
from ..tensor import TensorError


def parse(s: str) -> Dict[str, Any]:
    try:
        v = json.loads(s)
    except json.JSONDecodeError as e:
        raise TensorError(f"config.json parse error: {e}")
    if not isinstance(v, dict):
        raise TensorError("config.json: top level must be an object")
    return v


def required_i64(v, key: str) -> int:
    x = v.get(key)
    if isinstance(x, bool) or not isinstance(x, (int, float)) or int(x) != x:
        raise TensorError(f"config.json: missing or non-integer `{key}`")
    return int(x)


def optional_i64(v, key: str, default: int) -> int:
    x = v.get(key)
    return int(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else default


def optional_i64_or_none(v, key: str) -> Optional[int]:
    x = v.get(key)
    return int(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else None


def optional_f64(v, key: str, default: float) -> float:
    x = v.get(key)
    return float(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else default


def optional_hidden_act(v, key: str, default: str) -> GeluApprox:
    act = v.get(key, default)
    if act in ("gelu",):
        return GeluApprox.Exact
    if act in ("gelu_new", "gelu_pytorch_tanh", "gelu_fast"):
        return GeluApprox.Tanh
    raise TensorError(f"config.json: unsupported {key} `{act}` (supported: gelu, gelu_new, gelu_pytorch_tanh)")


def parse_id2label(v) -> Optional[List[str]]:
    m = v.get("id2label")
    if not isinstance(m, dict) or not m:
        return None
    try:
        items = sorted(((int(k), str(val)) for k, val in m.items()))
    except ValueError:
        raise TensorError("config.json: id2label keys must be integers")
    if [k for k, _ in items] != list(range(len(items))):
        raise TensorError("config.json: id2label keys must be 0..n-1")
    return [val for _, val in items]


def parse_num_labels(v, id2label) -> Optional[int]:
    if id2label is not None:
        return len(id2label)
    x = v.get("num_labels")
    return int(x) if isinstance(x, int) else None


def parse_architectures(v) -> Optional[List[str]]:
    a = v.get("architectures")
    return [str(x) for x in a] if isinstance(a, list) else None


def emit_hidden_act(a: GeluApprox) -> str:
    return "gelu" if a == GeluApprox.Exact else "gelu_new"


def emit_architectures(a, default: str) -> List[str]:
    return list(a) if a else [default]


def emit_id2label(labels) -> Dict[str, str]:
    return {str(i): l for i, l in enumerate(labels)}


def optional_bool(v, key: str, default: bool) -> bool:
    x = v.get(key)
    return bool(x) if isinstance(x, bool) else default
