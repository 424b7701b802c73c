"""Dotted HuggingFace key paths (flodl-hf/src/path.rs): `HfPath`, `prefix_params`,
`hf_key_from_flodl_key` (replace the LAST '/' of a graph key with '.')."""
from __future__ import annotations

from typing import List

from ..nn.module import Parameter
from ..tensor import TensorError


def _validate(seg: str) -> None:
    if not seg:
        raise TensorError("HfPath segment must not be empty")
    if "/" in seg:
        raise TensorError(f'HfPath segment "{seg}" must not contain \'/\'')
    if "." in seg:
        raise TensorError(f'HfPath segment "{seg}" must not contain \'.\' (use .sub() to add segments)')


class HfPath:
    def __init__(self, root: str):
        _validate(str(root))
        self.path = str(root)

    try_new = classmethod(lambda cls, root: cls(root))
    new = classmethod(lambda cls, root: cls(root))

    def sub(self, segment) -> "HfPath":
        seg = str(segment)
        _validate(seg)
        p = HfPath.__new__(HfPath)
        p.path = f"{self.path}.{seg}"
        return p

    try_sub = sub

    def leaf(self, name: str) -> str:
        _validate(name)
        return f"{self.path}.{name}"

    try_leaf = leaf

    def as_str(self) -> str:
        return self.path

    def __str__(self) -> str:
        return self.path

    def __eq__(self, other) -> bool:
        return isinstance(other, HfPath) and other.path == self.path


def prefix_params(prefix: str, params: List[Parameter]) -> List[Parameter]:
    return [Parameter(p.variable, f"{prefix}.{p.name}") for p in params]


def hf_key_from_flodl_key(key: str) -> str:
    if "/" in key:
        a, b = key.rsplit("/", 1)
        return f"{a}.{b}"
    return key
