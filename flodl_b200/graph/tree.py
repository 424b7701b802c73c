"""Graph tree: labelled child graphs addressed by dotted paths (flodl/src/graph/tree.rs).

`"a.b.tag"`: every segment but the last must be a child label; a single segment resolves to a
child graph first, then to a tag. Crossing into a child hides its internal tags (explicit
`.internal(tag)` or `_`-prefixed). Everything here is query-time; the forward path is untouched.
"""
from __future__ import annotations

from enum import Enum
from typing import Dict, List, Optional, Tuple

from ..nn import checkpoint as _ckpt
from ..nn.module import walk_modules
from ..tensor import TensorError
from .trend import Trend


class PathKind(Enum):
    Subgraph = "subgraph"
    Tag = "tag"


class TreeMixin:
    # ---- resolution -----------------------------------------------------------------------------
    def _resolve(self, path: str):
        if not path:
            raise TensorError("empty label path")
        return self._resolve_segments(path.split("."), path, False)

    def _resolve_segments(self, segs: List[str], full: str, cross: bool):
        first = segs[0]
        if len(segs) == 1:
            g = self.child_graph(first)
            if g is not None:
                return ("subgraph", g, None)
            if first in self.tag_names:
                if cross and first in self.internal_tags_set:
                    raise TensorError(f'tag "{first}" is internal and cannot be accessed from a parent graph (path: "{full}")')
                return ("tag", self, first)
            raise TensorError(f'"{first}" is not a subgraph or tag of this graph (path: "{full}")')
        child = self.child_graph(first)
        if child is None:
            raise TensorError(f'"{first}" is not a subgraph of this graph (path: "{full}")')
        return child._resolve_segments(segs[1:], full, True)

    # ---- navigation -----------------------------------------------------------------------------
    def tree_children(self) -> Dict[str, "TreeMixin"]:
        return {label: g for label, g in self._child_graphs()}

    def child_graph(self, label: str):
        ni = self.children.get(label)
        if ni is None:
            return None
        mod = self.nodes[ni].module
        return mod.as_graph() if mod is not None else None

    def subgraph(self, path: str):
        kind, g, _ = self._resolve(path)
        if kind != "subgraph":
            raise TensorError(f'path "{path}" resolves to a tag, not a subgraph')
        return g

    def is_composed(self) -> bool:
        return self.composed

    def internal_tags(self):
        return set(self.internal_tags_set)

    def validate_path(self, path: str) -> PathKind:
        kind, _, _ = self._resolve(path)
        return PathKind.Subgraph if kind == "subgraph" else PathKind.Tag

    # ---- parameters -----------------------------------------------------------------------------
    def _tag_module(self, g, tag):
        ni = g.tag_names[tag][0]
        return g.nodes[ni].module

    def parameters_at(self, path: str):
        kind, g, tag = self._resolve(path)
        if kind == "subgraph":
            return g.parameters()
        mod = self._tag_module(g, tag)
        return mod.parameters() if mod is not None else []

    def named_parameters_at(self, path: str):
        kind, g, tag = self._resolve(path)
        if kind == "subgraph":
            return g.named_parameters()
        mod = self._tag_module(g, tag)
        return [(f"{tag}/{p.name}", p) for p in mod.parameters()] if mod is not None else []

    def named_buffers_at(self, path: str):
        kind, g, tag = self._resolve(path)
        if kind == "subgraph":
            return g.named_buffers()
        mod = self._tag_module(g, tag)
        return [(f"{tag}/{b.name}", b) for b in mod.buffers()] if mod is not None else []

    def freeze(self, path: str) -> None:
        for p in self.parameters_at(path):
            p.freeze()

    def thaw(self, path: str) -> None:
        for p in self.parameters_at(path):
            p.unfreeze()

    def is_frozen(self, path: str) -> bool:
        ps = self.parameters_at(path)
        return bool(ps) and all(p.is_frozen() for p in ps)

    def load_subgraph_checkpoint(self, path: str, file: str) -> _ckpt.LoadReport:
        t = self.subgraph(path)
        return _ckpt.load_checkpoint_file(file, t.named_parameters(), t.named_buffers(), t.structural_hash())

    def set_training_at(self, path: str, training: bool) -> None:
        kind, g, tag = self._resolve(path)
        if kind == "subgraph":
            g.set_training(training)
            return
        mod = self._tag_module(g, tag)
        if mod is not None:
            for m in walk_modules(mod):
                m.training = training

    # ---- cross-boundary observation -------------------------------------------------------------
    def tagged_at(self, path: str):
        kind, g, tag = self._resolve(path)
        if kind == "subgraph":
            raise TensorError(f'path "{path}" resolves to a subgraph, not a tag')
        return g.tagged(tag)

    def collect_at(self, paths) -> None:
        for path in paths:
            kind, g, tag = self._resolve(path)
            if kind == "subgraph":
                raise TensorError(f'collect_at: "{path}" resolves to a subgraph, not a tag')
            g.collect([tag])

    def record_at(self, path: str, value: float) -> None:
        segs = path.split(".")
        if len(segs) < 2:
            self.record_scalar(path, value)
            return
        self.subgraph(".".join(segs[:-1])).record_scalar(segs[-1], value)

    def trend_at(self, path: str) -> Trend:
        segs = path.split(".")
        if len(segs) < 2:
            return self.trend(path)
        return self.subgraph(".".join(segs[:-1])).trend(segs[-1])
