"""Observation: tagged outputs -> per-batch buffers -> per-epoch history -> trends
(flodl/src/graph/observe.rs:52-464)."""
from __future__ import annotations

import time
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple

from ..autograd import Variable
from ..tensor import TensorError
from .trend import Trend, TrendGroup


class Reduce(Enum):
    Mean = "mean"
    Sum = "sum"
    Max = "max"
    Min = "min"
    Norm = "norm"

    def apply(self, v: Variable) -> float:
        t = v.data().float()
        return float({"mean": t.mean, "sum": t.sum, "max": t.max, "min": t.min, "norm": t.norm}[self.value]().item())


class ObserveMixin:
    def _init_observe(self) -> None:
        self.batch_buffer: Dict[str, List[float]] = {}
        self.epoch_history: Dict[str, List[float]] = {}
        self.metric_order: List[str] = []
        self.flush_count_ = 0
        self.flush_times: List[float] = []
        self._traces_validated = False

    def tagged(self, tag: str) -> Optional[Variable]:
        return self.tagged_outputs.get(tag)

    def tag_names_list(self) -> List[str]:
        """All tag names of this graph (`Graph::tag_names()`, observe.rs:44-47; the attribute
        `tag_names` is the name -> node map)."""
        return list(self.tag_names.keys())

    def _expand_groups(self, tags: Sequence[str]) -> List[str]:
        out = []
        for t in tags:
            out.extend(self.tag_groups_map.get(t, [t]))
        return out

    def _note(self, tag: str) -> None:
        if tag not in self.batch_buffer and tag not in self.metric_order:
            self.metric_order.append(tag)

    def collect(self, tags: Sequence[str]) -> None:
        for tag in tags:
            v = self.tagged_outputs.get(tag)
            if v is None:
                continue
            if v.numel() != 1:
                raise TensorError(f'tag "{tag}" has shape {v.shape()} (not scalar); use collect_with() to specify a reduction')
            self._note(tag)
            self.batch_buffer.setdefault(tag, []).append(v.item())

    def collect_with(self, tags: Sequence[str], reduce: Reduce) -> None:
        for tag in self._expand_groups(tags):
            v = self.tagged_outputs.get(tag)
            if v is None:
                continue
            val = v.item() if v.numel() == 1 else reduce.apply(v)
            self._note(tag)
            self.batch_buffer.setdefault(tag, []).append(val)

    def record(self, tag: str, values: Sequence[float]) -> None:
        self._note(tag)
        self.batch_buffer.setdefault(tag, []).extend(float(x) for x in values)

    def record_scalar(self, tag: str, value: float) -> None:
        self.record(tag, [value])

    def collected(self, tag: str) -> List[float]:
        return list(self.batch_buffer.get(tag, []))

    def _child_graphs(self):
        for label, ni in self.children.items():
            mod = self.nodes[ni].module
            g = mod.as_graph() if mod is not None else None
            if g is not None:
                yield label, g

    def latest_metrics_local(self) -> List[Tuple[str, float]]:
        return [(t, self.epoch_history[t][-1]) for t in self.metric_order if self.epoch_history.get(t)]

    def latest_metrics(self) -> List[Tuple[str, float]]:
        out = self.latest_metrics_local()
        for label, g in self._child_graphs():
            out.extend((f"{label}.{t}", v) for t, v in g.latest_metrics())
        return out

    def flush_local(self, tags: Sequence[str] = ()) -> None:
        keys = list(tags) if tags else list(self.batch_buffer.keys())
        flushed = False
        for k in keys:
            vals = self.batch_buffer.pop(k, None)
            if vals:
                self.epoch_history.setdefault(k, []).append(sum(vals) / len(vals))
                flushed = True
        if flushed:
            self.flush_count_ += 1
            self.flush_times.append(time.time() - (self.training_start or time.time()))

    def flush(self, tags: Sequence[str] = ()) -> None:
        """Push the MEAN of every batch buffer to the epoch history; recurses into labelled children."""
        self.flush_local(tags)
        for _, g in self._child_graphs():
            g.flush(())

    def flush_count(self) -> int:
        return self.flush_count_

    def trend(self, tag: str) -> Trend:
        return Trend(self.epoch_history.get(tag, []))

    def trends(self, tags: Sequence[str]) -> TrendGroup:
        return TrendGroup([Trend(self.epoch_history.get(t, [])) for t in self._expand_groups(tags)])

    def reset_trend(self, tags: Sequence[str] = ()) -> None:
        if not tags:
            self.epoch_history.clear()
        else:
            for t in self._expand_groups(tags):
                self.epoch_history.pop(t, None)

    # ---- loop traces ----------------------------------------------------------------------------
    def _validate_trace_namespace(self) -> None:
        if self._traces_validated:
            return
        legacy = {name for name, (ni, _) in self.tag_names.items() if self.nodes[ni].trace_buf is not None}
        seen: Dict[str, str] = {}
        for node in self.nodes:
            if node.named_trace_buf is None:
                continue
            for emit in node.named_trace_buf:
                if emit in legacy:
                    raise TensorError(f'trace namespace collision: emit name "{emit}" from loop "{node.id}" conflicts with a '
                                      "legacy post-loop trace tag of the same name")
                if emit in seen and seen[emit] != node.id:
                    raise TensorError(f'trace namespace collision: emit name "{emit}" published by both loop "{seen[emit]}" '
                                      f'and loop "{node.id}"')
                seen[emit] = node.id
        self._traces_validated = True

    def traces(self, name: str) -> Optional[List[Variable]]:
        self._validate_trace_namespace()
        if name in self.tag_names:
            buf = self.nodes[self.tag_names[name][0]].trace_buf
            if buf:
                return list(buf)
        for node in self.nodes:
            if node.named_trace_buf and node.named_trace_buf.get(name):
                return list(node.named_trace_buf[name])
        for node in self.nodes:
            if node.trace_buf and "loop" in node.id:
                return list(node.trace_buf)
        return None

    def traces_by_node(self, node_id: str) -> Optional[List[Variable]]:
        ni = self.node_index.get(node_id)
        if ni is not None and self.nodes[ni].trace_buf:
            return list(self.nodes[ni].trace_buf)
        return None

    def traces_named(self, name: str) -> Optional[List[Variable]]:
        self._validate_trace_namespace()
        for node in self.nodes:
            if node.named_trace_buf and node.named_trace_buf.get(name):
                return list(node.named_trace_buf[name])
        return None

    def last_trace(self, tag: str) -> Optional[Variable]:
        t = self.traces(tag)
        return t[-1] if t else None

    def eta(self, total_epochs: int) -> float:
        """Seconds left, extrapolated from the flush timestamps (one flush per epoch)."""
        done = self.flush_count_
        if done == 0 or total_epochs <= done or not self.flush_times:
            return 0.0
        return self.flush_times[-1] / done * (total_epochs - done)
