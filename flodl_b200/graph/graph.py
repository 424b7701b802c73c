"""`Graph`: the executable dataflow graph a `FlowBuilder` produces (flodl/src/graph/graph.rs).

Build: nodes are indexed in insertion order, Kahn levels give the execution order (ties broken by
node index so the order - and with it `named_parameters()` and the structural hash - is
deterministic, graph.rs:1276-1324), routes and input slots are precomputed. The level computation
and SHA-256 run in the C++ runtime.

Run: levels in order; each node gathers its input slots (an unconnected `ref_*` slot is filled
with zeros shaped like the primary input, which is how forward references start), executes, and
routes its outputs; tagged outputs and forward-reference state are captured on the way
(graph.rs:440-619).

A `Graph` is itself a `Module`, so graphs nest; labelled children form the graph tree (tree.py).
Observation, profiling, rendering, and the data-parallel driver are mixed in from sibling files.
"""
from __future__ import annotations

import json
import os
import struct
import time
from typing import Dict, List, Optional, Sequence, Set, Tuple

import torch

from .. import _ext
from ..autograd import Variable
from ..nn import checkpoint as _ckpt
from ..nn.module import Buffer, Module, Parameter, walk_modules
from ..tensor import Device, TensorError
from .distributed import DistributedMixin
from .node import DEFAULT_INPUT, Edge, ExposedPort, ForwardRefSpec, Node, NodeRef
from .observe import ObserveMixin
from .profile import ProfileMixin
from .render import RenderMixin
from .tree import TreeMixin


def topological_levels(n: int, edges: Sequence[Tuple[int, int]]) -> List[List[int]]:
    C = _ext.load()
    if C is not None and hasattr(C, "topo_levels"):
        try:
            return C.topo_levels(n, list(edges))
        except RuntimeError as e:
            raise TensorError(str(e))
    deps = [set() for _ in range(n)]
    dependents = [set() for _ in range(n)]
    for a, b in edges:
        deps[b].add(a)
        dependents[a].add(b)
    indeg = [len(d) for d in deps]
    queue = [i for i in range(n) if indeg[i] == 0]
    levels, visited = [], 0
    while queue:
        levels.append(list(queue))
        visited += len(queue)
        nxt = []
        for ni in queue:
            for d in sorted(dependents[ni]):
                indeg[d] -= 1
                if indeg[d] == 0:
                    nxt.append(d)
        queue = nxt
    if visited != n:
        raise TensorError("cycle detected in graph")
    return levels


class Graph(Module, TreeMixin, ObserveMixin, ProfileMixin, RenderMixin, DistributedMixin):
    def __init__(self, node_map: Dict[str, Node], edges: List[Edge], inputs: List[ExposedPort], outputs: List[ExposedPort],
                 tags: Dict[str, NodeRef], forward_refs: List[ForwardRefSpec], tag_groups: Dict[str, List[str]],
                 label: Optional[str], internal_tags: Set[str], verbose: bool):
        self.nodes: List[Node] = list(node_map.values())
        self.node_index: Dict[str, int] = {n.id: i for i, n in enumerate(self.nodes)}
        self.edges = edges
        self.inputs, self.outputs = inputs, outputs
        self.tag_groups_map = tag_groups
        self._label = label
        self.internal_tags_set = set(internal_tags)
        for e in edges:
            if e.from_node not in self.node_index:
                raise TensorError(f"unknown source node: {e.from_node}")
            if e.to_node not in self.node_index:
                raise TensorError(f"unknown target node: {e.to_node}")

        # forward-reference state
        self.state: List[dict] = []
        for fr in forward_refs:
            entry = {"name": fr.name, "value": None, "writer_ni": self.node_index.get(fr.writer_id, 0)}
            self.state.append(entry)
            reader = node_map.get(fr.reader_id)
            if reader is not None:
                reader.run = (lambda inputs, e=entry: [e["value"]] if e["value"] is not None else [])

        try:
            self.levels = topological_levels(len(self.nodes), [(self.node_index[e.from_node], self.node_index[e.to_node]) for e in edges])
        except RuntimeError as e:
            raise TensorError(str(e).split("\n")[0])
        self.order: List[int] = [ni for lvl in self.levels for ni in lvl]

        # tags
        self.tag_names: Dict[str, Tuple[int, int]] = {}
        self.tag_capture: Dict[int, List[Tuple[str, int]]] = {}
        for name, ref in tags.items():
            ni = self.node_index.get(ref.node_id)
            if ni is None:
                continue
            ports = self.nodes[ni].output_ports
            pi = ports.index(ref.port) if ref.port in ports else 0
            self.tag_names[name] = (ni, pi)
            self.tag_capture.setdefault(ni, []).append((name, pi))

        # labelled child graphs form the tree
        self.children: Dict[str, int] = {}
        self.composed = False
        for idx, node in enumerate(self.nodes):
            child = node.module.as_graph() if node.module is not None else None
            if child is None or child.label() is None:
                continue
            lbl = child.label()
            if "." in lbl:
                raise TensorError(f'child graph label "{lbl}" contains a dot — dots are reserved for path separators')
            if lbl in self.children:
                raise TensorError(f'duplicate child graph label "{lbl}" at the same tree level')
            if lbl in self.tag_names and self.tag_names[lbl][0] != idx:
                raise TensorError(f'child graph label "{lbl}" collides with a tag on a different node')
            self.children[lbl] = idx
            child.composed = True
        for name in self.tag_names:
            if name.startswith("_"):
                self.internal_tags_set.add(name)

        self.state_writers: Dict[int, List[Tuple[int, int]]] = {}
        for si, fr in enumerate(forward_refs):
            ni = self.node_index.get(fr.writer_id)
            if ni is None:
                continue
            ports = self.nodes[ni].output_ports
            self.state_writers.setdefault(ni, []).append((si, ports.index(fr.writer_port) if fr.writer_port in ports else 0))

        # routing tables
        n = len(self.nodes)
        self.routes_from: List[List[Tuple[int, int, int]]] = [[] for _ in range(n)]
        for e in edges:
            f, t = self.node_index[e.from_node], self.node_index[e.to_node]
            fp = self.nodes[f].output_ports.index(e.from_port) if e.from_port in self.nodes[f].output_ports else 0
            tp = self.nodes[t].input_ports.index(e.to_port) if e.to_port in self.nodes[t].input_ports else 0
            self.routes_from[f].append((fp, t, tp))
        self.input_routes: List[Tuple[int, int]] = []
        for ep in inputs:
            ni = self.node_index[ep.node_id]
            ports = self.nodes[ni].input_ports
            self.input_routes.append((ni, ports.index(ep.port) if ep.port in ports else 0))
        self.output_node_idx = self.node_index[outputs[0].node_id]
        oports = self.nodes[self.output_node_idx].output_ports
        self.output_port_idx = oports.index(outputs[0].port) if outputs[0].port in oports else 0
        self.node_input_count = [len(nd.input_ports) for nd in self.nodes]

        self.tagged_outputs: Dict[str, Variable] = {}
        self._hash_cache: Optional[str] = None
        self._source_config: Optional[str] = None
        self.training_start = 0.0
        self.step_count_ = 0
        self.epoch_count_ = 0
        self.training = True
        self._init_observe()
        self._init_profile()
        self._init_distributed()
        if verbose:
            from ..log import verbose as _vlog
            _vlog(self.tree_summary())

    # ---- Module ---------------------------------------------------------------------------------
    def name(self) -> str:
        return "graph"

    def as_graph(self):
        return self

    def label(self) -> Optional[str]:
        return self._label

    def sub_modules(self) -> List[Module]:
        return [n.module for n in self.nodes if n.module is not None]

    def as_loop_body(self):
        # `step()` on a graph is the distributed training step, not the loop-body protocol
        return None

    def forward(self, x) -> Variable:
        if self.is_distributed():
            return self.forward_distributed(x)
        if isinstance(x, (list, tuple)):
            return self.forward_multi(x)
        return self.forward_impl([x if isinstance(x, Variable) else Variable.wrap(x)])

    def forward_multi(self, inputs: Sequence[Variable]) -> Variable:
        return self.forward_impl([v if isinstance(v, Variable) else Variable.wrap(v) for v in inputs])

    def forward_impl(self, graph_inputs: Sequence[Variable]) -> Variable:
        if len(graph_inputs) != len(self.inputs):
            raise TensorError(f"expected {len(self.inputs)} inputs, got {len(graph_inputs)}")
        if self.training_start == 0.0:
            self.training_start = time.time()
        profiling = self._profiling
        if not profiling:
            ex = self._native_exec()
            if ex is not None:
                try:
                    final, tagged, state = ex.forward(list(graph_inputs))
                except RuntimeError as e:
                    if type(e) is RuntimeError and str(e).startswith(("node '", "expected ", "graph produced")):
                        raise TensorError(str(e)) from None          # the walk's own complaints keep the framework's error type
                    raise
                if self.tag_capture:
                    self.tagged_outputs.clear()
                    self.tagged_outputs.update(tagged)
                for si, v in state:
                    self.state[si]["value"] = v
                return final
        t_fwd = time.perf_counter() if profiling else 0.0
        prof_nodes, prof_levels = [], []
        slots: List[List[Optional[Variable]]] = [[None] * c for c in self.node_input_count]
        has_tags = bool(self.tag_capture)
        if has_tags:
            self.tagged_outputs.clear()
        for i, (ni, pi) in enumerate(self.input_routes):
            slots[ni][pi] = graph_inputs[i]
        final = None
        for li, level in enumerate(self.levels):
            t_lvl = time.perf_counter() if profiling else 0.0
            lvl_sum = 0.0
            for ni in level:
                node = self.nodes[ni]
                ins = slots[ni]
                if len(ins) != len(node.input_ports):      # ports added by a late .using()
                    ins = ins + [None] * (len(node.input_ports) - len(ins))
                for i, v in enumerate(ins):
                    if v is None:
                        if i > 0:
                            first = ins[0]
                            if first is None:
                                raise TensorError(f"node '{node.id}': ref port {i} has no data and primary input is also missing — "
                                                  "check that all inputs are connected")
                            ins[i] = Variable.wrap(torch.zeros_like(first.t))
                        elif node.input_ports:
                            raise TensorError(f"node '{node.id}': missing primary input (port {i}) — check that all inputs to this "
                                              "node are connected in the graph builder")
                slots[ni] = []
                t_node = time.perf_counter() if profiling else 0.0
                outs = node.run(ins)
                if profiling:
                    dt = time.perf_counter() - t_node
                    lvl_sum += dt
                    prof_nodes.append((node.id, self._first_tag(ni), dt, li))
                for fp, tn, tp in self.routes_from[ni]:
                    slots[tn][tp] = outs[fp] if fp < len(outs) else None
                for si, pi in self.state_writers.get(ni, ()):
                    if pi < len(outs):
                        self.state[si]["value"] = outs[pi]
                if has_tags:
                    for tag, pi in self.tag_capture.get(ni, ()):
                        if pi < len(outs):
                            self.tagged_outputs[tag] = outs[pi]
                if ni == self.output_node_idx:
                    final = outs
            if profiling:
                prof_levels.append((li, time.perf_counter() - t_lvl, lvl_sum, len(level)))
        if profiling:
            self._store_profile(time.perf_counter() - t_fwd, prof_levels, prof_nodes)
        if final is None or self.output_port_idx >= len(final):
            raise TensorError("graph produced no output")
        return final[self.output_port_idx]

    def _native_exec(self):
        """The C++ walk over this graph's precomputed tables (`csrc/runtime/graph_exec.cpp`), built at the first call;
        None when the native library is not there (the Python walk below does the same) or `FLODL_B200_NATIVE_GRAPH=0`."""
        ex = self.__dict__.get("_exec")
        if ex is not None or self.__dict__.get("_exec_unavailable"):
            return ex
        from .. import _ext
        if os.environ.get("FLODL_B200_NATIVE_GRAPH", "1") in ("0", "false", "off") or not _ext.available() or not hasattr(_ext.require(), "GraphExec"):
            self._exec_unavailable = True
            return None
        n = len(self.nodes)
        self._exec = _ext.require().GraphExec(
            [list(level) for level in self.levels], [int(c) for c in self.node_input_count], [len(nd.input_ports) for nd in self.nodes],
            [(int(ni), int(pi)) for ni, pi in self.input_routes], [[(int(fp), int(tn), int(tp)) for fp, tn, tp in self.routes_from[i]] for i in range(n)],
            [[(int(si), int(pi)) for si, pi in self.state_writers.get(i, ())] for i in range(n)],
            [[(str(tag), int(pi)) for tag, pi in self.tag_capture.get(i, ())] for i in range(n)],
            int(self.output_node_idx), int(self.output_port_idx), [nd.run for nd in self.nodes], [str(nd.id) for nd in self.nodes],
            lambda v: Variable.wrap(torch.zeros_like(v.t)))
        return self._exec

    def _first_tag(self, ni: int) -> str:
        caps = self.tag_capture.get(ni)
        return caps[0][0] if caps else ""

    # ---- forward-reference state ----------------------------------------------------------------
    def has_state(self) -> bool:
        return bool(self.state)

    def reset_state(self) -> None:
        for s in self.state:
            s["value"] = None
        for m in self.sub_modules():
            m.reset()

    def detach_state(self) -> None:
        for s in self.state:
            if s["value"] is not None:
                s["value"] = s["value"].detach()
        for k, v in list(self.tagged_outputs.items()):
            self.tagged_outputs[k] = v.detach()
        for m in self.sub_modules():
            m.detach_state()

    def reset(self) -> None:
        self.reset_state()

    def end_step(self) -> None:
        """After an optimizer step inside a sequence: keep the state values, cut their history."""
        self.detach_state()
        self.step_count_ += 1

    def end_sequence(self) -> None:
        self.reset_state()

    def end_epoch(self) -> None:
        self.reset_state()
        self.epoch_count_ += 1

    def step_count(self) -> int:
        return self.step_count_

    def epoch_count(self) -> int:
        return self.epoch_count_

    def tag_group(self, name: str) -> List[str]:
        return list(self.tag_groups_map.get(name, []))

    # ---- parameters -----------------------------------------------------------------------------
    def set_device(self, device) -> None:
        self.move_to_device(device)

    def _named(self, kind: str):
        idx_to_tag: Dict[int, str] = {}
        for tag, (ni, _) in self.tag_names.items():
            idx_to_tag.setdefault(ni, tag)
        out, seen = [], set()
        for ni in self.order:
            mod = self.nodes[ni].module
            if mod is None:
                continue
            prefix = idx_to_tag.get(ni, self.nodes[ni].id)
            items = mod.parameters() if kind == "p" else mod.buffers()
            counts: Dict[str, int] = {}
            for it in items:
                counts[it.name] = counts.get(it.name, 0) + 1
            running: Dict[str, int] = {}
            for it in items:
                if it.key() in seen:
                    continue
                seen.add(it.key())
                if counts[it.name] > 1:
                    k = running.get(it.name, 0)
                    running[it.name] = k + 1
                    out.append((f"{prefix}/{it.name}_{k}", it))
                else:
                    out.append((f"{prefix}/{it.name}", it))
        return out

    def named_parameters(self) -> List[Tuple[str, Parameter]]:
        """`"{tag or node id}/{param name}"`; duplicates within a node get `_0, _1, ...`
        (graph.rs:768-814). The first tag of a node wins as prefix."""
        return self._named("p")

    def named_buffers(self) -> List[Tuple[str, Buffer]]:
        return self._named("b")

    def parameters(self) -> List[Parameter]:
        return [p for _, p in self.named_parameters()]

    def buffers(self) -> List[Buffer]:
        return [b for _, b in self.named_buffers()]

    # ---- structural hash ------------------------------------------------------------------------
    def structural_hash(self) -> str:
        """SHA-256 over node ids, module names, sorted parameter/buffer names+shapes, nested graph
        hashes, edges, sorted tags and the exposed ports (graph.rs:943-1037). The label is not hashed."""
        if self._hash_cache is None:
            self._hash_cache = self._compute_hash()
        return self._hash_cache

    def short_hash(self) -> str:
        return self.structural_hash()[:8]

    def _compute_hash(self) -> str:
        b = bytearray()
        for ni in self.order:
            node = self.nodes[ni]
            b += node.id.encode() + b"\0"
            mod = node.module
            if mod is None:
                continue
            b += mod.name().encode() + b"\0"
            for nm, shape in sorted((p.name, p.shape()) for p in mod.parameters()):
                b += b"P" + nm.encode() + b"\0" + b"".join(struct.pack("<q", d) for d in shape)
            for nm, shape in sorted((x.name, x.shape()) for x in mod.buffers()):
                b += b"B" + nm.encode() + b"\0" + b"".join(struct.pack("<q", d) for d in shape)
            nested = mod.structural_hash()
            if nested is not None:
                b += b"G" + nested.encode()
        b += b"EDGES"
        for e in self.edges:
            b += e.from_node.encode() + b"\0" + e.from_port.encode() + b"\0" + e.to_node.encode() + b"\0" + e.to_port.encode() + b"\0"
        b += b"TAGS"
        for name in sorted(self.tag_names):
            ni, pi = self.tag_names[name]
            b += name.encode() + b"\0" + struct.pack("<QQ", ni, pi)
        b += b"INPUTS"
        for p in self.inputs:
            b += p.name.encode() + b"\0" + p.node_id.encode() + b"\0" + p.port.encode() + b"\0"
        b += b"OUTPUTS"
        for p in self.outputs:
            b += p.name.encode() + b"\0" + p.node_id.encode() + b"\0" + p.port.encode() + b"\0"
        C = _ext.load()
        if C is not None:
            return C.sha256_hex(bytes(b))
        import hashlib
        return hashlib.sha256(bytes(b)).hexdigest()

    # ---- checkpoints ----------------------------------------------------------------------------
    def set_source_config(self, config_json: str) -> None:
        self._source_config = config_json

    def source_config(self) -> Optional[str]:
        return self._source_config

    def clear_source_config(self) -> None:
        self._source_config = None

    def snapshot_cpu(self):
        """Host copies of every named parameter and buffer, to be written later off the training
        thread (`ModelSnapshot.save_file`; flodl/src/graph/snapshot.rs:90-120)."""
        from .snapshot import snapshot_cpu
        return snapshot_cpu(self)

    def save_checkpoint(self, path: str) -> None:
        """`.fdl` (gzip if the path ends in .gz) + `<stem>.config.json` sidecar when a source config
        is attached (graph.rs:891-907, :1046-1054)."""
        _ckpt.save_checkpoint_file(path, self.named_parameters(), self.named_buffers(), self.structural_hash())
        if self._source_config is not None:
            with open(sidecar_config_path(path), "w") as f:
                f.write(self._source_config)

    def load_checkpoint(self, path: str) -> _ckpt.LoadReport:
        return _ckpt.load_checkpoint_file(path, self.named_parameters(), self.named_buffers(), self.structural_hash())


def sidecar_config_path(checkpoint: str) -> str:
    p = checkpoint[:-3] if checkpoint.endswith(".gz") else checkpoint
    stem, _ = os.path.splitext(p)
    return stem + ".config.json"
