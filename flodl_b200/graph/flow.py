"""`FlowBuilder`: the fluent graph-construction DSL (flodl/src/graph/flow.rs:1-892,
loop_node.rs, switch.rs, gate.rs, map.rs).

Node ids are `"{prefix}_{n}"` with ONE counter shared by every kind of node, where prefix is
the module's `name()` or `add` / `merge` / `input_{name}` / `state_read_{tag}` / `loop` /
`switch` / `gate` / `map` (flow.rs:645-656, :769-852). Checkpoint keys are built from these ids,
so the numbering here reproduces the reference's exactly: `also` consumes two ids (module, then
add), `also_with` three, `input()` one per name, a forward `using()` one per unresolved name.
Errors accumulate in the builder and surface at `build()` (flow.rs:605-641).
"""
from __future__ import annotations

from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..autograd import Variable
from ..nn.module import LoopBodyEmit, Module
from ..tensor import TensorError
from .node import DEFAULT_INPUT, DEFAULT_OUTPUT, Edge, ExposedPort, ForwardRefSpec, Node, NodeRef, extract_refs


class MergeOp(Enum):
    Add = "add"
    Mean = "mean"


def _sum_inputs(inputs: Sequence[Variable]) -> Variable:
    r = inputs[0]
    for v in inputs[1:]:
        r = r.add(v)
    return r


class FlowBuilder:
    def __init__(self, module: Optional[Module] = None):
        from ..nn.activation import Identity
        self.nodes: Dict[str, Node] = {}
        self.edges: List[Edge] = []
        self.inputs: List[ExposedPort] = []
        self.current: List[NodeRef] = []
        self.taps: Dict[str, NodeRef] = {}
        self.on_target: Optional[NodeRef] = None
        self.fork_target: Optional[NodeRef] = None
        self.counter = 0
        self.err: Optional[str] = None
        self.pending: Dict[str, List[str]] = {}
        self.forward_refs: List[ForwardRefSpec] = []
        self.tag_groups: Dict[str, List[str]] = {}
        self._label: Optional[str] = None
        self.internal_tags: set = set()
        self._verbose = False
        ref = self._add_module(module if module is not None else Identity())
        self.inputs.append(ExposedPort(DEFAULT_INPUT, ref.node_id, DEFAULT_INPUT))
        self.on_target = ref
        self.current = [ref]

    # `FlowBuilder::new()` / `FlowBuilder::from(module)`
    @classmethod
    def new(cls) -> "FlowBuilder":
        return cls()

    @classmethod
    def from_module(cls, module: Module) -> "FlowBuilder":
        return cls(module)

    from_ = from_module

    # ---- metadata -------------------------------------------------------------------------------
    def label(self, name: str) -> "FlowBuilder":
        self._label = name
        return self

    def internal(self, tag: str) -> "FlowBuilder":
        self.internal_tags.add(tag)
        return self

    def verbose(self, enabled: bool = True) -> "FlowBuilder":
        self._verbose = enabled
        return self

    # ---- linear flow ----------------------------------------------------------------------------
    def _single(self, what: str) -> bool:
        if self.err is not None:
            return False
        if len(self.current) != 1:
            self.err = f"{what} requires single stream"
            return False
        return True

    def through(self, module: Module) -> "FlowBuilder":
        if not self._single("through"):
            return self
        prev = self.current[0]
        ref = self._add_module(module)
        self.edges.append(Edge(prev.node_id, prev.port, ref.node_id, DEFAULT_INPUT))
        self.on_target = ref
        self.current = [ref]
        return self

    def fork(self, module: Module) -> "FlowBuilder":
        """Side branch: the main stream continues from the node before the fork; the branch
        output can be tagged (`tag` right after `fork` names the branch)."""
        if not self._single("fork"):
            return self
        prev = self.current[0]
        ref = self._add_module(module)
        self.edges.append(Edge(prev.node_id, prev.port, ref.node_id, DEFAULT_INPUT))
        self.on_target = ref
        self.fork_target = ref
        return self

    def also(self, module: Module) -> "FlowBuilder":
        """Residual: out = x + module(x)."""
        if not self._single("also"):
            return self
        prev = self.current[0]
        mref = self._add_module(module)
        aref = self._add_add_node(2)
        self.edges.append(Edge(prev.node_id, prev.port, mref.node_id, DEFAULT_INPUT))
        self.edges.append(Edge(prev.node_id, prev.port, aref.node_id, "input_0"))
        self.edges.append(Edge(mref.node_id, mref.port, aref.node_id, "input_1"))
        self.on_target = mref
        self.current = [aref]
        return self

    def also_with(self, skip: Module, main: Module) -> "FlowBuilder":
        """out = skip(x) + main(x) (projection shortcut)."""
        if not self._single("also_with"):
            return self
        prev = self.current[0]
        sref = self._add_module(skip)
        mref = self._add_module(main)
        aref = self._add_add_node(2)
        self.edges.append(Edge(prev.node_id, prev.port, sref.node_id, DEFAULT_INPUT))
        self.edges.append(Edge(prev.node_id, prev.port, mref.node_id, DEFAULT_INPUT))
        self.edges.append(Edge(sref.node_id, sref.port, aref.node_id, "input_0"))
        self.edges.append(Edge(mref.node_id, mref.port, aref.node_id, "input_1"))
        self.on_target = mref
        self.current = [aref]
        return self

    # ---- tags / refs ----------------------------------------------------------------------------
    def _resolve_pending(self, name: str, ref: NodeRef) -> None:
        for reader_id in self.pending.pop(name, []):
            self.forward_refs.append(ForwardRefSpec(name, reader_id, ref.node_id, ref.port))

    def tag(self, name: str) -> "FlowBuilder":
        if not self._single("tag"):
            return self
        if name in self.taps:
            self.err = f"duplicate tag: {name}"
            return self
        cur = self.fork_target if self.fork_target is not None else self.current[0]
        self.fork_target = None
        self.taps[name] = cur
        self._resolve_pending(name, cur)
        return self

    def tag_group(self, name: str) -> "FlowBuilder":
        if self.err is not None:
            return self
        if len(self.current) < 2:
            self.err = f'tag_group("{name}") requires multiple streams (got {len(self.current)}); use tag for single-stream'
            return self
        if name in self.tag_groups:
            self.err = f'duplicate tag group: "{name}"'
            return self
        if name in self.taps:
            self.err = f'tag group "{name}" conflicts with existing tag'
            return self
        suffixed = []
        for i, cur in enumerate(self.current):
            t = f"{name}_{i}"
            if t in self.taps:
                self.err = f'tag_group("{name}"): suffixed name "{t}" conflicts with existing tag'
                return self
            self.taps[t] = cur
            suffixed.append(t)
            self._resolve_pending(t, cur)
        self.tag_groups[name] = suffixed
        return self

    def input(self, names: Sequence[str]) -> "FlowBuilder":
        """Extra graph inputs, addressable like tags (`forward_multi([x, a, b])` order)."""
        if self.err is not None:
            return self
        for name in names:
            if name in self.taps:
                self.err = f'input tag "{name}" conflicts with existing tag'
                return self
            ref = self._add_input_node(name)
            self.taps[name] = ref
            self.inputs.append(ExposedPort(name, ref.node_id, DEFAULT_INPUT))
            self._resolve_pending(name, ref)
        return self

    def using(self, refs, *more: str) -> "FlowBuilder":
        """Feed tagged values to the preceding node as named refs (`forward_named`). A name that
        is not tagged yet becomes a forward reference: the value of the PREVIOUS forward call.
        Takes a list of names, or the names themselves: `using(["a", "b"])`, `using("a", "b")`."""
        refs = ([refs] if isinstance(refs, str) else list(refs)) + list(more)
        if self.err is not None or not refs:
            return self
        if self.on_target is not None:
            targets = [self.on_target]
        elif len(self.current) > 1:
            targets = list(self.current)
        else:
            self.err = "using requires a preceding through, split, or merge"
            return self
        for t in targets:
            e = self._wire_using(t, refs)
            if e:
                self.err = e
                return self
        return self

    def _wire_using(self, target: NodeRef, refs: Sequence[str]) -> Optional[str]:
        node = self.nodes.get(target.node_id)
        if node is None:
            return f"unknown target node: {target.node_id}"
        if node.module is not None and node.ref_forward is None:
            hint = ("the router must implement NamedInputModule and override as_named_input"
                    if ("gate" in target.node_id or "switch" in target.node_id)
                    else "implement NamedInputModule and override as_named_input on the module")
            return f"node '{target.node_id}' does not support .using() refs — {hint}"
        for name in refs:
            port = f"ref_{name}"
            tap = self.taps.get(name)
            if tap is not None:
                node.input_ports.append(port)
                self.edges.append(Edge(tap.node_id, tap.port, target.node_id, port))
            else:
                reader = self._add_state_read_node(name)
                node.input_ports.append(port)
                self.edges.append(Edge(reader.node_id, reader.port, target.node_id, port))
                self.pending.setdefault(name, []).append(reader.node_id)
        return None

    # ---- fan-out / fan-in -----------------------------------------------------------------------
    def split(self, modules: Sequence[Module]) -> "FlowBuilder":
        if not self._single("split"):
            return self
        if len(modules) < 2:
            self.err = "split requires at least 2 branches"
            return self
        prev = self.current[0]
        branches = []
        for m in modules:
            ref = self._add_module(m)
            self.edges.append(Edge(prev.node_id, prev.port, ref.node_id, DEFAULT_INPUT))
            branches.append(ref)
        self.on_target = None
        self.current = branches
        return self

    def merge(self, op: MergeOp = MergeOp.Add) -> "FlowBuilder":
        if self.err is not None:
            return self
        if len(self.current) < 2:
            self.err = "merge requires multiple streams (after split)"
            return self
        branches = list(self.current)
        ref = self._add_merge_node(len(branches), op)
        for i, b in enumerate(branches):
            self.edges.append(Edge(b.node_id, b.port, ref.node_id, f"input_{i}"))
        self.on_target = ref
        self.current = [ref]
        return self

    # ---- control flow ---------------------------------------------------------------------------
    def loop_body(self, body: Module) -> "LoopBuilder":
        return LoopBuilder(self, body)

    def switch(self, router: Module, branches: Sequence[Module]) -> "FlowBuilder":
        """Hard routing: the router's output `.item()` picks ONE branch (host sync; switch.rs:83-110)."""
        if not self._single("switch"):
            return self
        if len(branches) < 2:
            self.err = "switch requires at least 2 branches"
            return self
        branches = list(branches)

        def route(stream: Variable, refs: Dict[str, Variable]) -> Variable:
            out = router.forward_named(stream, refs) if refs and router.as_named_input() else router.forward(stream)
            idx = int(out.data().reshape(-1)[0].item())
            if idx >= len(branches) or idx < 0:
                raise TensorError(f"switch: router selected branch {idx} but only {len(branches)} branches exist")
            return branches[idx].forward(stream)

        comp = _Composite("switch", [router] + branches, branches[0])
        return self._wire_composite("switch", comp, route, router.as_named_input() is not None)

    def gate(self, router: Module, experts: Sequence[Module]) -> "FlowBuilder":
        """Soft mixture: every expert runs; outputs are stacked on a new last dim, multiplied by
        the router weights `[B, N] -> [B, 1, N]` and summed (gate.rs:84-123)."""
        if not self._single("gate"):
            return self
        if len(experts) < 2:
            self.err = "gate requires at least 2 experts"
            return self
        experts = list(experts)

        def route(stream: Variable, refs: Dict[str, Variable]) -> Variable:
            w = router.forward_named(stream, refs) if refs and router.as_named_input() else router.forward(stream)
            outs = [e.forward(stream) for e in experts]
            stacked = Variable.stack(outs, -1)
            return stacked.mul(w.unsqueeze(-2)).sum_dim(-1, False)

        comp = _Composite("gate", [router] + experts, experts[0])
        return self._wire_composite("gate", comp, route, router.as_named_input() is not None)

    def map(self, body: Module) -> "MapBuilder":
        return MapBuilder(self, body)

    def _wire_composite(self, prefix: str, comp: Module, route: Callable, supports_refs: bool) -> "FlowBuilder":
        cur = self.current[0]
        nid = self.next_id(prefix)
        node = Node(nid, [DEFAULT_INPUT], [DEFAULT_OUTPUT], None, comp)
        node.run = lambda inputs, n=node: [route(inputs[0], extract_refs(n.input_ports, inputs))]
        node.ref_forward = route if supports_refs else None
        self.nodes[nid] = node
        self.edges.append(Edge(cur.node_id, cur.port, nid, DEFAULT_INPUT))
        ref = NodeRef(nid, DEFAULT_OUTPUT)
        self.current = [ref]
        self.on_target = ref
        return self

    # ---- build ----------------------------------------------------------------------------------
    def build(self):
        from .graph import Graph
        if self.err is not None:
            raise TensorError(self.err)
        if self.pending:
            raise TensorError(f"unresolved forward refs: {sorted(self.pending.keys())}")
        if len(self.current) != 1:
            raise TensorError("open streams: call merge before build")
        out = ExposedPort(DEFAULT_OUTPUT, self.current[0].node_id, self.current[0].port)
        return Graph(self.nodes, self.edges, self.inputs, [out], self.taps, self.forward_refs, self.tag_groups,
                     self._label, set(self.internal_tags), self._verbose)

    # ---- helpers --------------------------------------------------------------------------------
    def next_id(self, prefix: str) -> str:
        self.counter += 1
        return f"{prefix}_{self.counter}"

    def _add_module(self, module: Module) -> NodeRef:
        nid = self.next_id(module.name())
        node = Node(nid, [DEFAULT_INPUT], [DEFAULT_OUTPUT], None, module)
        if module.as_named_input() is not None:
            node.ref_forward = lambda x, refs, m=module: m.forward_named(x, refs)

        def run(inputs, n=node, m=module):
            refs = extract_refs(n.input_ports, inputs) if len(n.input_ports) > 1 else None
            return [m.forward_named(inputs[0], refs) if refs else m.forward(inputs[0])]

        node.run = run
        self.nodes[nid] = node
        return NodeRef(nid, DEFAULT_OUTPUT)

    def _add_add_node(self, n: int) -> NodeRef:
        nid = self.next_id("add")
        self.nodes[nid] = Node(nid, [f"input_{i}" for i in range(n)], [DEFAULT_OUTPUT], lambda inputs: [_sum_inputs(inputs)], None)
        return NodeRef(nid, DEFAULT_OUTPUT)

    def _add_merge_node(self, n: int, op: MergeOp) -> NodeRef:
        nid = self.next_id("merge")
        if op == MergeOp.Mean:
            run = lambda inputs: [_sum_inputs(inputs).mul_scalar(1.0 / n)]
        else:
            run = lambda inputs: [_sum_inputs(inputs)]
        self.nodes[nid] = Node(nid, [f"input_{i}" for i in range(n)], [DEFAULT_OUTPUT], run, None)
        return NodeRef(nid, DEFAULT_OUTPUT)

    def _add_state_read_node(self, ref_name: str) -> NodeRef:
        nid = self.next_id(f"state_read_{ref_name}")
        node = Node(nid, [], [DEFAULT_OUTPUT], None, None)
        node.is_state_read = True
        self.nodes[nid] = node
        return NodeRef(nid, DEFAULT_OUTPUT)

    def _add_input_node(self, name: str) -> NodeRef:
        nid = self.next_id(f"input_{name}")
        self.nodes[nid] = Node(nid, [DEFAULT_INPUT], [DEFAULT_OUTPUT], lambda inputs: list(inputs), None)
        return NodeRef(nid, DEFAULT_OUTPUT)


class _Composite(Module):
    """Module shell of a control-flow node: exposes the sub-modules' parameters under the node's
    prefix and forwards to a representative branch."""

    def __init__(self, kind: str, subs: List[Module], rep: Module):
        self._kind, self._subs, self._rep = kind, subs, rep
        # data-dependent control flow: which parameters receive a gradient can change from step to step
        self.dynamic = kind == "switch"

    def name(self): return "module"   # composites keep the trait's default name in the reference
    def forward(self, x): return self._rep.forward(x)
    def sub_modules(self): return list(self._subs)
    def reset(self):
        for m in self._subs:
            m.reset()
    def detach_state(self):
        for m in self._subs:
            m.detach_state()


class LoopBuilder:
    """`fb.loop_body(body).for_n(n) | .while_cond(cond, max) | .until_cond(cond, max)`
    (flodl/src/graph/loop_node.rs). `body.reset()` runs before iterating; `while` tests the halt
    module before each iteration (halt when `cond(state)[0] > 0`), `until` tests after and skips
    the test on the last iteration. Per-iteration traces: `body.trace()` (legacy) or named emits
    from `body.step(state, refs, emit)`; both are cleared at the start of every forward."""

    def __init__(self, fb: FlowBuilder, body: Module):
        self.fb, self.body = fb, body

    def _check(self, n: int, msg: str) -> bool:
        fb = self.fb
        if fb.err is not None:
            return False
        if len(fb.current) != 1:
            fb.err = "loop requires single stream"
            return False
        if n < 1:
            fb.err = msg
            return False
        return True

    def for_n(self, n: int) -> FlowBuilder:
        if not self._check(n, "loop requires at least 1 iteration"):
            return self.fb
        return self._wire("for", n, None)

    def while_cond(self, cond: Module, max_iter: int) -> FlowBuilder:
        if not self._check(max_iter, "loop requires max_iter >= 1"):
            return self.fb
        return self._wire("while", max_iter, cond)

    def until_cond(self, cond: Module, max_iter: int) -> FlowBuilder:
        if not self._check(max_iter, "loop requires max_iter >= 1"):
            return self.fb
        return self._wire("until", max_iter, cond)

    def _wire(self, kind: str, count: int, cond: Optional[Module]) -> FlowBuilder:
        fb, body = self.fb, self.body
        cur = fb.current[0]
        nid = fb.next_id("loop")
        comp = _Composite("loop", [body] + ([cond] if cond is not None else []), body)
        comp.dynamic = kind in ("while", "until")
        node = Node(nid, [DEFAULT_INPUT], [DEFAULT_OUTPUT], None, comp)
        node.trace_buf = []
        node.named_trace_buf = {}

        def halted(state: Variable, i: int) -> bool:
            try:
                v = cond.forward(state).data().reshape(-1)
            except Exception as e:
                raise TensorError(f"loop condition at iteration {i}: {e}")
            return v.numel() > 0 and float(v[0].item()) > 0.0

        def iteration(state: Variable, refs: Dict[str, Variable], i: int) -> Variable:
            try:
                if body.as_loop_body() is not None:
                    emit = LoopBodyEmit()
                    nxt = body.step(state, refs, emit)
                    for k, vs in emit.values.items():
                        node.named_trace_buf.setdefault(k, []).extend(vs)
                    return nxt
                nxt = body.forward_named(state, refs) if refs and body.as_named_input() is not None else body.forward(state)
                t = body.trace()
                if t is not None:
                    node.trace_buf.append(t)
                return nxt
            except TensorError as e:
                raise TensorError(f"loop iteration {i}: {e}")

        def run(inputs):
            state = inputs[0]
            refs = extract_refs(node.input_ports, inputs)
            node.trace_buf.clear()
            node.named_trace_buf.clear()
            body.reset()
            for i in range(count):
                if kind == "while" and halted(state, i):
                    break
                state = iteration(state, refs, i)
                if kind == "until" and i < count - 1 and halted(state, i):
                    break
            return [state]

        node.run = run
        if body.as_named_input() is not None:
            node.ref_forward = lambda x, refs: body.forward_named(x, refs)
        fb.nodes[nid] = node
        fb.edges.append(Edge(cur.node_id, cur.port, nid, DEFAULT_INPUT))
        ref = NodeRef(nid, DEFAULT_OUTPUT)
        fb.current = [ref]
        fb.on_target = ref
        return fb


class MapBuilder:
    """`fb.map(body).each() | .over(tag) | .slices(n)`, optionally `.batched()` first
    (flodl/src/graph/map.rs): apply `body` to every dim-0 element and concatenate; `batched`
    hands the whole tensor to the body in one call; `slices(n)` reshapes `[B, D]` to
    `[B*n, D/n]`, maps, and folds back to `[B, out*n]`."""

    def __init__(self, fb: FlowBuilder, body: Module):
        self.fb, self.body, self._batched = fb, body, False

    def batched(self) -> "MapBuilder":
        self._batched = True
        return self

    def _ok(self) -> bool:
        fb = self.fb
        if fb.err is not None:
            return False
        if len(fb.current) != 1:
            fb.err = "map requires single stream"
            return False
        return True

    def each(self) -> FlowBuilder:
        if not self._ok():
            return self.fb
        return self._wire(self.fb.current[0], self._each_fn())

    def over(self, tag: str) -> FlowBuilder:
        if not self._ok():
            return self.fb
        src = self.fb.taps.get(tag)
        if src is None:
            self.fb.err = f'Map.over("{tag}") references unknown tag; Map requires a backward reference'
            return self.fb
        return self._wire(src, self._each_fn())

    def slices(self, n: int) -> FlowBuilder:
        if not self._ok():
            return self.fb
        if n < 1:
            self.fb.err = f"Map.slices requires n >= 1 (got {n})"
            return self.fb
        body, batched = self.body, self._batched

        def run(inputs):
            src = inputs[0]
            shape = src.shape()
            if len(shape) < 2:
                raise TensorError(f"map slices: input must be at least 2D (got {len(shape)}D)")
            last = shape[-1]
            if last % n:
                raise TensorError(f"map slices: last dim {last} not divisible by {n}")
            b0 = shape[0]
            dec = src.reshape([b0 * n, last // n])
            if batched:
                r = body.forward(dec)
            else:
                r = Variable.cat_many([body.forward(dec.narrow(0, i, 1)) for i in range(b0 * n)], 0)
            return [r.reshape([b0, r.shape()[1] * n])]

        return self._wire(self.fb.current[0], run)

    def _each_fn(self):
        body, batched = self.body, self._batched

        def run(inputs):
            s = inputs[0]
            if batched:
                return [body.forward(s)]
            n = s.shape()[0]
            if n == 0:
                return [s]
            return [Variable.cat_many([body.forward(s.narrow(0, i, 1)) for i in range(n)], 0)]

        return run

    def _wire(self, source: NodeRef, run) -> FlowBuilder:
        fb = self.fb
        nid = fb.next_id("map")
        fb.nodes[nid] = Node(nid, [DEFAULT_INPUT], [DEFAULT_OUTPUT], run, self.body)
        fb.edges.append(Edge(source.node_id, source.port, nid, DEFAULT_INPUT))
        ref = NodeRef(nid, DEFAULT_OUTPUT)
        fb.current = [ref]
        fb.on_target = ref
        return fb
