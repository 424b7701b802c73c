"""Build-time and run-time records of the dataflow graph (flodl/src/graph/node.rs:1-120)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..autograd import Variable
from ..nn.module import Module

DEFAULT_INPUT = "input"
DEFAULT_OUTPUT = "output"


@dataclass
class Edge:
    from_node: str
    from_port: str
    to_node: str
    to_port: str


@dataclass
class NodeRef:
    node_id: str
    port: str


@dataclass
class ExposedPort:
    name: str
    node_id: str
    port: str


@dataclass
class ForwardRefSpec:
    """`using(x)` before `tag(x)`: the reader node yields the writer's value of the previous call."""
    name: str
    reader_id: str
    writer_id: str
    writer_port: str


class Node:
    __slots__ = ("id", "input_ports", "output_ports", "run", "module", "ref_forward", "trace_buf", "named_trace_buf",
                 "is_state_read")

    def __init__(self, id: str, input_ports: List[str], output_ports: List[str], run: Optional[Callable], module: Optional[Module]):
        self.id = id
        self.input_ports = input_ports
        self.output_ports = output_ports
        self.run = run
        self.module = module
        self.ref_forward = None
        self.trace_buf: Optional[List[Variable]] = None
        self.named_trace_buf: Optional[Dict[str, List[Variable]]] = None
        self.is_state_read = False


def extract_refs(ports: Sequence[str], inputs: Sequence[Variable]) -> Dict[str, Variable]:
    """`ref_*` ports -> {name: value} (node.rs `extract_refs`)."""
    refs = {}
    for i, port in enumerate(ports):
        if port.startswith("ref_") and i < len(inputs):
            refs[port[4:]] = inputs[i]
    return refs
