"""Pieces shared by the encoder families: a generic config base, small head modules."""
from __future__ import annotations

import json
from dataclasses import replace
from typing import Dict, List, Optional

import torch

from ...autograd import Variable
from ...nn.layers import Dropout, Linear
from ...nn.module import Module, Parameter
from .. import config_json as cj
from ..path import prefix_params


def attach(graph, config):
    graph.set_source_config(config.to_json_str())
    return graph


def zeros_bias(n: int, device=None) -> Parameter:
    d = None if device is None else (device.torch if hasattr(device, "torch") else torch.device(str(device)))
    return Parameter(torch.zeros(n, device=d), "bias")


def label_fields(v):
    id2label = cj.parse_id2label(v)
    return dict(num_labels=cj.parse_num_labels(v, id2label), id2label=id2label, architectures=cj.parse_architectures(v))


def emit_labels(m: dict, cfg) -> dict:
    if cfg.id2label:
        m["id2label"] = cj.emit_id2label(cfg.id2label)
        m["label2id"] = {l: i for i, l in enumerate(cfg.id2label)}
    elif cfg.num_labels is not None:
        m["num_labels"] = cfg.num_labels
    return m


def need_num_labels(cfg, what: str) -> int:
    if cfg.num_labels is None:
        from ...tensor import TensorError
        raise TensorError(f"{what}: config.json has no `num_labels` (nor `id2label`); cannot infer head size")
    return cfg.num_labels


class SelectCls(Module):
    """`x[:, 0]` — the first token's hidden state."""
    def name(self): return "select_cls"
    def forward(self, x): return x.select(1, 0).contiguous()


class SelectClsLinear(Module):
    def __init__(self, linear: Linear): self.linear = linear
    def name(self): return "select_cls_linear"
    def own_parameters(self): return self.linear.own_parameters()
    def forward(self, x): return self.linear.forward(x.select(1, 0).contiguous())


class ActivationDropoutLinear(Module):
    """relu -> dropout -> linear (DistilBERT's classifier tail)."""
    def __init__(self, p: float, linear: Linear):
        self.dropout, self.linear = Dropout(p), linear
    def name(self): return "activation_dropout_linear"
    def sub_modules(self): return [self.dropout]
    def own_parameters(self): return self.linear.own_parameters()
    def forward(self, x): return self.linear.forward(self.dropout.forward(x.relu()))
