"""ALBERT (flodl-hf/src/models/albert.rs): factorised embeddings (`embedding_size` -> Linear ->
`hidden_size`), ONE encoder block applied `num_hidden_layers` times (its parameters appear once,
under `albert.encoder.albert_layer_groups.0.albert_layers.0`), a flat-Linear pooler
(`albert.pooler.{weight,bias}`). Only `num_hidden_groups == inner_group_num == 1` is supported, as
in every published checkpoint."""
from __future__ import annotations

import json
from dataclasses import dataclass, replace
from typing import Dict, List, Optional

import torch

from ... import ops as _ops
from ...autograd import Variable
from ...graph import FlowBuilder, Graph
from ...nn.activation import GeluApprox
from ...nn.layers import Dropout, Embedding, LayerNorm, Linear
from ...nn.module import Module, Parameter
from ...tensor import TensorError
from .. import config_json as cj
from ..path import HfPath, prefix_params
from ..task_heads import ClassificationHead, MaskedLmHead, QaHead, TaggingHead, TiedDecoder, check_num_labels
from ..transformer_layer import LayerNaming, TransformerLayer, TransformerLayerConfig
from ._common import attach, emit_labels, label_fields, need_num_labels, zeros_bias
from .bert import build_extended_attention_mask


@dataclass
class AlbertConfig:
    vocab_size: int = 30000
    embedding_size: int = 128
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    pad_token_id: Optional[int] = 0
    layer_norm_eps: float = 1e-12
    hidden_dropout_prob: float = 0.0
    attention_probs_dropout_prob: float = 0.0
    hidden_act: GeluApprox = GeluApprox.Tanh
    num_labels: Optional[int] = None
    id2label: Optional[List[str]] = None
    architectures: Optional[List[str]] = None

    MODEL_TYPE = "albert"
    FAMILY_NAME = "Albert"
    MASK_TOKEN = "[MASK]"

    @classmethod
    def albert_base_v2(cls): return cls()

    @classmethod
    def from_json_str(cls, s: str):
        v = cj.parse(s)
        for key in ("num_hidden_groups", "inner_group_num"):
            if cj.optional_i64(v, key, 1) != 1:
                raise TensorError(f"AlbertConfig: {key} = {cj.optional_i64(v, key, 1)} is not supported — only 1 (every published ALBERT checkpoint)")
        return cls(vocab_size=cj.required_i64(v, "vocab_size"), embedding_size=cj.required_i64(v, "embedding_size"),
                   hidden_size=cj.required_i64(v, "hidden_size"), num_hidden_layers=cj.required_i64(v, "num_hidden_layers"),
                   num_attention_heads=cj.required_i64(v, "num_attention_heads"), intermediate_size=cj.required_i64(v, "intermediate_size"),
                   max_position_embeddings=cj.required_i64(v, "max_position_embeddings"), type_vocab_size=cj.optional_i64(v, "type_vocab_size", 2),
                   pad_token_id=cj.optional_i64_or_none(v, "pad_token_id"), layer_norm_eps=cj.optional_f64(v, "layer_norm_eps", 1e-12),
                   hidden_dropout_prob=cj.optional_f64(v, "hidden_dropout_prob", 0.0),
                   attention_probs_dropout_prob=cj.optional_f64(v, "attention_probs_dropout_prob", 0.0),
                   hidden_act=cj.optional_hidden_act(v, "hidden_act", "gelu_new"), **label_fields(v))

    def with_architectures(self, arch: str): return replace(self, architectures=[arch])

    def to_json_str(self) -> str:
        m = {"model_type": "albert", "architectures": cj.emit_architectures(self.architectures, "AlbertModel"), "vocab_size": self.vocab_size,
             "embedding_size": self.embedding_size, "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
             "num_hidden_groups": 1, "inner_group_num": 1, "num_attention_heads": self.num_attention_heads,
             "intermediate_size": self.intermediate_size, "max_position_embeddings": self.max_position_embeddings,
             "type_vocab_size": self.type_vocab_size, "layer_norm_eps": self.layer_norm_eps, "hidden_dropout_prob": self.hidden_dropout_prob,
             "attention_probs_dropout_prob": self.attention_probs_dropout_prob, "hidden_act": cj.emit_hidden_act(self.hidden_act)}
        if self.pad_token_id is not None:
            m["pad_token_id"] = self.pad_token_id
        return json.dumps(emit_labels(m, self), indent=2)

    def layer_config(self) -> TransformerLayerConfig:
        return TransformerLayerConfig(self.hidden_size, self.num_attention_heads, self.intermediate_size, self.hidden_dropout_prob,
                                      self.attention_probs_dropout_prob, self.layer_norm_eps, self.hidden_act)

    @staticmethod
    def encoder_inputs(enc) -> List[Variable]:
        return [Variable.wrap(enc.input_ids), Variable.wrap(enc.position_ids), Variable.wrap(enc.token_type_ids),
                Variable.wrap(build_extended_attention_mask(enc.attention_mask))]


class AlbertEmbeddings(Module):
    def __init__(self, config: AlbertConfig, device=None):
        E = config.embedding_size
        self.word_embeddings = Embedding(config.vocab_size, E, config.pad_token_id, device)
        self.position_embeddings = Embedding(config.max_position_embeddings, E, None, device)
        self.token_type_embeddings = Embedding(config.type_vocab_size, E, None, device)
        self.layer_norm = LayerNorm(E, config.layer_norm_eps, device)
        self.p, self.eps = config.hidden_dropout_prob, config.layer_norm_eps
    def name(self): return "albert_embeddings"
    def word_embeddings_weight(self) -> Parameter: return self.word_embeddings.weight
    def own_parameters(self):
        return (prefix_params("word_embeddings", self.word_embeddings.own_parameters())
                + prefix_params("position_embeddings", self.position_embeddings.own_parameters())
                + prefix_params("token_type_embeddings", self.token_type_embeddings.own_parameters())
                + prefix_params("LayerNorm", self.layer_norm.own_parameters()))
    def _finish(self, s):
        if s.is_cuda and _ops.FLAGS.autocast == torch.bfloat16:
            s = s.to(torch.bfloat16)
        y = _ops.layer_norm(s, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        return Variable.wrap(_ops.dropout(y, self.p, self.training))
    def forward(self, x): return self._finish(self.word_embeddings.forward(x).t)
    def forward_named(self, x, refs: Dict[str, Variable]):
        s = self.word_embeddings.forward(x).t
        if "position_ids" in refs:
            s = s + self.position_embeddings.forward(refs["position_ids"]).t
        if "token_type_ids" in refs:
            s = s + self.token_type_embeddings.forward(refs["token_type_ids"]).t
        return self._finish(s)


class AlbertLayerStack(Module):
    """One `TransformerLayer` whose weights are reused `num_repeats` times."""
    def __init__(self, layer_config: TransformerLayerConfig, num_repeats: int, device=None):
        self.layer = TransformerLayer(layer_config, LayerNaming.ALBERT, device)
        self.num_repeats = max(1, int(num_repeats))
    def name(self): return "albert_layer_stack"
    def sub_modules(self): return [self.layer]
    def forward(self, x):
        for _ in range(self.num_repeats):
            x = self.layer.forward(x)
        return x
    def forward_named(self, x, refs):
        for _ in range(self.num_repeats):
            x = self.layer.forward_named(x, refs)
        return x


class AlbertPooler(Module):
    def __init__(self, config, device=None): self.linear = Linear(config.hidden_size, config.hidden_size, True, device)
    def name(self): return "albert_pooler"
    def own_parameters(self): return self.linear.own_parameters()
    def forward(self, x): return self.linear.forward(x.select(1, 0).contiguous()).tanh()


class AlbertMLMHeadTransform(Module):
    def __init__(self, config, device=None):
        self.dense = Linear(config.hidden_size, config.embedding_size, True, device)
        self.layer_norm = LayerNorm(config.embedding_size, config.layer_norm_eps, device)
        self.act = "gelu" if config.hidden_act == GeluApprox.Exact else "gelu_tanh"
        self.eps = config.layer_norm_eps
    def name(self): return "albert_mlm_head_transform"
    def own_parameters(self):
        return prefix_params("dense", self.dense.own_parameters()) + prefix_params("LayerNorm", self.layer_norm.own_parameters())
    def forward(self, x):
        h = _ops.linear(x.t, self.dense.weight.t, self.dense.bias.t, self.act)
        return Variable.wrap(_ops.layer_norm(h, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps))


LAYER_TAG = str(HfPath("albert").sub("encoder").sub("albert_layer_groups").sub(0).sub("albert_layers").sub(0))


def albert_backbone_flow(config: AlbertConfig, device=None, with_pooler: bool = True, embeddings=None) -> FlowBuilder:
    emb = embeddings if embeddings is not None else AlbertEmbeddings(config, device)
    fb = (FlowBuilder.new().input(["position_ids", "token_type_ids", "attention_mask"]).through(emb).tag("albert.embeddings")
          .using(["position_ids", "token_type_ids"])
          .through(Linear(config.embedding_size, config.hidden_size, True, device)).tag("albert.encoder.embedding_hidden_mapping_in")
          .through(AlbertLayerStack(config.layer_config(), config.num_hidden_layers, device)).tag(LAYER_TAG).using(["attention_mask"]))
    if with_pooler:
        fb = fb.through(AlbertPooler(config, device)).tag("albert.pooler")
    return fb


class AlbertModel:
    @staticmethod
    def build(config): return AlbertModel.on_device(config, None)
    @staticmethod
    def on_device(config, device=None) -> Graph: return attach(albert_backbone_flow(config, device, True).build(), config)
    @staticmethod
    def on_device_without_pooler(config, device=None) -> Graph: return attach(albert_backbone_flow(config, device, False).build(), config)


class AlbertForSequenceClassification(ClassificationHead):
    @classmethod
    def on_device(cls, config, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (albert_backbone_flow(config, device, True).through(Dropout(config.hidden_dropout_prob))
             .through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
        return cls(attach(g, config.with_architectures("AlbertForSequenceClassification")), config, n, config.id2label)
    @staticmethod
    def num_labels_from_config(config): return need_num_labels(config, "AlbertForSequenceClassification")


class AlbertForTokenClassification(TaggingHead):
    @classmethod
    def on_device(cls, config, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (albert_backbone_flow(config, device, False).through(Dropout(config.hidden_dropout_prob))
             .through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
        return cls(attach(g, config.with_architectures("AlbertForTokenClassification")), config, n, config.id2label)
    @staticmethod
    def num_labels_from_config(config): return need_num_labels(config, "AlbertForTokenClassification")


class AlbertForQuestionAnswering(QaHead):
    @classmethod
    def on_device(cls, config, device=None):
        g = albert_backbone_flow(config, device, False).through(Linear(config.hidden_size, 2, True, device)).tag("qa_outputs").build()
        return cls(attach(g, config.with_architectures("AlbertForQuestionAnswering")), config)


class AlbertForMaskedLM(MaskedLmHead):
    @classmethod
    def on_device(cls, config, device=None):
        emb = AlbertEmbeddings(config, device)
        g = (albert_backbone_flow(config, device, False, emb).through(AlbertMLMHeadTransform(config, device)).tag("predictions")
             .through(TiedDecoder.from_shared_weight(emb.word_embeddings_weight(), zeros_bias(config.vocab_size, device)))
             .tag("predictions.decoder").build())
        return cls(attach(g, config.with_architectures("AlbertForMaskedLM")), config)
