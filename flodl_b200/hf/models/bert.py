"""BERT (flodl-hf/src/models/bert.rs): config, embeddings, pooler, MLM transform, the backbone
`FlowBuilder` graph with inputs `input_ids, position_ids, token_type_ids, attention_mask`, and the
four task heads. Tags are the HuggingFace module paths so graph keys map to safetensors keys by
replacing the last '/' with '.'."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, replace
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


def build_extended_attention_mask(mask: torch.Tensor, neg: float = -1e4) -> torch.Tensor:
    """`[B, S]` 1/0 mask -> additive fp32 `[B, 1, 1, S]` with `neg` on padded keys (bert.rs:42-48)."""
    if mask.dim() != 2:
        raise TensorError(f"expected [batch, seq_len], got {list(mask.shape)}")
    return ((1.0 - mask.float()) * neg).reshape(mask.shape[0], 1, 1, mask.shape[1])


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    pad_token_id: Optional[int] = 0
    layer_norm_eps: float = 1e-12
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    hidden_act: GeluApprox = GeluApprox.Exact
    num_labels: Optional[int] = None
    id2label: Optional[List[str]] = None
    architectures: Optional[List[str]] = None

    MODEL_TYPE = "bert"
    FAMILY_NAME = "Bert"
    MASK_TOKEN = "[MASK]"

    @classmethod
    def bert_base_uncased(cls) -> "BertConfig":
        return cls()

    @classmethod
    def from_json_str(cls, s: str) -> "BertConfig":
        v = cj.parse(s)
        id2label = cj.parse_id2label(v)
        return cls(
            vocab_size=cj.required_i64(v, "vocab_size"), hidden_size=cj.required_i64(v, "hidden_size"),
            num_hidden_layers=cj.required_i64(v, "num_hidden_layers"), num_attention_heads=cj.required_i64(v, "num_attention_heads"),
            intermediate_size=cj.required_i64(v, "intermediate_size"), max_position_embeddings=cj.required_i64(v, "max_position_embeddings"),
            type_vocab_size=cj.required_i64(v, "type_vocab_size"), pad_token_id=cj.optional_i64_or_none(v, "pad_token_id"),
            layer_norm_eps=cj.optional_f64(v, "layer_norm_eps", 1e-12), hidden_dropout_prob=cj.optional_f64(v, "hidden_dropout_prob", 0.1),
            attention_probs_dropout_prob=cj.optional_f64(v, "attention_probs_dropout_prob", 0.1),
            hidden_act=cj.optional_hidden_act(v, "hidden_act", "gelu"), num_labels=cj.parse_num_labels(v, id2label),
            id2label=id2label, architectures=cj.parse_architectures(v))

    def with_architectures(self, arch: str) -> "BertConfig":
        return replace(self, architectures=[arch])

    def to_json_str(self) -> str:
        m = {"model_type": self.MODEL_TYPE, "architectures": cj.emit_architectures(self.architectures, "BertModel"),
             "vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
             "num_attention_heads": self.num_attention_heads, "intermediate_size": self.intermediate_size,
             "max_position_embeddings": self.max_position_embeddings, "type_vocab_size": self.type_vocab_size,
             "layer_norm_eps": self.layer_norm_eps, "hidden_dropout_prob": self.hidden_dropout_prob,
             "attention_probs_dropout_prob": self.attention_probs_dropout_prob, "hidden_act": cj.emit_hidden_act(self.hidden_act)}
        if self.pad_token_id is not None:
            m["pad_token_id"] = self.pad_token_id
        if self.id2label:
            m["id2label"] = cj.emit_id2label(self.id2label)
            m["label2id"] = {l: i for i, l in enumerate(self.id2label)}
        elif self.num_labels is not None:
            m["num_labels"] = self.num_labels
        return json.dumps(m, indent=2)

    def layer_config(self) -> TransformerLayerConfig:
        return TransformerLayerConfig(self.hidden_size, self.num_attention_heads, self.intermediate_size, self.hidden_dropout_prob,
                                      self.attention_probs_dropout_prob, self.layer_norm_eps, self.hidden_act)

    @staticmethod
    def encoder_inputs(enc) -> List[Variable]:
        mask = build_extended_attention_mask(enc.attention_mask)
        return [Variable.wrap(enc.input_ids), Variable.wrap(enc.position_ids), Variable.wrap(enc.token_type_ids), Variable.wrap(mask)]


class BertEmbeddings(Module):
    """word + position + token-type embeddings -> LayerNorm -> dropout."""

    def __init__(self, config: BertConfig, device=None):
        self.word_embeddings = Embedding(config.vocab_size, config.hidden_size, config.pad_token_id, device)
        self.position_embeddings = Embedding(config.max_position_embeddings, config.hidden_size, None, device)
        self.token_type_embeddings = Embedding(config.type_vocab_size, config.hidden_size, None, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.p = config.hidden_dropout_prob
        self.eps = config.layer_norm_eps

    @classmethod
    def on_device(cls, config, device): return cls(config, device)
    def name(self): return "bert_embeddings"
    def word_embeddings_weight(self) -> Parameter: return self.word_embeddings.weight

    def own_parameters(self):
        return (prefix_params("word_embeddings", self.word_embeddings.own_parameters())
                + prefix_params("position_embeddings", self.position_embeddings.own_parameters())
                + prefix_params("token_type_embeddings", self.token_type_embeddings.own_parameters())
                + prefix_params("LayerNorm", self.layer_norm.own_parameters()))

    def _finish(self, summed: torch.Tensor) -> Variable:
        if summed.is_cuda and _ops.FLAGS.autocast == torch.bfloat16:
            summed = summed.to(torch.bfloat16)
        y = _ops.layer_norm(summed, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        return Variable.wrap(_ops.dropout(y, self.p, self.training))

    def forward(self, x):
        return self._finish(self.word_embeddings.forward(x).t)

    def forward_named(self, x, refs: Dict[str, Variable]):
        s = self.word_embeddings.forward(x).t
        if "position_ids" in refs:
            s = s + self.position_embeddings.forward(refs["position_ids"]).t
        if "token_type_ids" in refs:
            s = s + self.token_type_embeddings.forward(refs["token_type_ids"]).t
        return self._finish(s)


class BertPooler(Module):
    def __init__(self, config, device=None): self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
    @classmethod
    def on_device(cls, config, device): return cls(config, device)
    def name(self): return "bert_pooler"
    def own_parameters(self): return prefix_params("dense", self.dense.own_parameters())
    def forward(self, x): return self.dense.forward(x.select(1, 0).contiguous()).tanh()


class BertPredictionHeadTransform(Module):
    def __init__(self, config, device=None):
        self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.act = "gelu" if config.hidden_act == GeluApprox.Exact else "gelu_tanh"
        self.eps = config.layer_norm_eps
    @classmethod
    def on_device(cls, config, device): return cls(config, device)
    def name(self): return "bert_prediction_head_transform"
    def own_parameters(self):
        return prefix_params("dense", self.dense.own_parameters()) + prefix_params("LayerNorm", self.layer_norm.own_parameters())
    def forward(self, x):
        h = _ops.linear(x.t, self.dense.weight.t, self.dense.bias.t, self.act)
        return Variable.wrap(_ops.layer_norm(h, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps))


def bert_backbone_flow(config: BertConfig, device=None, with_pooler: bool = True, embeddings: Optional[BertEmbeddings] = None,
                       root: str = "bert", naming: LayerNaming = LayerNaming.BERT) -> FlowBuilder:
    emb = embeddings if embeddings is not None else BertEmbeddings(config, device)
    fb = (FlowBuilder.new().input(["position_ids", "token_type_ids", "attention_mask"])
          .through(emb).tag(f"{root}.embeddings").using(["position_ids", "token_type_ids"]))
    layer_root = HfPath(root).sub("encoder").sub("layer")
    lc = config.layer_config()
    for i in range(config.num_hidden_layers):
        fb = fb.through(TransformerLayer(lc, naming, device)).tag(str(layer_root.sub(i))).using(["attention_mask"])
    if with_pooler:
        fb = fb.through(BertPooler(config, device)).tag(f"{root}.pooler")
    return fb


def _attach(graph: Graph, config) -> Graph:
    graph.set_source_config(config.to_json_str())
    return graph


class BertModel:
    @staticmethod
    def build(config: BertConfig) -> Graph: return BertModel.on_device(config, None)
    @staticmethod
    def on_device(config: BertConfig, device=None) -> Graph: return _attach(bert_backbone_flow(config, device, True).build(), config)
    @staticmethod
    def on_device_without_pooler(config, device=None) -> Graph: return _attach(bert_backbone_flow(config, device, False).build(), config)


class BertForSequenceClassification(ClassificationHead):
    @classmethod
    def on_device(cls, config: BertConfig, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (bert_backbone_flow(config, device, True).through(Dropout(config.hidden_dropout_prob))
             .through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
        return cls(_attach(g, config.with_architectures("BertForSequenceClassification")), config, n, config.id2label)

    @staticmethod
    def num_labels_from_config(config):
        from ._common import need_num_labels
        return need_num_labels(config, "BertForSequenceClassification")


class BertForTokenClassification(TaggingHead):
    @classmethod
    def on_device(cls, config: BertConfig, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (bert_backbone_flow(config, device, False).through(Dropout(config.hidden_dropout_prob))
             .through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
        return cls(_attach(g, config.with_architectures("BertForTokenClassification")), config, n, config.id2label)

    @staticmethod
    def num_labels_from_config(config):
        from ._common import need_num_labels
        return need_num_labels(config, "BertForTokenClassification")


class BertForQuestionAnswering(QaHead):
    @classmethod
    def on_device(cls, config: BertConfig, device=None):
        g = bert_backbone_flow(config, device, False).through(Linear(config.hidden_size, 2, True, device)).tag("qa_outputs").build()
        return cls(_attach(g, config.with_architectures("BertForQuestionAnswering")), config)


class BertForMaskedLM(MaskedLmHead):
    @classmethod
    def on_device(cls, config: BertConfig, device=None):
        emb = BertEmbeddings(config, device)
        tied = emb.word_embeddings_weight()
        d = None if device is None else torch.device(str(device)) if not hasattr(device, "torch") else device.torch
        bias = Parameter(torch.zeros(config.vocab_size, device=d), "bias")
        g = (bert_backbone_flow(config, device, False, embeddings=emb)
             .through(BertPredictionHeadTransform(config, device)).tag("cls.predictions.transform")
             .through(TiedDecoder.from_shared_weight(tied, bias)).tag("cls.predictions.decoder").build())
        return cls(_attach(g, config.with_architectures("BertForMaskedLM")), config)
