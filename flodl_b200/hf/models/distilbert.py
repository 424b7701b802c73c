"""DistilBERT (flodl-hf/src/models/distilbert.rs): word + learned position embeddings (no token
types), 6 post-LN blocks with DistilBERT's key names, no pooler; graph inputs `input_ids,
attention_mask`."""
from __future__ import annotations

import json
from dataclasses import dataclass, replace
from typing import List, Optional

import torch

from ... import ops as _ops
from ...autograd import Variable
from ...graph import FlowBuilder, Graph
from ...nn.activation import GELU, GeluApprox
from ...nn.layers import Dropout, Embedding, LayerNorm, Linear
from ...nn.module import Module, Parameter
from .. import config_json as cj
from ..path import HfPath, prefix_params
from ..task_heads import ClassificationHead, MaskedLmHead, QaHead, TaggingHead, TiedDecoder, check_num_labels
from ..transformer_layer import LayerNaming, TransformerLayer, TransformerLayerConfig
from ._common import ActivationDropoutLinear, SelectClsLinear, attach, emit_labels, label_fields, need_num_labels, zeros_bias
from .bert import build_extended_attention_mask


@dataclass
class DistilBertConfig:
    vocab_size: int = 30522
    dim: int = 768
    n_layers: int = 6
    n_heads: int = 12
    hidden_dim: int = 3072
    max_position_embeddings: int = 512
    pad_token_id: int = 0
    dropout: float = 0.1
    attention_dropout: float = 0.1
    qa_dropout: float = 0.1
    seq_classif_dropout: float = 0.2
    sinusoidal_pos_embds: bool = False
    layer_norm_eps: float = 1e-12
    hidden_act: GeluApprox = GeluApprox.Exact
    num_labels: Optional[int] = None
    id2label: Optional[List[str]] = None
    architectures: Optional[List[str]] = None

    MODEL_TYPE = "distilbert"
    FAMILY_NAME = "DistilBert"
    MASK_TOKEN = "[MASK]"

    @classmethod
    def distilbert_base_uncased(cls): return cls()

    @classmethod
    def from_json_str(cls, s: str):
        v = cj.parse(s)
        return cls(vocab_size=cj.required_i64(v, "vocab_size"), dim=cj.required_i64(v, "dim"), n_layers=cj.required_i64(v, "n_layers"),
                   n_heads=cj.required_i64(v, "n_heads"), hidden_dim=cj.required_i64(v, "hidden_dim"),
                   max_position_embeddings=cj.required_i64(v, "max_position_embeddings"), pad_token_id=cj.optional_i64(v, "pad_token_id", 0),
                   dropout=cj.optional_f64(v, "dropout", 0.1), attention_dropout=cj.optional_f64(v, "attention_dropout", 0.1),
                   qa_dropout=cj.optional_f64(v, "qa_dropout", 0.1), seq_classif_dropout=cj.optional_f64(v, "seq_classif_dropout", 0.2),
                   sinusoidal_pos_embds=cj.optional_bool(v, "sinusoidal_pos_embds", False), layer_norm_eps=cj.optional_f64(v, "layer_norm_eps", 1e-12),
                   hidden_act=cj.optional_hidden_act(v, "activation", "gelu"), **label_fields(v))

    def with_architectures(self, arch: str): return replace(self, architectures=[arch])

    def to_json_str(self) -> str:
        m = {"model_type": "distilbert", "architectures": cj.emit_architectures(self.architectures, "DistilBertModel"),
             "vocab_size": self.vocab_size, "dim": self.dim, "n_layers": self.n_layers, "n_heads": self.n_heads, "hidden_dim": self.hidden_dim,
             "max_position_embeddings": self.max_position_embeddings, "pad_token_id": self.pad_token_id, "dropout": self.dropout,
             "attention_dropout": self.attention_dropout, "qa_dropout": self.qa_dropout, "seq_classif_dropout": self.seq_classif_dropout,
             "sinusoidal_pos_embds": self.sinusoidal_pos_embds, "layer_norm_eps": self.layer_norm_eps,
             "activation": cj.emit_hidden_act(self.hidden_act)}
        return json.dumps(emit_labels(m, self), indent=2)

    def layer_config(self) -> TransformerLayerConfig:
        return TransformerLayerConfig(self.dim, self.n_heads, self.hidden_dim, self.dropout, self.attention_dropout, self.layer_norm_eps, self.hidden_act)

    @staticmethod
    def encoder_inputs(enc) -> List[Variable]:
        return [Variable.wrap(enc.input_ids), Variable.wrap(build_extended_attention_mask(enc.attention_mask))]


class DistilBertEmbeddings(Module):
    def __init__(self, config: DistilBertConfig, device=None):
        self.word_embeddings = Embedding(config.vocab_size, config.dim, config.pad_token_id, device)
        self.position_embeddings = Embedding(config.max_position_embeddings, config.dim, None, device)
        self.layer_norm = LayerNorm(config.dim, config.layer_norm_eps, device)
        self.p, self.eps = config.dropout, config.layer_norm_eps
    def name(self): return "distilbert_embeddings"
    def word_embeddings_weight(self) -> Parameter: return self.word_embeddings.weight
    def own_parameters(self):
        return (prefix_params("word_embeddings", self.word_embeddings.own_parameters())
                + prefix_params("position_embeddings", self.position_embeddings.own_parameters())
                + prefix_params("LayerNorm", self.layer_norm.own_parameters()))
    def forward(self, x):
        ids = x.t
        pos = torch.arange(ids.shape[1], device=ids.device).unsqueeze(0).expand_as(ids)
        s = self.word_embeddings.forward(x).t + self.position_embeddings.forward(Variable.wrap(pos)).t
        if s.is_cuda and _ops.FLAGS.autocast == torch.bfloat16:
            s = s.to(torch.bfloat16)
        y = _ops.layer_norm(s, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        return Variable.wrap(_ops.dropout(y, self.p, self.training))


def distilbert_backbone_flow(config: DistilBertConfig, device=None, embeddings=None) -> FlowBuilder:
    emb = embeddings if embeddings is not None else DistilBertEmbeddings(config, device)
    fb = FlowBuilder.new().input(["attention_mask"]).through(emb).tag("distilbert.embeddings")
    root = HfPath("distilbert").sub("transformer").sub("layer")
    lc = config.layer_config()
    for i in range(config.n_layers):
        fb = fb.through(TransformerLayer(lc, LayerNaming.DISTILBERT, device)).tag(str(root.sub(i))).using(["attention_mask"])
    return fb


class DistilBertModel:
    @staticmethod
    def build(config): return DistilBertModel.on_device(config, None)
    @staticmethod
    def on_device(config, device=None) -> Graph: return attach(distilbert_backbone_flow(config, device).build(), config)


class DistilBertForSequenceClassification(ClassificationHead):
    @classmethod
    def on_device(cls, config, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (distilbert_backbone_flow(config, device).through(SelectClsLinear(Linear(config.dim, config.dim, True, device))).tag("pre_classifier")
             .through(ActivationDropoutLinear(config.seq_classif_dropout, Linear(config.dim, n, True, device))).tag("classifier").build())
        return cls(attach(g, config.with_architectures("DistilBertForSequenceClassification")), config, n, config.id2label)
    @staticmethod
    def num_labels_from_config(config): return need_num_labels(config, "DistilBertForSequenceClassification")


class DistilBertForTokenClassification(TaggingHead):
    @classmethod
    def on_device(cls, config, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (distilbert_backbone_flow(config, device).through(Dropout(config.dropout)).through(Linear(config.dim, n, True, device))
             .tag("classifier").build())
        return cls(attach(g, config.with_architectures("DistilBertForTokenClassification")), config, n, config.id2label)
    @staticmethod
    def num_labels_from_config(config): return need_num_labels(config, "DistilBertForTokenClassification")


class DistilBertForQuestionAnswering(QaHead):
    @classmethod
    def on_device(cls, config, device=None):
        g = (distilbert_backbone_flow(config, device).through(Dropout(config.qa_dropout)).through(Linear(config.dim, 2, True, device))
             .tag("qa_outputs").build())
        return cls(attach(g, config.with_architectures("DistilBertForQuestionAnswering")), config)


class DistilBertForMaskedLM(MaskedLmHead):
    @classmethod
    def on_device(cls, config, device=None):
        emb = DistilBertEmbeddings(config, device)
        g = (distilbert_backbone_flow(config, device, emb).through(Linear(config.dim, config.dim, True, device)).tag("vocab_transform")
             .through(GELU(config.hidden_act)).through(LayerNorm(config.dim, config.layer_norm_eps, device)).tag("vocab_layer_norm")
             .through(TiedDecoder.from_shared_weight(emb.word_embeddings_weight(), zeros_bias(config.vocab_size, device)))
             .tag("vocab_projector").build())
        return cls(attach(g, config.with_architectures("DistilBertForMaskedLM")), config)
