"""RoBERTa and XLM-RoBERTa (flodl-hf/src/models/roberta.rs, xlm_roberta.rs).

Same encoder block as BERT; differences: position ids are computed from the input ids
(`padding_idx + cumsum(non_pad) * non_pad`, so real tokens start at `padding_idx + 1`), the graph
takes three inputs (`input_ids, token_type_ids, attention_mask`), the classification head is
dense -> tanh -> out_proj on the first token, and the MLM head lives under `lm_head`."""
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
from .. import config_json as cj
from ..path import HfPath, prefix_params
from ..task_heads import ClassificationHead, MaskedLmHead, QaHead, TaggingHead, TiedDecoder, check_num_labels
from ..transformer_layer import LayerNaming, TransformerLayer, TransformerLayerConfig
from ._common import attach, emit_labels, label_fields, need_num_labels, zeros_bias
from .bert import build_extended_attention_mask


@dataclass
class RobertaConfig:
    vocab_size: int = 50265
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 514      # rows 0..padding_idx are reserved: 512 real positions
    type_vocab_size: int = 1
    pad_token_id: int = 1
    layer_norm_eps: float = 1e-5
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    hidden_act: GeluApprox = GeluApprox.Exact
    num_labels: Optional[int] = None
    id2label: Optional[List[str]] = None
    architectures: Optional[List[str]] = None

    MODEL_TYPE = "roberta"
    FAMILY_NAME = "Roberta"
    MASK_TOKEN = "<mask>"
    BASE_ARCH = "RobertaModel"

    @classmethod
    def roberta_base(cls) -> "RobertaConfig":
        return cls()

    @classmethod
    def from_json_str(cls, s: str):
        v = cj.parse(s)
        return cls(vocab_size=cj.required_i64(v, "vocab_size"), hidden_size=cj.required_i64(v, "hidden_size"),
                   num_hidden_layers=cj.required_i64(v, "num_hidden_layers"), num_attention_heads=cj.required_i64(v, "num_attention_heads"),
                   intermediate_size=cj.required_i64(v, "intermediate_size"), max_position_embeddings=cj.required_i64(v, "max_position_embeddings"),
                   type_vocab_size=cj.optional_i64(v, "type_vocab_size", 1), pad_token_id=cj.optional_i64(v, "pad_token_id", 1),
                   layer_norm_eps=cj.optional_f64(v, "layer_norm_eps", 1e-5), hidden_dropout_prob=cj.optional_f64(v, "hidden_dropout_prob", 0.1),
                   attention_probs_dropout_prob=cj.optional_f64(v, "attention_probs_dropout_prob", 0.1),
                   hidden_act=cj.optional_hidden_act(v, "hidden_act", "gelu"), **label_fields(v))

    def with_architectures(self, arch: str):
        return replace(self, architectures=[arch])

    def to_json_str(self) -> str:
        m = {"model_type": self.MODEL_TYPE, "architectures": cj.emit_architectures(self.architectures, self.BASE_ARCH),
             "vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
             "num_attention_heads": self.num_attention_heads, "intermediate_size": self.intermediate_size,
             "max_position_embeddings": self.max_position_embeddings, "type_vocab_size": self.type_vocab_size,
             "pad_token_id": self.pad_token_id, "layer_norm_eps": self.layer_norm_eps, "hidden_dropout_prob": self.hidden_dropout_prob,
             "attention_probs_dropout_prob": self.attention_probs_dropout_prob, "hidden_act": cj.emit_hidden_act(self.hidden_act)}
        return json.dumps(emit_labels(m, self), indent=2)

    def layer_config(self) -> TransformerLayerConfig:
        return TransformerLayerConfig(self.hidden_size, self.num_attention_heads, self.intermediate_size, self.hidden_dropout_prob,
                                      self.attention_probs_dropout_prob, self.layer_norm_eps, self.hidden_act)

    @staticmethod
    def encoder_inputs(enc) -> List[Variable]:
        return [Variable.wrap(enc.input_ids), Variable.wrap(enc.token_type_ids),
                Variable.wrap(build_extended_attention_mask(enc.attention_mask))]


class RobertaEmbeddings(Module):
    def __init__(self, config: RobertaConfig, device=None):
        self.word_embeddings = Embedding(config.vocab_size, config.hidden_size, config.pad_token_id, device)
        self.position_embeddings = Embedding(config.max_position_embeddings, config.hidden_size, config.pad_token_id, device)
        self.token_type_embeddings = Embedding(config.type_vocab_size, config.hidden_size, None, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.p, self.eps, self.padding_idx = config.hidden_dropout_prob, config.layer_norm_eps, config.pad_token_id

    @classmethod
    def on_device(cls, config, device): return cls(config, device)
    def name(self): return "roberta_embeddings"
    def word_embeddings_weight(self) -> Parameter: return self.word_embeddings.weight

    def own_parameters(self):
        return (prefix_params("word_embeddings", self.word_embeddings.own_parameters())
                + prefix_params("position_embeddings", self.position_embeddings.own_parameters())
                + prefix_params("token_type_embeddings", self.token_type_embeddings.own_parameters())
                + prefix_params("LayerNorm", self.layer_norm.own_parameters()))

    def position_ids_from_input_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        mask = (input_ids != self.padding_idx).long()
        return torch.cumsum(mask, dim=1) * mask + self.padding_idx

    def _run(self, x: Variable, token_type: Optional[Variable]) -> Variable:
        ids = x.t
        s = self.word_embeddings.forward(x).t + self.position_embeddings.forward(Variable.wrap(self.position_ids_from_input_ids(ids))).t
        tt = token_type if token_type is not None else Variable.wrap(torch.zeros_like(ids))
        s = s + self.token_type_embeddings.forward(tt).t
        if s.is_cuda and _ops.FLAGS.autocast == torch.bfloat16:
            s = s.to(torch.bfloat16)
        y = _ops.layer_norm(s, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        return Variable.wrap(_ops.dropout(y, self.p, self.training))

    def forward(self, x): return self._run(x, None)
    def forward_named(self, x, refs: Dict[str, Variable]): return self._run(x, refs.get("token_type_ids"))


class RobertaPooler(Module):
    def __init__(self, config, device=None): self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
    def name(self): return "roberta_pooler"
    def own_parameters(self): return prefix_params("dense", self.dense.own_parameters())
    def forward(self, x): return self.dense.forward(x.select(1, 0).contiguous()).tanh()


class RobertaClassificationHead(Module):
    def __init__(self, config, num_labels: int, device=None):
        self.dropout = Dropout(config.hidden_dropout_prob)
        self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
        self.out_proj = Linear(config.hidden_size, num_labels, True, device)
    def name(self): return "roberta_classification_head"
    def sub_modules(self): return [self.dropout]
    def own_parameters(self):
        return prefix_params("dense", self.dense.own_parameters()) + prefix_params("out_proj", self.out_proj.own_parameters())
    def forward(self, x):
        h = self.dropout.forward(x.select(1, 0).contiguous())
        h = self.dropout.forward(self.dense.forward(h).tanh())
        return self.out_proj.forward(h)


class RobertaLMHeadTransform(Module):
    def __init__(self, config, device=None):
        self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.act = "gelu" if config.hidden_act == GeluApprox.Exact else "gelu_tanh"
        self.eps = config.layer_norm_eps
    def name(self): return "roberta_lm_head_transform"
    def own_parameters(self):
        return prefix_params("dense", self.dense.own_parameters()) + prefix_params("layer_norm", self.layer_norm.own_parameters())
    def forward(self, x):
        h = _ops.linear(x.t, self.dense.weight.t, self.dense.bias.t, self.act)
        return Variable.wrap(_ops.layer_norm(h, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps))


def roberta_backbone_flow(config: RobertaConfig, device=None, with_pooler: bool = True,
                          embeddings: Optional[RobertaEmbeddings] = None) -> FlowBuilder:
    emb = embeddings if embeddings is not None else RobertaEmbeddings(config, device)
    fb = FlowBuilder.new().input(["token_type_ids", "attention_mask"]).through(emb).tag("roberta.embeddings").using(["token_type_ids"])
    root = HfPath("roberta").sub("encoder").sub("layer")
    lc = config.layer_config()
    for i in range(config.num_hidden_layers):
        fb = fb.through(TransformerLayer(lc, LayerNaming.BERT, device)).tag(str(root.sub(i))).using(["attention_mask"])
    if with_pooler:
        fb = fb.through(RobertaPooler(config, device)).tag("roberta.pooler")
    return fb


def roberta_masked_lm_graph(config: RobertaConfig, device=None) -> Graph:
    emb = RobertaEmbeddings(config, device)
    return (roberta_backbone_flow(config, device, False, emb).through(RobertaLMHeadTransform(config, device)).tag("lm_head")
            .through(TiedDecoder.from_shared_weight(emb.word_embeddings_weight(), zeros_bias(config.vocab_size, device)))
            .tag("lm_head.decoder").build())


def _family(prefix: str, config_cls):
    """The five public classes of one RoBERTa-shaped family."""
    class Model:
        @staticmethod
        def build(config): return Model.on_device(config, None)
        @staticmethod
        def on_device(config, device=None): return attach(roberta_backbone_flow(config, device, True).build(), config)
        @staticmethod
        def on_device_without_pooler(config, device=None): return attach(roberta_backbone_flow(config, device, False).build(), config)

    class ForSequenceClassification(ClassificationHead):
        @classmethod
        def on_device(cls, config, num_labels: int, device=None):
            n = check_num_labels(num_labels)
            g = roberta_backbone_flow(config, device, False).through(RobertaClassificationHead(config, n, device)).tag("classifier").build()
            return cls(attach(g, config.with_architectures(f"{prefix}ForSequenceClassification")), config, n, config.id2label)
        @staticmethod
        def num_labels_from_config(config): return need_num_labels(config, f"{prefix}ForSequenceClassification")

    class ForTokenClassification(TaggingHead):
        @classmethod
        def on_device(cls, config, num_labels: int, device=None):
            n = check_num_labels(num_labels)
            g = (roberta_backbone_flow(config, device, False).through(Dropout(config.hidden_dropout_prob))
                 .through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
            return cls(attach(g, config.with_architectures(f"{prefix}ForTokenClassification")), config, n, config.id2label)
        @staticmethod
        def num_labels_from_config(config): return need_num_labels(config, f"{prefix}ForTokenClassification")

    class ForQuestionAnswering(QaHead):
        @classmethod
        def on_device(cls, config, device=None):
            g = roberta_backbone_flow(config, device, False).through(Linear(config.hidden_size, 2, True, device)).tag("qa_outputs").build()
            return cls(attach(g, config.with_architectures(f"{prefix}ForQuestionAnswering")), config)

    class ForMaskedLM(MaskedLmHead):
        @classmethod
        def on_device(cls, config, device=None):
            return cls(attach(roberta_masked_lm_graph(config, device), config.with_architectures(f"{prefix}ForMaskedLM")), config)

    for c, n in ((Model, "Model"), (ForSequenceClassification, "ForSequenceClassification"), (ForTokenClassification, "ForTokenClassification"),
                 (ForQuestionAnswering, "ForQuestionAnswering"), (ForMaskedLM, "ForMaskedLM")):
        c.__name__ = c.__qualname__ = prefix + n
    return Model, ForSequenceClassification, ForTokenClassification, ForQuestionAnswering, ForMaskedLM


(RobertaModel, RobertaForSequenceClassification, RobertaForTokenClassification, RobertaForQuestionAnswering,
 RobertaForMaskedLM) = _family("Roberta", RobertaConfig)
