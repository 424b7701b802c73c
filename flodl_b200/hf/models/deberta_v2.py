"""DeBERTa-v2 / v3 (flodl-hf/src/models/deberta_v2.rs, deberta_transformer_layer.rs).

Disentangled attention: score = (content->content + content->position + position->content) /
sqrt(3 * head_dim), where the position terms come from one shared table of relative-position
embeddings (`rel_embeddings`, LayerNormed once per forward) projected by the SAME query/key
projections (`share_att_key = true`) and indexed by log-bucketed relative distance. No absolute
position embeddings (`position_biased_input = false`), no token types. Graph inputs: `input_ids,
attention_mask` with the mask as a plain `[B, S]` 1/0 tensor.

The score matrix carries an additive, per-(i, j) learned bias, which the flash-attention kernel of
this library does not take; this family runs the attention math as batched GEMMs.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, replace
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ... import ops as _ops
from ...autograd import Variable
from ...graph import FlowBuilder, Graph
from ...nn.activation import GELU, GeluApprox
from ...nn.layers import Dropout, Embedding, LayerNorm, Linear
from ...nn.module import Module, Parameter
from ...tensor import TensorError
from .. import config_json as cj
from ..path import prefix_params
from ..task_heads import ClassificationHead, MaskedLmHead, QaHead, TaggingHead, TiedDecoder, check_num_labels
from ._common import attach, emit_labels, label_fields, need_num_labels, zeros_bias


@dataclass
class DebertaV2Config:
    vocab_size: int = 128100
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    layer_norm_eps: float = 1e-7
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    pad_token_id: Optional[int] = 0
    position_buckets: int = 256
    max_relative_positions: int = 512
    hidden_act: GeluApprox = GeluApprox.Exact
    pooler_hidden_act: GeluApprox = GeluApprox.Exact
    num_labels: Optional[int] = None
    id2label: Optional[List[str]] = None
    architectures: Optional[List[str]] = None

    MODEL_TYPE = "deberta-v2"
    FAMILY_NAME = "DebertaV2"
    MASK_TOKEN = "[MASK]"

    @classmethod
    def deberta_v3_base(cls): return cls()

    @classmethod
    def from_json_str(cls, s: str):
        v = cj.parse(s)
        if not cj.optional_bool(v, "relative_attention", False):
            raise TensorError("DebertaV2Config: relative_attention = false is not supported — every published DeBERTa-v2/v3 checkpoint sets relative_attention=true.")
        if not cj.optional_bool(v, "share_att_key", False):
            raise TensorError("DebertaV2Config: share_att_key = false is not supported (separate pos_query_proj / pos_key_proj weights are unsupported).")
        if cj.optional_bool(v, "position_biased_input", True):
            raise TensorError("DebertaV2Config: position_biased_input = true is not supported (absolute position embeddings are not part of this port).")
        pat = v.get("pos_att_type")
        if pat is not None:
            kinds = sorted(pat.split("|") if isinstance(pat, str) else list(pat))
            if kinds != ["c2p", "p2c"]:
                raise TensorError(f"DebertaV2Config: pos_att_type {pat!r} is not supported — expected c2p|p2c")
        archs = v.get("architectures") or []
        if cj.optional_bool(v, "legacy", False) and archs and str(archs[0]).endswith("ForMaskedLM"):
            # `legacy` only selects the masked-LM head's layout; Transformers writes `legacy: true` into every config it
            # saves, so for the encoder and the other heads the key is ignored
            raise TensorError("DebertaV2Config: legacy = true is not supported: the masked-LM head here is the non-legacy one "
                              "(`lm_predictions.lm_head`: dense(H, H), GELU, LayerNorm, tied decoder), not `cls.predictions`.")
        if str(v.get("norm_rel_ebd", "layer_norm")) != "layer_norm":
            raise TensorError("DebertaV2Config: norm_rel_ebd must be \"layer_norm\"")
        mrp = cj.optional_i64(v, "max_relative_positions", -1)
        mpe = cj.required_i64(v, "max_position_embeddings")
        return cls(vocab_size=cj.required_i64(v, "vocab_size"), hidden_size=cj.required_i64(v, "hidden_size"),
                   num_hidden_layers=cj.required_i64(v, "num_hidden_layers"), num_attention_heads=cj.required_i64(v, "num_attention_heads"),
                   intermediate_size=cj.required_i64(v, "intermediate_size"), max_position_embeddings=mpe,
                   layer_norm_eps=cj.optional_f64(v, "layer_norm_eps", 1e-7), hidden_dropout_prob=cj.optional_f64(v, "hidden_dropout_prob", 0.1),
                   attention_probs_dropout_prob=cj.optional_f64(v, "attention_probs_dropout_prob", 0.1),
                   pad_token_id=cj.optional_i64_or_none(v, "pad_token_id"), position_buckets=cj.optional_i64(v, "position_buckets", 256),
                   max_relative_positions=mpe if mrp < 1 else mrp, hidden_act=cj.optional_hidden_act(v, "hidden_act", "gelu"),
                   pooler_hidden_act=cj.optional_hidden_act(v, "pooler_hidden_act", "gelu"), **label_fields(v))

    def with_architectures(self, arch: str): return replace(self, architectures=[arch])

    def to_json_str(self) -> str:
        m = {"model_type": "deberta-v2", "architectures": cj.emit_architectures(self.architectures, "DebertaV2Model"),
             "vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
             "num_attention_heads": self.num_attention_heads, "intermediate_size": self.intermediate_size,
             "max_position_embeddings": self.max_position_embeddings, "layer_norm_eps": self.layer_norm_eps,
             "hidden_dropout_prob": self.hidden_dropout_prob, "attention_probs_dropout_prob": self.attention_probs_dropout_prob,
             "position_buckets": self.position_buckets, "max_relative_positions": self.max_relative_positions,
             "hidden_act": cj.emit_hidden_act(self.hidden_act), "pooler_hidden_act": cj.emit_hidden_act(self.pooler_hidden_act),
             "pooler_hidden_size": self.hidden_size, "relative_attention": True, "share_att_key": True, "position_biased_input": False,
             "pos_att_type": ["p2c", "c2p"], "norm_rel_ebd": "layer_norm", "type_vocab_size": 0, "legacy": False}
        if self.pad_token_id is not None:
            m["pad_token_id"] = self.pad_token_id
        return json.dumps(emit_labels(m, self), indent=2)

    @staticmethod
    def encoder_inputs(enc) -> List[Variable]:
        return [Variable.wrap(enc.input_ids), Variable.wrap(enc.attention_mask)]


# ---- relative positions ----------------------------------------------------------------------------
def make_log_bucket_position(rel_pos: torch.Tensor, bucket_size: int, max_position: int) -> torch.Tensor:
    """Distances up to bucket_size/2 keep their value; larger ones share logarithmically spaced buckets, `mid .. 2 mid - 1`
    at `max_position - 1`. A distance beyond `max_position - 1` (a sequence longer than the model's relative range) maps
    past the last bucket, as in the Transformers implementation; the index clamp of the attention then folds it onto the
    outermost embedding row of its side. The ratio is snapped to 1 within rounding error so that the distance
    `max_position - 1` itself lands exactly on the last bucket."""
    mid = bucket_size // 2
    rp = rel_pos.float()
    sign = torch.sign(rp)
    near = (rp < mid) & (rp > -mid)
    abs_pos = torch.where(near, torch.full_like(rp, float(mid - 1)), rp.abs())
    ratio = torch.log(abs_pos / mid) / math.log((max_position - 1) / mid)
    ratio = torch.where((ratio - 1.0).abs() < 1e-5, torch.ones_like(ratio), ratio).clamp_min(0.0)
    log_pos = torch.ceil(ratio * (mid - 1)) + mid
    return torch.where(rp.abs() <= mid, rp, log_pos * sign).long()


def build_relative_position(seq_len: int, position_buckets: int, max_relative_positions: int, device=None) -> torch.Tensor:
    """`[1, S, S]` bucketed `i - j`."""
    ids = torch.arange(seq_len, device=device)
    return make_log_bucket_position(ids[:, None] - ids[None, :], position_buckets, max_relative_positions).unsqueeze(0)


def build_deberta_attention_mask(flat_mask: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """`[B, S]` 1/0 -> additive `[B, 1, S, S]`: 0 where query and key are both real tokens, the
    dtype's most negative finite value elsewhere."""
    if flat_mask.dim() != 2:
        raise TensorError(f"flat_mask must be [B, S], got shape {list(flat_mask.shape)}")
    m = flat_mask.to(dtype)
    grid = m[:, None, :, None] * m[:, None, None, :]
    return torch.zeros_like(grid).masked_fill(grid == 0, torch.finfo(dtype).min)


@dataclass
class DebertaV2LayerConfig:
    hidden_size: int
    num_attention_heads: int
    intermediate_size: int
    hidden_dropout_prob: float
    attention_probs_dropout_prob: float
    layer_norm_eps: float
    position_buckets: int
    max_relative_positions: int
    hidden_act: GeluApprox = GeluApprox.Exact


class DisentangledSelfAttention(Module):
    def __init__(self, c: DebertaV2LayerConfig, device=None):
        if c.hidden_size % c.num_attention_heads:
            raise TensorError(f"hidden_size ({c.hidden_size}) must be divisible by num_attention_heads ({c.num_attention_heads})")
        H = c.hidden_size
        self.query_proj, self.key_proj, self.value_proj = Linear(H, H, True, device), Linear(H, H, True, device), Linear(H, H, True, device)
        self.num_heads, self.head_dim = c.num_attention_heads, H // c.num_attention_heads
        self.p_attn, self.p_pos = c.attention_probs_dropout_prob, c.hidden_dropout_prob
        self.position_buckets = c.position_buckets

    def name(self): return "disentangled_self_attention"
    def own_parameters(self):
        return (prefix_params("query_proj", self.query_proj.own_parameters()) + prefix_params("key_proj", self.key_proj.own_parameters())
                + prefix_params("value_proj", self.value_proj.own_parameters()))

    def _heads(self, x: torch.Tensor) -> torch.Tensor:          # [B, S, H] -> [B, Nh, S, D]
        B, S, _ = x.shape
        return x.view(B, S, self.num_heads, self.head_dim).transpose(1, 2)

    def _proj(self, lin: Linear, x: torch.Tensor) -> torch.Tensor:
        return _ops.linear(x, lin.weight.t, lin.bias.t)

    def attend(self, h: torch.Tensor, mask: torch.Tensor, rel_pos: torch.Tensor, rel_emb: torch.Tensor) -> torch.Tensor:
        B, S, _ = h.shape
        q, k, v = (self._heads(self._proj(l, h)) for l in (self.query_proj, self.key_proj, self.value_proj))
        scale = math.sqrt(self.head_dim * 3.0)
        P = self.position_buckets
        rel = _ops.dropout(rel_emb[:2 * P].unsqueeze(0), self.p_pos, self.training)            # [1, 2P, H]
        pos_k = self._heads(self._proj(self.key_proj, rel)).to(q.dtype)                           # [1, Nh, 2P, D]
        pos_q = self._heads(self._proj(self.query_proj, rel)).to(q.dtype)
        c2p_idx = torch.clamp(rel_pos + P, 0, 2 * P - 1).expand(B, self.num_heads, S, S)
        p2c_idx = torch.clamp(-rel_pos + P, 0, 2 * P - 1).expand(B, self.num_heads, S, S)
        c2p = torch.gather(q @ pos_k.transpose(-1, -2), -1, c2p_idx)
        p2c = torch.gather(k @ pos_q.transpose(-1, -2), -1, p2c_idx).transpose(-1, -2)
        scores = (q @ k.transpose(-1, -2) + c2p + p2c) / scale + mask.to(q.dtype)
        probs = torch.softmax(scores.float(), dim=-1).to(q.dtype)
        probs = _ops.dropout(probs, self.p_attn, self.training)
        return (probs @ v).transpose(1, 2).reshape(B, S, self.num_heads * self.head_dim)


class DebertaV2TransformerLayer(Module):
    def __init__(self, c: DebertaV2LayerConfig, device=None):
        H, I = c.hidden_size, c.intermediate_size
        self.c = c
        self.attention_self = DisentangledSelfAttention(c, device)
        self.attn_dense, self.attn_ln = Linear(H, H, True, device), LayerNorm(H, c.layer_norm_eps, device)
        self.inter = Linear(H, I, True, device)
        self.out_dense, self.out_ln = Linear(I, H, True, device), LayerNorm(H, c.layer_norm_eps, device)
        self.act = "gelu" if c.hidden_act == GeluApprox.Exact else "gelu_tanh"

    def name(self): return "deberta_v2_layer"
    def sub_modules(self): return [self.attention_self]
    def own_parameters(self):
        return (prefix_params("attention.output", prefix_params("dense", self.attn_dense.own_parameters())
                              + prefix_params("LayerNorm", self.attn_ln.own_parameters()))
                + prefix_params("intermediate", prefix_params("dense", self.inter.own_parameters()))
                + prefix_params("output", prefix_params("dense", self.out_dense.own_parameters())
                                + prefix_params("LayerNorm", self.out_ln.own_parameters())))

    def parameters(self):
        # attention.self first, as in the reference's key order
        return prefix_params("attention.self", self.attention_self.own_parameters()) + self.own_parameters()

    def run(self, h: torch.Tensor, mask, rel_pos, rel_emb) -> torch.Tensor:
        c = self.c
        a = self.attention_self.attend(h, mask, rel_pos, rel_emb)
        a = _ops.linear(a, self.attn_dense.weight.t, self.attn_dense.bias.t)
        h1 = _ops.layer_norm(a, self.attn_ln.weight.t, self.attn_ln.bias.t, c.layer_norm_eps, residual=h, p_drop=c.hidden_dropout_prob,
                             training=self.training)
        f = _ops.feed_forward(h1, self.inter.weight.t, self.inter.bias.t, self.out_dense.weight.t, self.out_dense.bias.t, self.act)
        return _ops.layer_norm(f, self.out_ln.weight.t, self.out_ln.bias.t, c.layer_norm_eps, residual=h1, p_drop=c.hidden_dropout_prob,
                               training=self.training)


class DebertaV2SelfOutput(Module):
    """Post-attention stage on its own: `LN(dropout(dense(x)) + residual)`, HF's `DebertaV2SelfOutput`
    (deberta_transformer_layer.rs:382-415). `DebertaV2TransformerLayer` runs the same math as one fused
    residual + dropout + LayerNorm op; this class is the stage as a separate module (`forward_pair(x, residual)`)."""

    def __init__(self, c: DebertaV2LayerConfig, device=None, in_features: Optional[int] = None):
        self.dense = Linear(in_features or c.hidden_size, c.hidden_size, True, device)
        self.layer_norm = LayerNorm(c.hidden_size, c.layer_norm_eps, device)
        self.p, self.eps = c.hidden_dropout_prob, c.layer_norm_eps

    @classmethod
    def on_device(cls, config: DebertaV2LayerConfig, device=None): return cls(config, device)
    def name(self): return "deberta_v2_self_output"
    def own_parameters(self):
        return prefix_params("dense", self.dense.own_parameters()) + prefix_params("LayerNorm", self.layer_norm.own_parameters())

    def forward_pair(self, x: Variable, residual: Variable) -> Variable:
        a = _ops.linear(x.t, self.dense.weight.t, self.dense.bias.t)
        return Variable.wrap(_ops.layer_norm(a, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps, residual=residual.t, p_drop=self.p,
                                             training=self.training))

    def forward(self, x: Variable) -> Variable:
        return self.forward_pair(x, x)


class DebertaV2Intermediate(Module):
    """FFN up-projection `act(dense(H -> I))`, HF's `DebertaV2Intermediate` (deberta_transformer_layer.rs:417-440)."""

    def __init__(self, c: DebertaV2LayerConfig, device=None):
        self.dense = Linear(c.hidden_size, c.intermediate_size, True, device)
        self.act = "gelu" if c.hidden_act == GeluApprox.Exact else "gelu_tanh"

    @classmethod
    def on_device(cls, config: DebertaV2LayerConfig, device=None): return cls(config, device)
    def name(self): return "deberta_v2_intermediate"
    def own_parameters(self): return prefix_params("dense", self.dense.own_parameters())
    def forward(self, x: Variable) -> Variable:
        return Variable.wrap(_ops.linear(x.t, self.dense.weight.t, self.dense.bias.t, self.act))


class DebertaV2Output(DebertaV2SelfOutput):
    """FFN down-projection + residual stage `LN(dropout(dense(I -> H)) + residual)`, HF's `DebertaV2Output`
    (deberta_transformer_layer.rs:441-480)."""

    def __init__(self, c: DebertaV2LayerConfig, device=None):
        super().__init__(c, device, in_features=c.intermediate_size)

    def name(self): return "deberta_v2_output"


class DebertaV2Embeddings(Module):
    def __init__(self, config: DebertaV2Config, device=None):
        self.word_embeddings = Embedding(config.vocab_size, config.hidden_size, config.pad_token_id, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.p, self.eps = config.hidden_dropout_prob, config.layer_norm_eps
    def name(self): return "deberta_v2_embeddings"
    def word_embeddings_weight(self) -> Parameter: return self.word_embeddings.weight
    def own_parameters(self):
        return prefix_params("word_embeddings", self.word_embeddings.own_parameters()) + prefix_params("LayerNorm", self.layer_norm.own_parameters())
    def _run(self, x, mask: Optional[Variable]):
        s = self.word_embeddings.forward(x).t
        if s.is_cuda and _ops.FLAGS.autocast == torch.bfloat16:
            s = s.to(torch.bfloat16)
        y = _ops.layer_norm(s, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        if mask is not None:
            y = y * mask.t.to(y.dtype).unsqueeze(-1)             # padded positions are zeroed
        return Variable.wrap(_ops.dropout(y, self.p, self.training))
    def forward(self, x): return self._run(x, None)
    def forward_named(self, x, refs): return self._run(x, refs.get("attention_mask"))


class DebertaV2Encoder(Module):
    def __init__(self, config: DebertaV2Config, device=None):
        lc = DebertaV2LayerConfig(config.hidden_size, config.num_attention_heads, config.intermediate_size, config.hidden_dropout_prob,
                                  config.attention_probs_dropout_prob, config.layer_norm_eps, config.position_buckets,
                                  config.max_relative_positions, config.hidden_act)
        self.layers = [DebertaV2TransformerLayer(lc, device) for _ in range(config.num_hidden_layers)]
        self.rel_embeddings = Embedding(2 * config.position_buckets, config.hidden_size, None, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.position_buckets, self.max_relative_positions, self.eps = config.position_buckets, config.max_relative_positions, config.layer_norm_eps

    def name(self): return "deberta_v2_encoder"

    def parameters(self):
        out = prefix_params("rel_embeddings", self.rel_embeddings.own_parameters()) + prefix_params("LayerNorm", self.layer_norm.own_parameters())
        for i, layer in enumerate(self.layers):
            out += prefix_params(f"layer.{i}", layer.parameters())
        return out

    def set_training(self, training: bool) -> None:
        self.training = training
        for l in self.layers:
            l.training = training
            l.attention_self.training = training

    def _run(self, x: Variable, flat_mask: Optional[torch.Tensor]) -> Variable:
        h = x.t
        B, S, _ = h.shape
        mask = build_deberta_attention_mask(flat_mask, h.dtype) if flat_mask is not None else torch.zeros(B, 1, S, S, dtype=h.dtype, device=h.device)
        rel_pos = build_relative_position(S, self.position_buckets, self.max_relative_positions, h.device)
        w = self.rel_embeddings.weight.t
        rel_emb = F.layer_norm(w, (w.shape[-1],), self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        for layer in self.layers:
            h = layer.run(h, mask, rel_pos, rel_emb)
        return Variable.wrap(h)

    def forward(self, x): return self._run(x, None)

    def forward_named(self, x, refs):
        m = refs.get("attention_mask")
        if m is None:
            raise TensorError('DebertaV2Encoder: missing "attention_mask" ref — the graph must plumb a [B, S] padding mask to the encoder input.')
        return self._run(x, m.t)


class ContextPooler(Module):
    def __init__(self, config, device=None):
        self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
        self.dropout = Dropout(config.hidden_dropout_prob)
        self.act = GELU(config.pooler_hidden_act)
    def name(self): return "context_pooler"
    def sub_modules(self): return [self.dropout]
    def own_parameters(self): return prefix_params("dense", self.dense.own_parameters())
    def forward(self, x): return self.act.forward(self.dense.forward(self.dropout.forward(x.select(1, 0).contiguous())))


class DebertaV2LMHead(Module):
    """dense -> GELU -> LayerNorm -> tied decoder; the module owns the decoder bias as `bias`."""
    def __init__(self, config, tied: Parameter, device=None):
        self.dense = Linear(config.hidden_size, config.hidden_size, True, device)
        self.layer_norm = LayerNorm(config.hidden_size, config.layer_norm_eps, device)
        self.decoder = TiedDecoder.from_shared_weight(tied, zeros_bias(config.vocab_size, device))
        self.act = "gelu" if config.hidden_act == GeluApprox.Exact else "gelu_tanh"
        self.eps = config.layer_norm_eps
    def name(self): return "deberta_v2_lm_head"
    def sub_modules(self): return [self.decoder]
    def own_parameters(self):
        return prefix_params("dense", self.dense.own_parameters()) + prefix_params("LayerNorm", self.layer_norm.own_parameters())
    def forward(self, x):
        h = _ops.linear(x.t, self.dense.weight.t, self.dense.bias.t, self.act)
        h = _ops.layer_norm(h, self.layer_norm.weight.t, self.layer_norm.bias.t, self.eps)
        return self.decoder.forward(Variable.wrap(h))


def deberta_v2_backbone_flow(config: DebertaV2Config, device=None, embeddings=None) -> FlowBuilder:
    emb = embeddings if embeddings is not None else DebertaV2Embeddings(config, device)
    return (FlowBuilder.new().input(["attention_mask"]).through(emb).tag("deberta.embeddings").using(["attention_mask"])
            .through(DebertaV2Encoder(config, device)).tag("deberta.encoder").using(["attention_mask"]))


class DebertaV2Model:
    @staticmethod
    def build(config): return DebertaV2Model.on_device(config, None)
    @staticmethod
    def on_device(config, device=None) -> Graph: return attach(deberta_v2_backbone_flow(config, device).build(), config)


class DebertaV2ForSequenceClassification(ClassificationHead):
    @classmethod
    def on_device(cls, config, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (deberta_v2_backbone_flow(config, device).through(ContextPooler(config, device)).tag("pooler")
             .through(Dropout(config.hidden_dropout_prob)).through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
        return cls(attach(g, config.with_architectures("DebertaV2ForSequenceClassification")), config, n, config.id2label)
    @staticmethod
    def num_labels_from_config(config): return need_num_labels(config, "DebertaV2ForSequenceClassification")


class DebertaV2ForTokenClassification(TaggingHead):
    @classmethod
    def on_device(cls, config, num_labels: int, device=None):
        n = check_num_labels(num_labels)
        g = (deberta_v2_backbone_flow(config, device).through(Dropout(config.hidden_dropout_prob))
             .through(Linear(config.hidden_size, n, True, device)).tag("classifier").build())
        return cls(attach(g, config.with_architectures("DebertaV2ForTokenClassification")), config, n, config.id2label)
    @staticmethod
    def num_labels_from_config(config): return need_num_labels(config, "DebertaV2ForTokenClassification")


class DebertaV2ForQuestionAnswering(QaHead):
    @classmethod
    def on_device(cls, config, device=None):
        g = deberta_v2_backbone_flow(config, device).through(Linear(config.hidden_size, 2, True, device)).tag("qa_outputs").build()
        return cls(attach(g, config.with_architectures("DebertaV2ForQuestionAnswering")), config)


class DebertaV2ForMaskedLM(MaskedLmHead):
    @classmethod
    def on_device(cls, config, device=None):
        emb = DebertaV2Embeddings(config, device)
        g = (deberta_v2_backbone_flow(config, device, emb).through(DebertaV2LMHead(config, emb.word_embeddings_weight(), device))
             .tag("lm_predictions.lm_head").build())
        return cls(attach(g, config.with_architectures("DebertaV2ForMaskedLM")), config)
