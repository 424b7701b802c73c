"""Task heads over an encoder graph (flodl-hf/src/task_heads.rs): sequence classification, token
classification, extractive QA and masked-LM, with their losses."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops as _ops
from ..autograd import Variable
from ..autograd.variable import _t
from ..nn.layers import Linear
from ..nn.loss import cross_entropy_loss
from ..tensor import TensorError


def check_num_labels(n: int) -> int:
    if n < 1:
        raise TensorError(f"num_labels must be >= 1, got {n}")
    return n


def default_labels(n: int) -> List[str]:
    return [f"LABEL_{i}" for i in range(n)]


def sequence_classification_loss(logits, labels) -> Variable:
    """`[B, num_labels]` logits, `[B]` class ids (float labels -> regression MSE when num_labels == 1)."""
    lg = _t(logits)
    lb = _t(labels)
    if lg.shape[-1] == 1:
        return Variable.wrap(torch.nn.functional.mse_loss(lg.squeeze(-1).float(), lb.float()))
    return cross_entropy_loss(Variable.wrap(lg.reshape(-1, lg.shape[-1])), Variable.wrap(lb.reshape(-1)))


def token_classification_loss(logits, labels) -> Variable:
    """`[B, S, num_labels]` logits, `[B, S]` labels with -100 on ignored positions."""
    lg = _t(logits)
    return cross_entropy_loss(Variable.wrap(lg.reshape(-1, lg.shape[-1])), Variable.wrap(_t(labels).reshape(-1)))


def masked_lm_loss(logits, labels) -> Variable:
    """`[B, S, V]` logits, `[B, S]` labels, -100 everywhere except the masked positions
    (task_heads.rs:170-183)."""
    lg = _t(logits)
    return cross_entropy_loss(Variable.wrap(lg.reshape(-1, lg.shape[-1])), Variable.wrap(_t(labels).reshape(-1)))


def question_answering_loss(logits, start_positions, end_positions) -> Variable:
    lg = _t(logits)
    if lg.dim() != 3 or lg.shape[2] != 2:
        raise TensorError(f"question_answering_loss: logits must be [batch, seq_len, 2], got {list(lg.shape)}")
    s = cross_entropy_loss(Variable.wrap(lg[..., 0].contiguous()), start_positions)
    e = cross_entropy_loss(Variable.wrap(lg[..., 1].contiguous()), end_positions)
    return s.add(e).mul_scalar(0.5)


class TiedDecoder(Linear):
    """Vocabulary projection that shares the word-embedding matrix. While `labels` are armed
    (`with_labels`) its forward returns the fused projection + cross-entropy scalar instead of the
    `[B, S, V]` logits, so the masked-LM loss never materialises fp32 logits."""

    _labels: Optional[torch.Tensor] = None
    ignore_index: int = -100

    def forward(self, x):
        if self._labels is not None:
            return Variable.wrap(_ops.linear_cross_entropy(x.t, self.weight.t, None if self.bias is None else self.bias.t,
                                                           self._labels.reshape(-1), self.ignore_index, sparse_targets=True))
        return super().forward(x)


@dataclass
class Answer:
    """One extracted span of `QaHead.answer` / `answer_batch` / `extract`: the decoded text, the first and last
    token index (inclusive) and `P(start) + P(end)` of the chosen span (task_heads.rs:18-31)."""
    text: str
    start: int
    end: int
    score: float


@dataclass
class TokenPrediction:
    """One token of a `TaggingHead.tag` / `predict` result: the sub-word, its best label with probability, and
    whether the position is a real token (`attention_mask != 0`) rather than padding (task_heads.rs:33-46)."""
    token: str
    label: str
    score: float
    attends: bool


class EncoderInputs:
    """What a family config provides so that the generic heads can feed its graph: `encoder_inputs(enc)` turns an
    `EncodedBatch` into the graph's `forward_multi` inputs (BERT 4 tensors, RoBERTa 3, DistilBERT 2), plus the
    `FAMILY_NAME` used in messages and the `MASK_TOKEN` spelling (task_heads.rs `EncoderInputs`)."""
    FAMILY_NAME = ""
    MASK_TOKEN = "[MASK]"

    @staticmethod
    def encoder_inputs(enc) -> list:
        raise NotImplementedError


def _is_texts(x) -> bool:
    return isinstance(x, str) or (isinstance(x, (list, tuple)) and len(x) > 0 and all(isinstance(t, str) for t in x))


def _is_encoded(x) -> bool:
    return hasattr(x, "input_ids") and hasattr(x, "attention_mask")


class _Head:
    TASK = ""

    def __init__(self, graph, config):
        self._graph, self._config = graph, config
        self.tokenizer = None

    @classmethod
    def on_device(cls, config, *args):
        """The generic head for whichever family `config` belongs to: `ClassificationHead.on_device(bert_config, 3, device)`
        builds a `BertForSequenceClassification` (the reference specialises the generic head per config type;
        each family's own class overrides this with its graph layout)."""
        from .models import auto as _auto
        for model_type, (cfg_cls, _name, mod) in _auto._FAMILIES.items():
            if type(config) is cfg_cls:
                return getattr(mod, _auto._PREFIX[model_type] + cls.TASK).on_device(config, *args)
        raise TensorError(f"{cls.__name__}.on_device: {type(config).__name__} is not a known family config")

    def _need_tokenizer(self, what: str):
        if self.tokenizer is None:
            fam = getattr(self._config, "FAMILY_NAME", "")
            raise TensorError(f"{fam}{self.TASK}::{what} needs a tokenizer: load with from_pretrained or call with_tokenizer(HfTokenizer.from_file(..))")
        return self.tokenizer

    def _encode(self, texts, what: str):
        tok = self._need_tokenizer(what)
        dev = self._graph.parameters()[0].t.device
        return tok.encode_on_device([texts] if isinstance(texts, str) else list(texts), dev)

    def graph(self):
        return self._graph

    def into_graph(self):
        return self._graph

    def config(self):
        return self._config

    def with_tokenizer(self, tok):
        self.tokenizer = tok
        return self

    def forward(self, inputs: Sequence) -> Variable:
        return self._graph.forward_multi(list(inputs))

    def forward_encoded(self, enc) -> Variable:
        return self._graph.forward_multi(self._config.encoder_inputs(enc))

    def parameters(self):
        return self._graph.parameters()


class ClassificationHead(_Head):
    TASK = "ForSequenceClassification"

    def __init__(self, graph, config, num_labels: int, id2label=None):
        super().__init__(graph, config)
        self.id2label = list(id2label) if id2label else default_labels(num_labels)

    from_graph = classmethod(lambda cls, graph, config, num_labels, id2label=None: cls(graph, config, num_labels, id2label))

    def labels(self):
        return self.id2label

    def compute_loss(self, inputs, labels) -> Variable:
        return sequence_classification_loss(self.forward(inputs), labels)

    def classify(self, inputs):
        """Per example: [(label, probability)] sorted by probability, from an `EncodedBatch` or the graph's
        input tensors. Runs in eval mode."""
        self._graph.set_training(False)
        with torch.no_grad():
            logits = self.forward_encoded(inputs) if _is_encoded(inputs) else self.forward(inputs)
            probs = torch.softmax(logits.t.float(), -1).cpu()
        return [sorted(zip(self.id2label, row.tolist()), key=lambda kv: -kv[1]) for row in probs]

    def predict(self, texts):
        """Text in, label distributions out (needs the tokenizer); tensors / an `EncodedBatch` go to `classify`."""
        return self.classify(self._encode(texts, "predict") if _is_texts(texts) else texts)


class TaggingHead(_Head):
    TASK = "ForTokenClassification"

    def __init__(self, graph, config, num_labels: int, id2label=None):
        super().__init__(graph, config)
        self.id2label = list(id2label) if id2label else default_labels(num_labels)

    from_graph = classmethod(lambda cls, graph, config, num_labels, id2label=None: cls(graph, config, num_labels, id2label))

    def labels(self):
        return self.id2label

    def compute_loss(self, inputs, labels) -> Variable:
        return token_classification_loss(self.forward(inputs), labels)

    def tag(self, inputs):
        """Per example, per token, the arg-max label. From an `EncodedBatch` (tokenizer attached): `TokenPrediction`s
        with the sub-word and the padding flag; from the graph's input tensors: `(label, probability)` pairs."""
        self._graph.set_training(False)
        with torch.no_grad():
            logits = self.forward_encoded(inputs) if _is_encoded(inputs) else self.forward(inputs)
            probs = torch.softmax(logits.t.float(), -1).cpu()
        best = probs.max(-1)
        if not _is_encoded(inputs):
            return [[(self.id2label[i], p) for i, p in zip(idx.tolist(), val.tolist())] for idx, val in zip(best.indices, best.values)]
        tok = self._need_tokenizer("tag")
        ids, attn = inputs.input_ids.cpu().tolist(), inputs.attention_mask.cpu().tolist()
        out = []
        for b, (idx, val) in enumerate(zip(best.indices.tolist(), best.values.tolist())):
            out.append([TokenPrediction(tok.id_to_token(ids[b][s]) or f"<unk_id={ids[b][s]}>", self.id2label[k], p, attn[b][s] != 0)
                        for s, (k, p) in enumerate(zip(idx, val))])
        return out

    def predict(self, texts):
        return self.tag(self._encode(texts, "predict") if _is_texts(texts) else texts)


class QaHead(_Head):
    TASK = "ForQuestionAnswering"
    from_graph = classmethod(lambda cls, graph, config: cls(graph, config))

    def compute_loss(self, inputs, start_positions, end_positions) -> Variable:
        return question_answering_loss(self.forward(inputs), start_positions, end_positions)

    def answer_batch(self, pairs) -> List[Answer]:
        """One `Answer` per `(question, context)` pair (needs the tokenizer)."""
        tok = self._need_tokenizer("answer")
        dev = self._graph.parameters()[0].t.device
        return self.extract(tok.encode_pairs_on_device([tuple(p) for p in pairs], dev))

    def extract(self, enc) -> List[Answer]:
        """Best span over the context tokens (`sequence_ids == 1`) of a pre-tokenised pair batch, decoded."""
        tok = self._need_tokenizer("extract")
        if getattr(enc, "sequence_ids", None) is None:
            raise TensorError("QA extract: the batch has no sequence_ids (encode the pairs with HfTokenizer.encode_pairs)")
        ctx = enc.sequence_ids == 1
        if not bool(ctx.any(dim=1).all()):
            raise TensorError("QA extract: no context tokens (sequence_id == 1) found; tokenizer did not produce a pair encoding")
        self._graph.set_training(False)
        with torch.no_grad():
            logits = self.forward_encoded(enc)
        spans = self._spans(logits, ctx.cpu())
        ids = enc.input_ids.cpu().tolist()
        return [Answer(tok.decode(ids[b][i:j + 1], True), i, j, sc) for b, (i, j, sc) in enumerate(spans)]

    def answer(self, inputs, context=None):
        """`answer(question, context)` with two strings gives an `Answer`; `answer(input_tensors, context_mask)`
        gives the best (start, end, score) span per example among the positions where the mask is set."""
        if isinstance(inputs, str) and isinstance(context, str):
            return self.answer_batch([(inputs, context)])[0]
        with torch.no_grad():
            lg = self.forward(inputs)
        return self._spans(lg, context)

    def _spans(self, logits, context_mask: Optional[torch.Tensor] = None):
        with torch.no_grad():
            lg = logits.t.float()
        return self._best_spans(lg, context_mask)

    @staticmethod
    def _best_spans(lg: torch.Tensor, context_mask: Optional[torch.Tensor] = None):
        """Per row of `[B, S, 2]` logits the (start, end, score) with the largest P(start) + P(end), end >= start,
        both inside the mask."""
        starts, ends = torch.softmax(lg[..., 0], 1).cpu(), torch.softmax(lg[..., 1], 1).cpu()
        out = []
        for b in range(lg.shape[0]):
            valid = [i for i in range(lg.shape[1]) if context_mask is None or bool(context_mask[b, i])]
            best = (valid[0], valid[0], float("-inf"))
            for i in valid:
                for j in valid:
                    if j >= i and starts[b, i] + ends[b, j] > best[2]:
                        best = (i, j, float(starts[b, i] + ends[b, j]))
            out.append(best)
        return out

    predict = answer


class MaskedLmHead(_Head):
    TASK = "ForMaskedLM"
    from_graph = classmethod(lambda cls, graph, config: cls(graph, config))

    def _decoder(self) -> Optional[TiedDecoder]:
        for node in self._graph.nodes:
            if isinstance(node.module, TiedDecoder):
                return node.module
        return None

    def compute_loss(self, inputs, labels) -> Variable:
        """Mean cross-entropy over the positions whose label is not -100. On CUDA the decoder GEMM
        and the softmax cross-entropy run as one fused op."""
        lb = _t(labels)
        dec = self._decoder()
        if dec is not None and _t(inputs[0]).is_cuda and _ops.native_enabled():
            dec._labels = lb
            try:
                return self.forward(inputs)
            finally:
                dec._labels = None
        return masked_lm_loss(self.forward(inputs), lb)

    def fill_mask(self, inputs, mask_positions=5, top_k: int = 5):
        """`fill_mask(text, top_k)`: for every mask token of `text` (the family's spelling, `[MASK]` or `<mask>`) the
        top-k `(token, probability)` candidates (needs the tokenizer). `fill_mask(input_tensors, [(batch, position), ..],
        top_k)`: top-k `(token id, probability)` for each listed position."""
        if isinstance(inputs, str):
            return self._fill_text(inputs, int(mask_positions))
        with torch.no_grad():
            probs = torch.softmax(self.forward(inputs).t.float(), -1)
        out = []
        for b, s in mask_positions:
            top = probs[b, s].topk(top_k)
            out.append(list(zip(top.indices.tolist(), top.values.tolist())))
        return out

    def _fill_text(self, text: str, top_k: int):
        if top_k <= 0:
            raise TensorError("fill_mask: top_k must be > 0")
        tok = self._need_tokenizer("fill_mask")
        mask_tok = getattr(self._config, "MASK_TOKEN", "[MASK]")
        mask_id = tok.token_to_id(mask_tok)
        if mask_id is None:
            raise TensorError(f"fill_mask: tokenizer has no {mask_tok} token")
        self._graph.set_training(False)
        enc = self._encode(text, "fill_mask")
        with torch.no_grad():
            probs = torch.softmax(self.forward_encoded(enc).t.float(), -1)[0].cpu()
        out = []
        for pos, tid in enumerate(enc.input_ids[0].cpu().tolist()):
            if tid == mask_id:
                top = probs[pos].topk(top_k)
                out.append([(tok.id_to_token(i) or f"[UNK_{i}]", p) for i, p in zip(top.indices.tolist(), top.values.tolist())])
        if not out:
            raise TensorError(f"fill_mask: input contains no {mask_tok} token")
        return out

    predict = fill_mask
