"""Task heads over an encoder graph (flodl-hf/src/task_heads.rs): sequence classification, token
classification, extractive QA and masked-LM, with their losses."""
from __future__ import annotations

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


class _Head:
    def __init__(self, graph, config):
        self._graph, self._config = graph, config
        self.tokenizer = None

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
    def __init__(self, graph, config, num_labels: int, id2label=None):
        super().__init__(graph, config)
        self.id2label = list(id2label) if id2label else default_labels(num_labels)

    from_graph = classmethod(lambda cls, graph, config, num_labels, id2label=None: cls(graph, config, num_labels, id2label))

    def labels(self):
        return self.id2label

    def compute_loss(self, inputs, labels) -> Variable:
        return sequence_classification_loss(self.forward(inputs), labels)

    def predict(self, inputs):
        """Per example: [(label, probability)] sorted by probability."""
        with torch.no_grad():
            probs = torch.softmax(self.forward(inputs).t.float(), -1).cpu()
        return [sorted(zip(self.id2label, row.tolist()), key=lambda kv: -kv[1]) for row in probs]

    classify = predict


class TaggingHead(_Head):
    def __init__(self, graph, config, num_labels: int, id2label=None):
        super().__init__(graph, config)
        self.id2label = list(id2label) if id2label else default_labels(num_labels)

    from_graph = classmethod(lambda cls, graph, config, num_labels, id2label=None: cls(graph, config, num_labels, id2label))

    def labels(self):
        return self.id2label

    def compute_loss(self, inputs, labels) -> Variable:
        return token_classification_loss(self.forward(inputs), labels)

    def tag(self, inputs):
        """Per example, per token: (label, probability) of the arg-max class."""
        with torch.no_grad():
            probs = torch.softmax(self.forward(inputs).t.float(), -1).cpu()
        best = probs.max(-1)
        return [[(self.id2label[i], p) for i, p in zip(idx.tolist(), val.tolist())] for idx, val in zip(best.indices, best.values)]

    predict = tag


class QaHead(_Head):
    from_graph = classmethod(lambda cls, graph, config: cls(graph, config))

    def compute_loss(self, inputs, start_positions, end_positions) -> Variable:
        return question_answering_loss(self.forward(inputs), start_positions, end_positions)

    def answer(self, inputs, context_mask: Optional[torch.Tensor] = None):
        """Best (start, end, score) span per example among positions where `context_mask` is set."""
        with torch.no_grad():
            lg = self.forward(inputs).t.float()
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

    def fill_mask(self, inputs, mask_positions, top_k: int = 5):
        """Top-k (token id, probability) for each (batch, position) pair."""
        with torch.no_grad():
            probs = torch.softmax(self.forward(inputs).t.float(), -1)
        out = []
        for b, s in mask_positions:
            top = probs[b, s].topk(top_k)
            out.append(list(zip(top.indices.tolist(), top.values.tolist())))
        return out

    predict = fill_mask
