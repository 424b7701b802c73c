"""`AutoConfig` / `AutoModel*`: pick the family from `config.json`'s `model_type`
(flodl-hf/src/models/auto.rs)."""
from __future__ import annotations

import json
from typing import Optional

from ...tensor import TensorError
from . import albert, bert, deberta_v2, distilbert, roberta, xlm_roberta

_FAMILIES = {
    "bert": (bert.BertConfig, "BertModel", bert),
    "roberta": (roberta.RobertaConfig, "RobertaModel", roberta),
    "xlm-roberta": (xlm_roberta.XlmRobertaConfig, "XLMRobertaModel", xlm_roberta),
    "distilbert": (distilbert.DistilBertConfig, "DistilBertModel", distilbert),
    "albert": (albert.AlbertConfig, "AlbertModel", albert),
    "deberta-v2": (deberta_v2.DebertaV2Config, "DebertaV2Model", deberta_v2),
}
_PREFIX = {"bert": "Bert", "roberta": "Roberta", "xlm-roberta": "XlmRoberta", "distilbert": "DistilBert", "albert": "Albert",
           "deberta-v2": "DebertaV2"}


class AutoConfig:
    """A family config plus its `model_type`."""

    def __init__(self, model_type: str, config):
        self._type, self.config = model_type, config

    @classmethod
    def from_json_str(cls, s: str) -> "AutoConfig":
        try:
            v = json.loads(s)
        except Exception as e:
            raise TensorError(f"config.json parse error: {e}")
        mt = v.get("model_type")
        if not isinstance(mt, str):
            raise TensorError("config.json has no `model_type`; cannot pick a model family")
        if mt not in _FAMILIES:
            raise TensorError(f"unsupported model_type {mt!r}; supported: {sorted(_FAMILIES)}")
        return cls(mt, _FAMILIES[mt][0].from_json_str(s))

    def model_type(self) -> str: return self._type
    def to_json_str(self) -> str: return self.config.to_json_str()
    def architectures(self): return self.config.architectures
    def base_class_name(self) -> str: return _FAMILIES[self._type][1]

    def into_normalized_config_json(self, arch_class: str) -> str:
        return self.config.with_architectures(arch_class).to_json_str()

    def _cls(self, suffix: str):
        mod = _FAMILIES[self._type][2]
        return getattr(mod, _PREFIX[self._type] + suffix)


class AutoModel:
    @staticmethod
    def from_config(config: AutoConfig, device=None, with_pooler: bool = True):
        m = config._cls("Model")
        if not with_pooler and hasattr(m, "on_device_without_pooler"):
            return m.on_device_without_pooler(config.config, device)
        return m.on_device(config.config, device)

    @staticmethod
    def from_json_str(s: str, device=None):
        return AutoModel.from_config(AutoConfig.from_json_str(s), device)


class _AutoHead:
    SUFFIX = ""
    NEEDS_LABELS = False

    @classmethod
    def from_config(cls, config: AutoConfig, device=None, num_labels: Optional[int] = None):
        head_cls = config._cls(cls.SUFFIX)
        if cls.NEEDS_LABELS:
            n = num_labels if num_labels is not None else head_cls.num_labels_from_config(config.config) \
                if hasattr(head_cls, "num_labels_from_config") else config.config.num_labels
            if n is None:
                raise TensorError(f"{head_cls.__name__}: config.json has no `num_labels` (nor `id2label`); cannot infer head size")
            return head_cls.on_device(config.config, n, device)
        return head_cls.on_device(config.config, device)

    @classmethod
    def from_json_str(cls, s: str, device=None, num_labels: Optional[int] = None):
        return cls.from_config(AutoConfig.from_json_str(s), device, num_labels)


class AutoModelForSequenceClassification(_AutoHead):
    SUFFIX, NEEDS_LABELS = "ForSequenceClassification", True


class AutoModelForTokenClassification(_AutoHead):
    SUFFIX, NEEDS_LABELS = "ForTokenClassification", True


class AutoModelForQuestionAnswering(_AutoHead):
    SUFFIX = "ForQuestionAnswering"


class AutoModelForMaskedLM(_AutoHead):
    SUFFIX = "ForMaskedLM"
