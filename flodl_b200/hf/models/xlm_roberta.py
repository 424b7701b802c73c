"""XLM-RoBERTa: RoBERTa's architecture and key names (`roberta.*`), its own config type and
architecture strings (flodl-hf/src/models/xlm_roberta.rs)."""
from .roberta import (XlmRobertaConfig, XlmRobertaForMaskedLM, XlmRobertaForQuestionAnswering,  # noqa: F401
                      XlmRobertaForSequenceClassification, XlmRobertaForTokenClassification, XlmRobertaModel)
