"""XLM-RoBERTa (flodl-hf/src/models/xlm_roberta.rs): RoBERTa's architecture and checkpoint key names (`roberta.*`) with
a config type, presets and architecture strings of its own, so that `model_type: "xlm-roberta"` and
`architectures: ["XLMRoberta..."]` survive a load / export round trip and `AutoModel*` dispatches on them.

What differs from RoBERTa in practice is the data, not the graph: a 250 002-entry SentencePiece vocabulary shared by
100 languages (the embedding matrix is 192 M of the base model's 278 M parameters), `<s>` / `<pad>` / `</s>` / `<unk>` at
ids 0..3 and position ids that start at `pad_token_id + 1 = 2` (hence 514 position rows for 512 tokens).
"""
from __future__ import annotations

from dataclasses import dataclass

from .roberta import RobertaConfig, _family


@dataclass
class XlmRobertaConfig(RobertaConfig):
    """Same fields as RoBERTa; the defaults are those of `xlm-roberta-base`."""
    vocab_size: int = 250002

    MODEL_TYPE = "xlm-roberta"
    FAMILY_NAME = "XlmRoberta"
    BASE_ARCH = "XLMRobertaModel"

    @classmethod
    def xlm_roberta_base(cls) -> "XlmRobertaConfig":
        """12 layers x 768, 12 heads, feed-forward 3072 (278 M parameters)."""
        return cls()

    @classmethod
    def xlm_roberta_large(cls) -> "XlmRobertaConfig":
        """24 layers x 1024, 16 heads, feed-forward 4096 (560 M parameters)."""
        return cls(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096)

    def embedding_parameters(self) -> int:
        """Rows x width of the word-embedding matrix (what dominates the memory of this family)."""
        return self.vocab_size * self.hidden_size


(XlmRobertaModel, XlmRobertaForSequenceClassification, XlmRobertaForTokenClassification, XlmRobertaForQuestionAnswering,
 XlmRobertaForMaskedLM) = _family("XLMRoberta", XlmRobertaConfig)
