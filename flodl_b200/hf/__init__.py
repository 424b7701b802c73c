"""HuggingFace interop: encoder families (BERT, RoBERTa, XLM-R, DistilBERT, ALBERT, DeBERTa-v2) as
`FlowBuilder` graphs whose keys map 1:1 to HF checkpoint keys, task heads, safetensors I/O, export,
tokenizer wrapper, local `from_pretrained` (flodl-hf/src/lib.rs)."""
from . import config_json, export, hub, path, safetensors_io, task_heads  # noqa: F401
from .export import build_for_export, export_checkpoint, export_hf_dir  # noqa: F401
from .hub import HubExportHead, from_pretrained  # noqa: F401
from .task_heads import Answer, EncoderInputs, TokenPrediction  # noqa: F401
from .tokenizer import EncodedBatch, HfTokenizer  # noqa: F401
from .models.auto import (AutoConfig, AutoModel, AutoModelForMaskedLM, AutoModelForQuestionAnswering,  # noqa: F401
                          AutoModelForSequenceClassification, AutoModelForTokenClassification)
from .safetensors_io import (load_safetensors_file_into_graph, load_safetensors_into_graph, save_safetensors_file_from_graph,  # noqa: F401
                             save_safetensors_from_graph)
