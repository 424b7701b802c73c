"""Export a graph as a HuggingFace model directory (`model.safetensors` + `config.json`) and
rebuild the right graph for a checkpoint from its config (flodl-hf/src/export.rs)."""
from __future__ import annotations

import os
from typing import Optional

from ..tensor import TensorError
from .models.auto import AutoConfig, AutoModel, AutoModelForMaskedLM, AutoModelForQuestionAnswering, \
    AutoModelForSequenceClassification, AutoModelForTokenClassification
from .safetensors_io import save_safetensors_file_from_graph

HEAD_KINDS = ("base", "seqcls", "tokcls", "qa", "mlm")


def export_hf_dir(graph, config_json: str, out_dir: str) -> None:
    os.makedirs(out_dir, exist_ok=True)
    save_safetensors_file_from_graph(graph, os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        f.write(config_json)


def classify_architecture(arch: str) -> str:
    for suffix, kind in (("ForSequenceClassification", "seqcls"), ("ForTokenClassification", "tokcls"), ("ForQuestionAnswering", "qa"),
                         ("ForMaskedLM", "mlm")):
        if arch.endswith(suffix):
            return kind
    if arch.endswith("Model") or "For" not in arch:
        return "base"
    raise TensorError(f"build_for_export: unsupported architecture {arch!r}. Dispatched heads: Model, ForSequenceClassification, "
                      "ForTokenClassification, ForQuestionAnswering, ForMaskedLM.")


def parse_head(s: str) -> str:
    """`--head` values of the export tool."""
    k = s.strip().lower().replace("-", "").replace("_", "")
    alias = {"base": "base", "model": "base", "seqcls": "seqcls", "sequenceclassification": "seqcls", "tokcls": "tokcls",
             "tokenclassification": "tokcls", "qa": "qa", "questionanswering": "qa", "mlm": "mlm", "maskedlm": "mlm"}
    if k not in alias:
        raise TensorError(f"unknown head {s!r}; expected one of base, seqcls, tokcls, qa, mlm")
    return alias[k]


def build_for_export(config: AutoConfig, has_pooler: bool = True, device=None, head: Optional[str] = None):
    """The graph whose keys match the checkpoint described by `config` (its `architectures[0]`
    unless `head` overrides it)."""
    if head is None:
        arch = (config.architectures() or [None])[0]
        head = classify_architecture(arch) if arch else "base"
    if head == "base":
        return AutoModel.from_config(config, device, with_pooler=has_pooler)
    cls = {"seqcls": AutoModelForSequenceClassification, "tokcls": AutoModelForTokenClassification, "qa": AutoModelForQuestionAnswering,
           "mlm": AutoModelForMaskedLM}[head]
    return cls.from_config(config, device).graph()


def export_checkpoint(fdl_path: str, out_dir: str, device=None) -> None:
    """`.fdl` checkpoint + its `<stem>.config.json` sidecar -> HuggingFace directory."""
    from ..graph import sidecar_config_path
    from .safetensors_io import keys_have_pooler
    from ..nn.checkpoint import checkpoint_keys
    side = sidecar_config_path(fdl_path)
    if not os.path.exists(side):
        raise TensorError(f"export: no config sidecar next to {fdl_path} (expected {side})")
    cfg_json = open(side).read()
    cfg = AutoConfig.from_json_str(cfg_json)
    g = build_for_export(cfg, keys_have_pooler(checkpoint_keys(fdl_path)), device)
    g.load_checkpoint(fdl_path)
    export_hf_dir(g, cfg_json, out_dir)
