"""`python -m flodl_b200.hf.verify_export <dir> [--hub-source REPO | --no-hub-source]`: check that a directory written by
this library's exporter is a good Hugging Face checkpoint (flodl-hf/scripts/verify_export.py), and
`python -m flodl_b200.hf.verify_export --matrix`: export and check every (family, head) cell
(flodl-hf/scripts/verify_matrix.py).

Three checks per directory:

1. **Loadability**: `transformers.AutoModel[For*].from_pretrained(dir)` (the class follows the suffix of
   `architectures[0]`) reports no missing and no unexpected keys. This alone catches naming drift (head names, dropped
   pooler keys, ...).
2. **Forward parity with this library**: the same directory loaded here gives the same output as the Transformers model on a
   fixed input (max abs difference below `--tol`).
3. **Forward parity with the upstream** (unless `--no-hub-source`): the source repo, from `--hub-source`, else the
   `flodl_source_repo` the exporter stamped into `config.json`, else `_name_or_path`, loaded through Transformers gives
   bit-identical output to the export. An export without an upstream (a fine-tuned checkpoint) needs `--no-hub-source`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from typing import Dict, List, Optional, Tuple

import torch

from ..tensor import TensorError

_AUTO = (("ForSequenceClassification", "AutoModelForSequenceClassification", "seqcls"), ("ForTokenClassification", "AutoModelForTokenClassification", "tokcls"),
         ("ForQuestionAnswering", "AutoModelForQuestionAnswering", "qa"), ("ForMaskedLM", "AutoModelForMaskedLM", "mlm"))


def auto_class_for(arch: str) -> Tuple[str, str]:
    """(`transformers` auto class name, this library's head kind) for `architectures[0]`, by suffix."""
    for suffix, cls, kind in _AUTO:
        if arch.endswith(suffix):
            return cls, kind
    if arch.endswith("Model") or "For" not in arch:
        return "AutoModel", "base"
    raise TensorError(f"verify_export: unsupported architecture {arch!r}")


def hub_source_of(cfg: dict, flag: Optional[str]) -> Optional[str]:
    return flag or cfg.get("flodl_source_repo") or (cfg.get("_name_or_path") or None)


def _fixed_inputs(vocab: int, seq: int = 12, batch: int = 2):
    g = torch.Generator().manual_seed(1234)
    ids = torch.randint(5, max(6, vocab), (batch, seq), generator=g)
    mask = torch.ones(batch, seq, dtype=torch.long)
    mask[1, seq - 3:] = 0
    return ids, mask


def _hf_outputs(out, kind: str) -> List[torch.Tensor]:
    if kind == "qa":
        return [torch.stack([out.start_logits, out.end_logits], -1)]
    if kind == "base":
        return [out.last_hidden_state]
    return [out.logits]


def _load_with_transformers(transformers, auto_name: str, directory: str):
    """(model in eval mode, missing keys, unexpected keys). `from_pretrained` first; where that trips over the library's
    own bookkeeping (Transformers 5.5 cannot finish loading a non-legacy `DebertaV2ForMaskedLM`: its tied-weight table
    names a parameter the head does not have), the model is built from the config and the file's tensors are loaded
    with `load_state_dict`, keys that are ties of loaded tensors not counted as missing."""
    auto = getattr(transformers, auto_name)
    try:
        model, info = auto.from_pretrained(directory, output_loading_info=True)
        return model.eval(), list(info["missing_keys"]), list(info["unexpected_keys"])
    except AttributeError:
        from .safetensors_io import read_safetensors
        cfg = transformers.AutoConfig.from_pretrained(directory)
        model = auto.from_config(cfg).eval()
        state = {k: torch.as_tensor(v) for k, v in read_safetensors(open(os.path.join(directory, "model.safetensors"), "rb").read()).items()}
        res = model.load_state_dict(state, strict=False)
        if hasattr(model, "tie_weights"):
            model.tie_weights()
        loaded_ptrs = {p.data_ptr() for n, p in model.named_parameters() if n in state}
        params = dict(model.named_parameters())
        missing = [k for k in res.missing_keys if k in params and params[k].data_ptr() not in loaded_ptrs]     # phantom table entries aside
        return model, missing, list(res.unexpected_keys)


def verify(directory: str, hub_source: Optional[str] = None, no_hub_source: bool = False, tol: float = 1e-4) -> Dict[str, object]:
    import transformers
    from . import hub
    from .models.auto import AutoConfig
    cfg_text = open(os.path.join(directory, "config.json")).read()
    cfg = json.loads(cfg_text)
    archs = cfg.get("architectures") or []
    if not archs:
        raise TensorError(f"{directory}/config.json has no `architectures`; cannot pick the class to load it with")
    auto_name, kind = auto_class_for(archs[0])
    report: Dict[str, object] = {"dir": directory, "architecture": archs[0], "auto_class": auto_name}
    model, missing, unexpected = _load_with_transformers(transformers, auto_name, directory)
    report["missing_keys"], report["unexpected_keys"] = sorted(missing), sorted(unexpected)
    report["loadable"] = not missing and not unexpected
    ids, mask = _fixed_inputs(int(cfg.get("vocab_size", 100)), min(12, int(cfg.get("max_position_embeddings", 12)) - 2))
    with torch.no_grad():
        theirs = _hf_outputs(model(input_ids=ids, attention_mask=mask), kind)[0]
    # this library on the same directory
    from .parity import _inputs
    acfg = AutoConfig.from_json_str(cfg_text)
    g = hub.from_pretrained(directory, None, kind)
    if kind == "base" and theirs.dim() == 3:
        g = hub._backbone_from_pretrained(directory, None, None, False)            # sequence output, as AutoModel gives it
    g.set_training(False)
    with torch.no_grad():
        ours = g.forward_multi(_inputs(acfg.model_type(), ids, mask.float())).t
    report["max_abs_diff_vs_transformers"] = float((ours.float() - theirs.float()).abs().max())
    report["forward_parity"] = report["max_abs_diff_vs_transformers"] <= tol
    source = None if no_hub_source else hub_source_of(cfg, hub_source)
    if not no_hub_source and source is None:
        raise TensorError("verify_export: no upstream to compare with (no --hub-source, no `flodl_source_repo` / `_name_or_path` in config.json); "
                          "pass --hub-source <repo>, or --no-hub-source for a loadability-only check")
    if source is not None:
        src_dir = os.path.dirname(hub.resolve_files(source)[0])
        upstream = getattr(transformers, auto_name).from_pretrained(src_dir).eval()
        with torch.no_grad():
            up = _hf_outputs(upstream(input_ids=ids, attention_mask=mask), kind)[0]
        report["hub_source"] = source
        report["max_abs_diff_vs_source"] = float((up.float() - theirs.float()).abs().max())
        report["source_parity"] = report["max_abs_diff_vs_source"] == 0.0
    report["ok"] = bool(report["loadable"] and report["forward_parity"] and report.get("source_parity", True))
    return report


# ---- the whole head matrix ---------------------------------------------------------------------------------------
FAMILIES = ("bert", "roberta", "xlm-roberta", "distilbert", "albert", "deberta-v2")
HEADS = ("base", "seqcls", "tokcls", "qa", "mlm")


def export_tiny(family: str, head: str, out_dir: str) -> None:
    """A small randomly initialised model of this library for one cell, written with its exporter."""
    import transformers
    from .export import build_for_export, export_hf_dir
    from .models.auto import AutoConfig
    from .parity import _tiny
    arch_suffix = {"base": "Model", "seqcls": "ForSequenceClassification", "tokcls": "ForTokenClassification", "qa": "ForQuestionAnswering",
                   "mlm": "ForMaskedLM"}[head]
    hc, prefix, _key_prefix = _tiny(transformers, family)
    hc.architectures = [prefix + arch_suffix]
    if head == "qa":
        hc.num_labels = 2                               # start / end logits
    cfg = AutoConfig.from_json_str(hc.to_json_string())
    torch.manual_seed(0)
    g = build_for_export(cfg, True, None, head)
    export_hf_dir(g, g.source_config() or cfg.to_json_str(), out_dir)


def verify_matrix(families=FAMILIES, heads=HEADS, staging: Optional[str] = None, keep: bool = False, tol: float = 1e-4):
    """{(family, head): report or error text}; fail-soft over the cells."""
    import shutil
    results = {}
    root = staging or tempfile.mkdtemp(prefix="flodl_export_matrix_")
    for fam in families:
        for head in heads:
            d = os.path.join(root, f"{fam}-{head}")
            try:
                export_tiny(fam, head, d)
                results[(fam, head)] = verify(d, no_hub_source=True, tol=tol)
            except Exception as e:  # noqa: BLE001  (one failing cell must not stop the grid)
                results[(fam, head)] = f"{type(e).__name__}: {e}"
            if not keep:
                shutil.rmtree(d, ignore_errors=True)
    if not keep and staging is None:
        shutil.rmtree(root, ignore_errors=True)
    return results


def render_matrix(results, families=FAMILIES, heads=HEADS) -> str:
    lines = ["| family | " + " | ".join(heads) + " |", "|---|" + "---|" * len(heads)]
    for fam in families:
        cells = []
        for h in heads:
            r = results.get((fam, h))
            cells.append("-" if r is None else f"FAIL ({r[:40]})" if isinstance(r, str) else
                         ("PASS" if r["ok"] else "FAIL") + f" {r['max_abs_diff_vs_transformers']:.1e}")
        lines.append(f"| {fam} | " + " | ".join(cells) + " |")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="flodl_b200.hf.verify_export")
    ap.add_argument("dir", nargs="?", help="exported directory (model.safetensors + config.json)")
    ap.add_argument("--hub-source", help="upstream repo to compare the export with")
    ap.add_argument("--no-hub-source", action="store_true", help="loadability and parity with this library only")
    ap.add_argument("--tol", type=float, default=1e-4, help="max abs difference allowed against this library's forward")
    ap.add_argument("--matrix", action="store_true", help="export and verify every (family, head) cell")
    ap.add_argument("--families", help="comma list (with --matrix)")
    ap.add_argument("--heads", help="comma list (with --matrix)")
    ap.add_argument("--keep", action="store_true", help="keep the staged exports (with --matrix)")
    ap.add_argument("--staging-dir", help="where --matrix stages its exports")
    from ..cli.args import answer_schema_probe
    answer_schema_probe(ap, argv)
    a = ap.parse_args(argv)
    try:
        if a.matrix:
            fams = [f for f in (a.families or ",".join(FAMILIES)).split(",") if f]
            heads = [h for h in (a.heads or ",".join(HEADS)).split(",") if h]
            res = verify_matrix(fams, heads, a.staging_dir, a.keep, a.tol)
            print(render_matrix(res, fams, heads))
            return 0 if all(not isinstance(r, str) and r["ok"] for r in res.values()) else 1
        if not a.dir:
            ap.error("give a directory, or --matrix")
        rep = verify(a.dir, a.hub_source, a.no_hub_source, a.tol)
    except (TensorError, OSError) as e:
        print(f"verify_export: {e}", file=sys.stderr)
        return 2
    print(json.dumps(rep, indent=2))
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
