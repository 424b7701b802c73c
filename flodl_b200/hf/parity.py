"""`python -m flodl_b200.hf.parity [family ...] [--heads base,mlm,seqcls,tokcls,qa] [--device cuda]`

Parity matrix against the `transformers` package (the job of flodl-hf/scripts/parity_*.py and verify_matrix.py):
for every encoder family and task head, build the HuggingFace model from a small random-initialised config, move
its weights through the safetensors writer/reader into this package's graph, run both on the same batch and report
the largest absolute difference of the outputs at the unmasked positions. No download is needed; with `--repo <id>`
the same comparison runs on a real checkpoint resolved by `hub.resolve_files` (local cache or hub).

Exit status 0 when every cell is within tolerance.
"""
from __future__ import annotations

import argparse
import sys
from typing import Callable, Dict, List, Optional, Tuple

import torch

from . import safetensors_io as st
from .models import bert as _bert
from .models.auto import (AutoConfig, AutoModel, AutoModelForMaskedLM, AutoModelForQuestionAnswering, AutoModelForSequenceClassification,
                          AutoModelForTokenClassification)

HEADS = ("base", "mlm", "seqcls", "tokcls", "qa")
_OURS = {"mlm": AutoModelForMaskedLM, "seqcls": AutoModelForSequenceClassification, "tokcls": AutoModelForTokenClassification,
         "qa": AutoModelForQuestionAnswering}
_HF_SUFFIX = {"base": "Model", "mlm": "ForMaskedLM", "seqcls": "ForSequenceClassification", "tokcls": "ForTokenClassification",
              "qa": "ForQuestionAnswering"}


def _tiny(tf, family: str):
    common = dict(vocab_size=60, max_position_embeddings=24, num_labels=3)
    if family == "bert":
        return tf.BertConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, hidden_dropout_prob=0.0,
                             attention_probs_dropout_prob=0.0, **common), "Bert", "bert."
    if family == "roberta":
        return tf.RobertaConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, hidden_dropout_prob=0.0,
                                attention_probs_dropout_prob=0.0, pad_token_id=1, type_vocab_size=1, **common), "Roberta", "roberta."
    if family == "xlm-roberta":
        return tf.XLMRobertaConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, hidden_dropout_prob=0.0,
                                   attention_probs_dropout_prob=0.0, pad_token_id=1, type_vocab_size=1, **common), "XLMRoberta", "roberta."
    if family == "distilbert":
        return tf.DistilBertConfig(dim=32, n_layers=2, n_heads=4, hidden_dim=64, dropout=0.0, attention_dropout=0.0, seq_classif_dropout=0.0,
                                   qa_dropout=0.0, **common), "DistilBert", "distilbert."
    if family == "albert":
        return tf.AlbertConfig(embedding_size=16, hidden_size=32, num_hidden_layers=3, num_attention_heads=4, intermediate_size=64,
                               hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, classifier_dropout_prob=0.0, **common), "Albert", "albert."
    if family == "deberta-v2":
        return tf.DebertaV2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, hidden_dropout_prob=0.0,
                                  attention_probs_dropout_prob=0.0, relative_attention=True, position_buckets=4, max_relative_positions=8,
                                  share_att_key=True, pos_att_type=["p2c", "c2p"], norm_rel_ebd="layer_norm", position_biased_input=False,
                                  type_vocab_size=0, pooler_dropout=0.0, legacy=False, **common), "DebertaV2", "deberta."
    raise ValueError(f"unknown family {family!r}")


FAMILIES = ("bert", "roberta", "xlm-roberta", "distilbert", "albert", "deberta-v2")


def _inputs(model_type: str, ids: torch.Tensor, mask: torch.Tensor) -> List[torch.Tensor]:
    """Graph inputs of each family, in the order its graph declares them."""
    B, S = ids.shape
    ext = _bert.build_extended_attention_mask(mask)
    pos = torch.arange(S, device=ids.device).expand(B, S)
    tt = torch.zeros_like(ids)
    if model_type in ("bert", "albert"):
        return [ids, pos, tt, ext]
    if model_type in ("roberta", "xlm-roberta"):
        return [ids, tt, ext]
    if model_type == "distilbert":
        return [ids, ext]
    if model_type == "deberta-v2":
        return [ids, mask]
    raise ValueError(model_type)


def _state_bytes(model) -> bytes:
    # like `save_pretrained`: a tied tensor is written once, under its source name
    tied = getattr(model, "_tied_weights_keys", None) or ()
    drop = set(tied.keys() if isinstance(tied, dict) else tied)
    sd = {k: v.detach().clone().contiguous() for k, v in model.state_dict().items() if v.is_floating_point() and k not in drop}
    return st.write_safetensors(sd)


def _outputs(out, head: str) -> List[torch.Tensor]:
    if head == "base":
        return [out.last_hidden_state]
    if head == "qa":
        return [out.start_logits, out.end_logits]
    return [out.logits]


def compare(family: str, head: str, device: str = "cpu", seed: int = 0, stress: bool = False, seq_len: int = 12) -> Tuple[float, Optional[str]]:
    """(largest |difference|, note). Raises ImportError when `transformers` is missing.

    `stress` redraws the reference model's matrices with a standard deviation of 0.3 instead of the initialiser's 0.02.
    With the small default weights every attention score is close to zero and whole terms of a layer (DeBERTa's
    position-to-content bias, for one) can be wrong without moving the output beyond the tolerance; with weights of
    ordinary trained size they cannot. `seq_len` beyond the tiny model's relative-position range exercises the
    out-of-range buckets."""
    import transformers as tf
    hc, prefix, key_prefix = _tiny(tf, family)
    if head == "qa":
        hc.num_labels = 2                              # start / end logits
    if seq_len + 2 > hc.max_position_embeddings:
        hc.max_position_embeddings = seq_len + 2
    torch.manual_seed(seed)
    hf = getattr(tf, prefix + _HF_SUFFIX[head])(hc).eval().to(device)
    if stress:
        with torch.no_grad():
            for n, p in hf.named_parameters():
                if p.dim() >= 2 and "embeddings" not in n:
                    p.normal_(0, 0.3)
                elif n.endswith("bias"):
                    p.normal_(0, 0.1)
        if hasattr(hf, "tie_weights"):
            hf.tie_weights()
    cfg = AutoConfig.from_json_str(hc.to_json_string())
    if head == "base":
        graph = AutoModel.from_config(cfg, torch.device(device), with_pooler=False)
        rename: Callable[[str], str] = (lambda k: k if k.startswith(key_prefix) else key_prefix + k)
    else:
        graph = _OURS[head].from_config(cfg, torch.device(device)).graph()
        rename = st.bert_legacy_key_rename
    graph.set_training(False)
    st.load_safetensors_into_graph_with_rename_allow_unused(graph, _state_bytes(hf), rename)
    pad = int(getattr(hc, "pad_token_id", 0) or 0)
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(5, hc.vocab_size, (2, seq_len), generator=g)
    ids[0, seq_len - 4:] = pad
    mask = (ids != pad).float()
    ids, mask = ids.to(device), mask.to(device)
    with torch.no_grad():
        mine = graph.forward(_inputs(cfg.model_type(), ids, mask))
        ref = _outputs(hf(input_ids=ids, attention_mask=mask.long()), head)
    mine_t = mine.t if hasattr(mine, "t") else mine
    if head == "qa":                                   # ours: [B, S, 2]
        parts = [mine_t[..., 0], mine_t[..., 1]]
    else:
        parts = [mine_t]
    worst = 0.0
    for a, b in zip(parts, ref):
        if a.dim() >= 2 and a.shape[:2] == mask.shape:
            a, b = a[mask.bool()], b[mask.bool()]
        worst = max(worst, (a.float() - b.float()).abs().max().item())
    return worst, None


def run(families, heads, device: str, tol: float, stress: bool = False, seq_len: int = 12) -> Dict[Tuple[str, str], Tuple[Optional[float], Optional[str]]]:
    res = {}
    for f in families:
        for h in heads:
            try:
                res[(f, h)] = compare(f, h, device, 0, stress, seq_len)
            except ImportError:
                raise
            except Exception as e:  # noqa: BLE001  (a cell that cannot be built is reported, the matrix goes on)
                res[(f, h)] = (None, f"{type(e).__name__}: {str(e)[:120]}")
    return res


def render(res, families, heads, tol: float) -> str:
    lines = ["| family | " + " | ".join(heads) + " |", "|---|" + "---|" * len(heads)]
    for f in families:
        cells = []
        for h in heads:
            v, note = res[(f, h)]
            cells.append("n/a" if v is None else f"{v:.1e}" + ("" if v <= tol else " FAIL"))
        lines.append(f"| {f} | " + " | ".join(cells) + " |")
    notes = [f"- {f}/{h}: {n}" for (f, h), (v, n) in res.items() if n]
    return "\n".join(lines + ([""] + notes if notes else []))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m flodl_b200.hf.parity")
    ap.add_argument("families", nargs="*", default=list(FAMILIES))
    ap.add_argument("--heads", default=",".join(HEADS))
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tol", type=float, default=2e-4)
    ap.add_argument("--stress", action="store_true", help="weights of trained size (std 0.3) instead of the initialiser's 0.02")
    ap.add_argument("--seq-len", type=int, default=12, help="sequence length of the probe batch")
    a = ap.parse_args(argv)
    heads = [h for h in a.heads.split(",") if h]
    try:
        res = run(a.families, heads, a.device, a.tol, a.stress, a.seq_len)
    except ImportError as e:
        print(f"parity: the `transformers` package is required ({e})", file=sys.stderr)
        return 2
    print(render(res, a.families, heads, a.tol))
    bad = [(k, v) for k, v in res.items() if v[0] is None or v[0] > a.tol]
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
