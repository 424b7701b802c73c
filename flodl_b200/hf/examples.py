"""Runnable demos of the Hugging Face integration: `python -m flodl_b200.hf.examples [name] [--repo REPO] [text ...]`
(flodl-hf/examples/*.rs: auto_classify, {bert,roberta,distilbert}_{embed,classify,ner,qa}, distilbert_finetune).

Without a name the list is printed. Every demo takes `--repo` (a hub id, or a local directory with `config.json`,
`model.safetensors` and `tokenizer.json`); the defaults are the public checkpoints the reference's demos use. Weights come
from the local caches first and are downloaded otherwise (`HF_HUB_OFFLINE=1` forbids that).
"""
from __future__ import annotations

import argparse
import sys
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..tensor import TensorError

EXAMPLES: Dict[str, Tuple[str, str, Callable]] = {}


def example(name: str, default_repo: str, doc: str):
    def deco(fn):
        EXAMPLES[name] = (default_repo, doc, fn)
        return fn
    return deco


# ---- the four task shapes, family-agnostic -------------------------------------------------------------------------
def embed(repo: str, texts: List[str], out=print) -> torch.Tensor:
    """Mean-pooled sentence embeddings from the bare encoder and their cosine similarities."""
    from . import AutoConfig, AutoModel, HfTokenizer
    from .models import auto as _auto
    cfg = AutoConfig.from_pretrained(repo)
    graph = AutoModel.from_pretrained(repo)
    graph.set_training(False)
    enc = HfTokenizer.from_pretrained(repo).encode(texts)
    with torch.no_grad():
        hidden = graph.forward_multi(type(cfg.config).encoder_inputs(enc)).t          # [B, S, H]
    mask = enc.attention_mask.unsqueeze(-1)
    emb = torch.nn.functional.normalize((hidden * mask).sum(1) / mask.sum(1).clamp_min(1.0), dim=-1)
    sim = emb @ emb.T
    out(f"{_auto._PREFIX[cfg.model_type()]} encoder, hidden size {hidden.shape[-1]}")
    for i, t in enumerate(texts):
        out(f"  [{i}] {t}")
    for i in range(len(texts)):
        out("  " + " ".join(f"{sim[i, j]:6.3f}" for j in range(len(texts))))
    return emb


def classify(repo: str, texts: List[str], out=print):
    from . import AutoModelForSequenceClassification
    head = AutoModelForSequenceClassification.from_pretrained(repo)
    res = head.predict(texts)
    for text, dist in zip(texts, res):
        out(f"  {dist[0][0]:<12} {dist[0][1]:.3f}  {text}")
    return res


def ner(repo: str, texts: List[str], out=print):
    from . import AutoModelForTokenClassification
    head = AutoModelForTokenClassification.from_pretrained(repo)
    res = head.predict(texts)
    for text, row in zip(texts, res):
        out(f"  {text}")
        for p in row:
            if p.attends and p.label not in ("O", "LABEL_0") and not (p.token.startswith("[") or p.token.startswith("<")):
                out(f"    {p.token:<16} {p.label:<10} {p.score:.3f}")
    return res


def qa(repo: str, pairs: List[Tuple[str, str]], out=print):
    from . import AutoModelForQuestionAnswering
    head = AutoModelForQuestionAnswering.from_pretrained(repo)
    res = head.answer_batch(pairs)
    for (q, _ctx), a in zip(pairs, res):
        out(f"  Q: {q}\n  A: {a.text!r}  (tokens {a.start}..{a.end}, score {a.score:.3f})")
    return res


def finetune(repo: str, texts: List[str], labels: List[int], steps: int = 20, lr: float = 5e-4, out=print, export_dir: Optional[str] = None):
    """Fine-tune a sequence classifier on a handful of labelled sentences: the loss curve, the predictions after training
    and (with `export_dir`) the export recipe back to a Hugging Face directory."""
    from .. import nn
    from ..autograd import Variable
    from . import AutoModelForSequenceClassification, export_hf_dir
    head = AutoModelForSequenceClassification.from_pretrained(repo)
    enc = head.tokenizer.encode(texts)
    inputs = type(head.config()).encoder_inputs(enc)
    target = Variable.wrap(torch.tensor(labels))
    graph = head.graph()
    opt = nn.AdamW(graph.parameters(), lr, 0.01)
    graph.set_training(True)
    curve = []
    for step in range(steps):
        opt.zero_grad()
        loss = head.compute_loss(inputs, target)
        loss.backward()
        nn.clip_grad_norm(graph.parameters(), 1.0)
        opt.step()
        curve.append(float(loss.item()))
        if step % max(1, steps // 5) == 0 or step == steps - 1:
            out(f"  step {step:>3}  loss {curve[-1]:.4f}")
    preds = [dist[0][0] for dist in head.predict(texts)]
    out("  predictions: " + ", ".join(preds))
    if export_dir:
        export_hf_dir(graph, graph.source_config(), export_dir)
        out(f"  exported to {export_dir} (load with transformers.AutoModelForSequenceClassification.from_pretrained)")
    return curve, preds


# ---- the named demos -----------------------------------------------------------------------------------------------
SENTENCES = ["The movie was a delight from start to finish.", "I want my money back.", "A film about a boy and his dog."]
NER_TEXT = ["Hugging Face was founded in New York by Clement Delangue."]
QA_PAIRS = [("Where was Hugging Face founded?", "Hugging Face was founded in New York City in 2016 by three French engineers.")]


def _register():
    for fam, emb_repo, cls_repo, ner_repo, qa_repo in (
            ("bert", "bert-base-uncased", "nlptown/bert-base-multilingual-uncased-sentiment", "dslim/bert-base-NER",
             "deepset/bert-base-cased-squad2"),
            ("roberta", "roberta-base", "cardiffnlp/twitter-roberta-base-sentiment-latest", "Jean-Baptiste/roberta-large-ner-english",
             "deepset/roberta-base-squad2"),
            ("distilbert", "distilbert/distilbert-base-uncased", "distilbert/distilbert-base-uncased-finetuned-sst-2-english",
             "dslim/distilbert-NER", "distilbert/distilbert-base-cased-distilled-squad")):
        example(f"{fam}-embed", emb_repo, "sentence embeddings and their cosine similarities")(lambda repo, texts, out: embed(repo, texts or SENTENCES, out))
        example(f"{fam}-classify", cls_repo, "sequence classification")(lambda repo, texts, out: classify(repo, texts or SENTENCES, out))
        example(f"{fam}-ner", ner_repo, "token classification (named entities)")(lambda repo, texts, out: ner(repo, texts or NER_TEXT, out))
        example(f"{fam}-qa", qa_repo, "extractive question answering: [question context] pairs")(
            lambda repo, texts, out: qa(repo, list(zip(texts[0::2], texts[1::2])) if len(texts) >= 2 else QA_PAIRS, out))
    example("auto-classify", "distilbert/distilbert-base-uncased-finetuned-sst-2-english",
            "classification with the family picked from config.json")(lambda repo, texts, out: classify(repo, texts or SENTENCES, out))
    example("distilbert-finetune", "distilbert/distilbert-base-uncased-finetuned-sst-2-english",
            "fine-tune a classifier on four sentences: loss curve, predictions, export recipe")(
        lambda repo, texts, out: finetune(repo, texts or ["great", "awful", "wonderful", "terrible"], [1, 0, 1, 0][:len(texts) or 4], out=out))


_register()


def main(argv=None, out=print) -> int:
    ap = argparse.ArgumentParser(prog="flodl_b200.hf.examples")
    ap.add_argument("name", nargs="?", help="which demo (omit for the list)")
    ap.add_argument("--repo", help="hub id or local directory (default: the demo's public checkpoint)")
    ap.add_argument("texts", nargs="*", help="input sentences (question / context pairs for the qa demos)")
    from ..cli.args import answer_schema_probe
    answer_schema_probe(ap, argv)
    a = ap.parse_intermixed_args(argv)          # `name --repo X text ...`: positionals on both sides of the option
    if not a.name:
        for name, (repo, doc, _fn) in EXAMPLES.items():
            out(f"  {name:<22} {doc}  [{repo}]")
        return 0
    if a.name not in EXAMPLES:
        print(f"unknown example {a.name!r}; one of: {', '.join(EXAMPLES)}", file=sys.stderr)
        return 2
    repo, _doc, fn = EXAMPLES[a.name]
    try:
        fn(a.repo or repo, list(a.texts), out)
    except TensorError as e:
        print(f"{a.name}: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
