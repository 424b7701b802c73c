"""`from_pretrained`: resolve a repo id to files and build + load the model (flodl-hf/src/hub/mod.rs).
Files are looked up, in this order, in `repo_id` itself when it is a directory, in
`<HF_HOME>/flodl-converted/<repo>/` (where `python -m flodl_b200.hf.convert` writes), and in the HuggingFace hub
cache layout (`<HF_HOME>/hub/models--org--name/snapshots/*/`). What is not on disk is fetched from the hub
(`fetch_file`: `<HF_ENDPOINT or https://huggingface.co>/<repo>/resolve/<revision>/<file>`, bearer token from `HF_TOKEN`)
into that cache layout, unless `HF_HUB_OFFLINE=1`; a repo that can be neither found nor fetched is reported with
the paths and the URL that were tried."""
from __future__ import annotations

import glob
import os
from typing import List, Optional, Tuple

from ..tensor import TensorError
from .export import build_for_export, parse_head
from .models.auto import (AutoConfig, AutoModelForMaskedLM, AutoModelForQuestionAnswering, AutoModelForSequenceClassification,
                          AutoModelForTokenClassification)
from .safetensors_io import (bert_legacy_key_rename, load_safetensors_into_graph_with_rename_allow_unused, weights_have_pooler)


def hf_home() -> str:
    return os.environ.get("HF_HOME") or os.path.join(os.path.expanduser("~"), ".cache", "huggingface")


def candidate_dirs(repo_id: str) -> List[str]:
    out = []
    if os.path.isdir(repo_id):
        out.append(repo_id)
    out.append(os.path.join(hf_home(), "flodl-converted", repo_id))
    snap = os.path.join(hf_home(), "hub", "models--" + repo_id.replace("/", "--"), "snapshots")
    out.extend(sorted(glob.glob(os.path.join(snap, "*")), reverse=True))
    return out


def offline() -> bool:
    return os.environ.get("HF_HUB_OFFLINE", "0") not in ("0", "", "false", "False")


def endpoint() -> str:
    return (os.environ.get("HF_ENDPOINT") or "https://huggingface.co").rstrip("/")


def snapshot_dir(repo_id: str, revision: str = "main") -> str:
    return os.path.join(hf_home(), "hub", "models--" + repo_id.replace("/", "--"), "snapshots", revision)


def fetch_file(repo_id: str, filename: str, revision: str = "main", timeout_s: float = 30.0) -> str:
    """Download one file of a hub repo into the cache layout and return its path (an existing copy is reused).
    The body is streamed to `<name>.part` and renamed when complete, so an interrupted download leaves no
    half-written file under the final name."""
    import shutil
    import urllib.error
    import urllib.request
    dst = os.path.join(snapshot_dir(repo_id, revision), filename)
    if os.path.exists(dst):
        return dst
    if offline():
        raise TensorError(f"fetch_file({repo_id}, {filename}): HF_HUB_OFFLINE is set and {dst} does not exist")
    url = f"{endpoint()}/{repo_id}/resolve/{revision}/{filename}"
    req = urllib.request.Request(url, headers={"User-Agent": "flodl_b200"})
    token = os.environ.get("HF_TOKEN") or os.environ.get("HUGGING_FACE_HUB_TOKEN")
    if token:
        req.add_header("Authorization", f"Bearer {token}")
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    part = dst + ".part"
    try:
        with urllib.request.urlopen(req, timeout=timeout_s) as r, open(part, "wb") as f:
            shutil.copyfileobj(r, f, 1 << 20)
    except (urllib.error.URLError, OSError) as e:
        if os.path.exists(part):
            os.remove(part)
        raise TensorError(f"fetch_file: GET {url} failed: {e}") from e
    os.replace(part, dst)
    return dst


def resolve_files(repo_id: str, revision: str = "main") -> Tuple[str, str, Optional[str]]:
    """(config.json, model.safetensors, tokenizer.json or None); fetches what is missing when allowed."""
    tried = candidate_dirs(repo_id)
    cfg = st = tok = None
    for d in tried:
        c, s, t = (os.path.join(d, n) for n in ("config.json", "model.safetensors", "tokenizer.json"))
        cfg = cfg or (c if os.path.exists(c) else None)
        st = st or (s if os.path.exists(s) else None)
        tok = tok or (t if os.path.exists(t) else None)
    errors = []
    if (cfg is None or st is None) and not os.path.isdir(repo_id) and not offline():
        try:
            cfg = cfg or fetch_file(repo_id, "config.json", revision)
            st = st or fetch_file(repo_id, "model.safetensors", revision)
        except TensorError as e:
            errors.append(str(e))
        if tok is None and cfg is not None and st is not None:
            try:
                tok = fetch_file(repo_id, "tokenizer.json", revision)
            except TensorError:
                tok = None                    # optional: many repos ship only vocab.txt
    if cfg is None or st is None:
        raise TensorError(f"from_pretrained({repo_id}): config.json / model.safetensors not found; looked in: {tried}"
                          + (f"; {'; '.join(errors)}" if errors else "; HF_HUB_OFFLINE is set" if offline() else "")
                          + ". If the repo ships only `pytorch_model.bin`, run `python -m flodl_b200.hf.convert <repo or file>` first.")
    return cfg, st, tok


def resolve_tokenizer(repo_id: str, revision: str = "main") -> Optional[str]:
    """Path of the repo's `tokenizer.json` (on disk, else fetched when allowed), or None."""
    for d in candidate_dirs(repo_id):
        t = os.path.join(d, "tokenizer.json")
        if os.path.exists(t):
            return t
    if os.path.isdir(repo_id) or offline():
        return None
    try:
        return fetch_file(repo_id, "tokenizer.json", revision)
    except TensorError:
        return None


def fetch_config_str(repo_id: str, revision: str = "main") -> str:
    """The text of the repo's `config.json` alone (cheap: decides the family and head before any weights move)."""
    for d in candidate_dirs(repo_id):
        c = os.path.join(d, "config.json")
        if os.path.exists(c):
            return open(c).read()
    if os.path.isdir(repo_id) or offline():
        raise TensorError(f"config.json of {repo_id} not found; looked in: {candidate_dirs(repo_id)}")
    return open(fetch_file(repo_id, "config.json", revision)).read()


def _rename_for(model_type: str):
    prefix = {"distilbert": "distilbert.", "albert": "albert.", "deberta-v2": "deberta.", "bert": "bert.", "roberta": "roberta.",
              "xlm-roberta": "roberta."}[model_type]

    def rename(key: str) -> str:
        k = bert_legacy_key_rename(key)
        return k
    return rename, prefix


def _load(graph, weights: bytes, model_type: str, base_only: bool) -> List[str]:
    rename, prefix = _rename_for(model_type)
    if base_only:
        # a bare backbone checkpoint may lack the family prefix (saved from `XModel`), a head
        # checkpoint carries it: accept both
        from .safetensors_io import parse_header
        names = list(parse_header(weights)[0])
        if not any(n.startswith(prefix) for n in names):
            return load_safetensors_into_graph_with_rename_allow_unused(graph, weights, lambda k: prefix + rename(k))
    return load_safetensors_into_graph_with_rename_allow_unused(graph, weights, rename)


def from_pretrained(repo_id: str, device=None, head: Optional[str] = None):
    """Backbone graph (`head` None/"base") or the graph of a task head ("seqcls", "tokcls", "qa", "mlm")."""
    cfg_path, st_path, _ = resolve_files(repo_id)
    cfg = AutoConfig.from_json_str(open(cfg_path).read())
    weights = open(st_path, "rb").read()
    kind = parse_head(head) if head else "base"
    g = build_for_export(cfg, weights_have_pooler(weights), device, kind)
    _load(g, weights, cfg.model_type(), kind == "base")
    return g


def _head_from_pretrained(auto_cls, repo_id: str, device=None, family: Optional[str] = None):
    """`auto_cls`: an `AutoModelFor*` class (the family comes from config.json) or a family's own head class
    (`family` then names the `model_type` the repo must have)."""
    cfg_path, st_path, tok_path = resolve_files(repo_id)
    cfg = AutoConfig.from_json_str(open(cfg_path).read())
    if family is not None:
        _check_family(cfg, family, auto_cls.__name__, repo_id)
        h = _AUTO_BY_SUFFIX[_suffix_of(auto_cls)].from_config(cfg, device)
    else:
        h = auto_cls.from_config(cfg, device)
    _load(h.graph(), open(st_path, "rb").read(), cfg.model_type(), False)
    h.graph().set_training(False)
    if tok_path is not None:
        try:
            from .tokenizer import HfTokenizer
            h = h.with_tokenizer(HfTokenizer.from_file(tok_path))
        except TensorError:
            pass
    return h


def sequence_classification_from_pretrained(repo_id: str, device=None): return _head_from_pretrained(AutoModelForSequenceClassification, repo_id, device)
def token_classification_from_pretrained(repo_id: str, device=None): return _head_from_pretrained(AutoModelForTokenClassification, repo_id, device)
def question_answering_from_pretrained(repo_id: str, device=None): return _head_from_pretrained(AutoModelForQuestionAnswering, repo_id, device)
def masked_lm_from_pretrained(repo_id: str, device=None): return _head_from_pretrained(AutoModelForMaskedLM, repo_id, device)


# ---- `X.from_pretrained(repo)` on every family class and on the Auto classes (flodl-hf/src/hub/{mod,auto}.rs) ------
class HubExportHead:
    """Which head `AutoModel.from_pretrained_for_export_with_head` builds (hub/auto.rs `HubExportHead`)."""
    Base, SeqCls, TokCls, Qa, Mlm = "base", "seqcls", "tokcls", "qa", "mlm"

    @staticmethod
    def parse(s: str) -> str:
        if s not in ("base", "seqcls", "tokcls", "qa", "mlm"):
            raise TensorError(f"unsupported head `{s}`; expected one of auto|base|seqcls|tokcls|qa|mlm")
        return s


_AUTO_BY_SUFFIX = {"ForSequenceClassification": AutoModelForSequenceClassification, "ForTokenClassification": AutoModelForTokenClassification,
                   "ForQuestionAnswering": AutoModelForQuestionAnswering, "ForMaskedLM": AutoModelForMaskedLM}
_HEAD_OF_SUFFIX = {"ForSequenceClassification": HubExportHead.SeqCls, "ForTokenClassification": HubExportHead.TokCls,
                   "ForQuestionAnswering": HubExportHead.Qa, "ForMaskedLM": HubExportHead.Mlm}


def _suffix_of(cls) -> str:
    for suf in _AUTO_BY_SUFFIX:
        if cls.__name__.endswith(suf):
            return suf
    return "Model"


def _check_family(cfg: AutoConfig, family: str, cls_name: str, repo_id: str) -> None:
    if cfg.model_type() != family:
        raise TensorError(f"{cls_name}.from_pretrained({repo_id}): config.json says model_type {cfg.model_type()!r}, this class loads {family!r}; "
                          f"use the matching family class or AutoModel")


def _backbone_from_pretrained(repo_id: str, device=None, family: Optional[str] = None, keep_pooler: bool = True, cls_name: str = "AutoModel"):
    cfg_path, st_path, _ = resolve_files(repo_id)
    cfg = AutoConfig.from_json_str(open(cfg_path).read())
    if family is not None:
        _check_family(cfg, family, cls_name, repo_id)
    weights = open(st_path, "rb").read()
    g = build_for_export(cfg, keep_pooler and weights_have_pooler(weights), device, "base")
    _load(g, weights, cfg.model_type(), True)
    # the sidecar of a later save_checkpoint names the class that was built, not the repo's pretraining class
    g.set_source_config(cfg.into_normalized_config_json(cfg.base_class_name()))
    return g


def classify_for_hub_export(arch: str) -> str:
    """`architectures[0]` of a repo -> the head to rebuild for export; pretraining classes fall back to the backbone."""
    for suf, kind in _HEAD_OF_SUFFIX.items():
        if arch.endswith(suf):
            return kind
    return HubExportHead.Base


def _export_graph(repo_id: str, head: Optional[str], device=None):
    if head is None:
        archs = AutoConfig.from_json_str(fetch_config_str(repo_id)).architectures() or []
        head = classify_for_hub_export(archs[0]) if archs else HubExportHead.Base
    if head == HubExportHead.Base:
        return _backbone_from_pretrained(repo_id, device, None, True)
    auto = {v: _AUTO_BY_SUFFIX[k] for k, v in _HEAD_OF_SUFFIX.items()}[head]
    return _head_from_pretrained(auto, repo_id, device).into_graph()


def _install_from_pretrained() -> None:
    from .models import auto as _auto
    from .tokenizer import HfTokenizer  # noqa: F401  (HfTokenizer.from_pretrained resolves through this module)

    def on(cls, name, fn):
        setattr(cls, name, classmethod(fn) if not isinstance(fn, staticmethod) else fn)

    for model_type, (_cfg_cls, _base_name, mod) in _auto._FAMILIES.items():
        prefix = _auto._PREFIX[model_type]
        base = getattr(mod, prefix + "Model")
        on(base, "from_pretrained_on_device", lambda cls, repo_id, device=None, _f=model_type: _backbone_from_pretrained(repo_id, device, _f, True, cls.__name__))
        on(base, "from_pretrained", lambda cls, repo_id: cls.from_pretrained_on_device(repo_id, None))
        for suf in _AUTO_BY_SUFFIX:
            head = getattr(mod, prefix + suf, None)
            if head is None:
                continue
            on(head, "from_pretrained_on_device", lambda cls, repo_id, device=None, _f=model_type: _head_from_pretrained(cls, repo_id, device, _f))
            on(head, "from_pretrained", lambda cls, repo_id: cls.from_pretrained_on_device(repo_id, None))
    for auto_head in _AUTO_BY_SUFFIX.values():
        on(auto_head, "from_pretrained_on_device", lambda cls, repo_id, device=None: _head_from_pretrained(cls, repo_id, device))
        on(auto_head, "from_pretrained", lambda cls, repo_id: cls.from_pretrained_on_device(repo_id, None))
    A = _auto.AutoModel
    # uniform `[batch, seq, hidden]` output over all families: pooler-bearing ones are built without it
    A.from_pretrained_on_device = staticmethod(lambda repo_id, device=None: _backbone_from_pretrained(repo_id, device, None, False))
    A.from_pretrained = staticmethod(lambda repo_id: A.from_pretrained_on_device(repo_id, None))
    A.from_pretrained_for_export_on_device = staticmethod(lambda repo_id, device=None: _export_graph(repo_id, None, device))
    A.from_pretrained_for_export = staticmethod(lambda repo_id: _export_graph(repo_id, None, None))
    A.from_pretrained_for_export_with_head_on_device = staticmethod(lambda repo_id, head, device=None: _export_graph(repo_id, parse_head(head), device))
    A.from_pretrained_for_export_with_head = staticmethod(lambda repo_id, head: _export_graph(repo_id, parse_head(head), None))
    _auto.AutoConfig.from_pretrained = classmethod(lambda cls, repo_id: cls.from_json_str(fetch_config_str(repo_id)))


_install_from_pretrained()
