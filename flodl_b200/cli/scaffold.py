"""Project scaffolds: `fdl init <name> [--docker | --native] [--with-hf]` and `fdl add flodl-hf`
(flodl-cli/src/{init,add}.rs).

Every mode writes `train.py`, `requirements.txt`, `.gitignore`, `README.md` and `fdl.yml.example` (copied to a git-ignored
`fdl.yml` on first use). The docker modes add a `Dockerfile`, a `docker-compose.yml` with a `dev` (CPU) and a `cuda` service,
and `docker: dev` / `docker: cuda` on the manifest's commands so that `fdl train` runs inside the service; native mode runs
on the host. `--with-hf` (or `fdl add flodl-hf` later) adds a side directory with a Hugging Face playground and a manifest
of its own; it never edits the project's files.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

TRAIN = '''"""Training entry point."""
import torch
from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder
from flodl_b200.parallel.ddp import Trainer

dev = "cuda" if torch.cuda.is_available() else "cpu"
model = (FlowBuilder.from_(nn.Linear(2, 16, True, dev)).through(nn.GELU()).through(nn.LayerNorm(16, device=dev))
         .also(nn.Linear(16, 16, True, dev)).through(nn.Linear(16, 2, True, dev)).build())
Trainer.setup(model, None, lambda ps: nn.Adam(ps, 1e-2))      # one rank or many: the same three lines below
for step in range(200):
    x = torch.randn(32, 2, device=dev)
    y = torch.stack([x[:, 0].sin(), x[:, 1].cos()], 1)
    loss = nn.mse_loss(model.forward(Variable.wrap(x)), Variable.wrap(y))
    loss.backward()
    model.step()
    if step % 50 == 0:
        print(step, loss.item())
model.save_checkpoint("model.fdl")
'''

DOCKERFILE = '''# {kind} image for {name}: PyTorch + flodl_b200 (the native kernels build for sm_100a inside the cuda image)
FROM {base}
WORKDIR /workspace
COPY requirements.txt .
RUN python -m pip install --no-cache-dir -r requirements.txt
'''

COMPOSE = '''services:
  dev:
    build: {{context: ., dockerfile: Dockerfile}}
    volumes: [".:/workspace"]
    working_dir: /workspace
  cuda:
    build: {{context: ., dockerfile: Dockerfile.cuda}}
    volumes: [".:/workspace"]
    working_dir: /workspace
    deploy:
      resources:
        reservations:
          devices: [{{driver: nvidia, count: all, capabilities: [gpu]}}]
'''

GITIGNORE = "__pycache__/\n*.pyc\n/fdl.yml\n.fdl/\n*.fdl\nruns/\n"


def manifest_text(name: str, docker: bool, with_hf: bool) -> str:
    def cmd(key: str, desc: str, run: str, service: Optional[str]) -> str:
        return f"  {key}:\n    description: {desc}\n    run: {run}\n" + (f"    docker: {service}\n" if docker and service else "")
    out = f"description: {name}\n\ncommands:\n"
    if with_hf:
        out += "  flodl-hf:                    # ./flodl-hf/fdl.yml\n"
    out += cmd("train", "Train the model", "python train.py", "dev")
    out += cmd("test", "Run the tests", "python -m pytest -q", "dev")
    out += cmd("check", "Import the package and report the machine", "python -m flodl_b200.cli diagnose", "dev")
    out += cmd("cuda-train", "Train on the GPU(s)", "python train.py", "cuda")
    out += cmd("cuda-train-ddp", "One process per GPU", "python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node gpu train.py", "cuda")
    out += cmd("cuda-build", "Compile the native kernels for sm_100a", "python -m flodl_b200.cli build", "cuda")
    if docker:
        out += cmd("shell", "Interactive shell in the dev container", "bash", "dev") + cmd("cuda-shell", "Interactive shell in the CUDA container", "bash", "cuda")
    return out


def project_files(name: str, mode: str = "docker", with_hf: bool = False) -> Dict[str, str]:
    """Relative path -> content of a new project. `mode`: "docker" or "native"."""
    if mode not in ("docker", "native"):
        raise ValueError(f"unknown scaffold mode {mode!r}")
    docker = mode == "docker"
    files = {"train.py": TRAIN, "requirements.txt": "torch>=2.6\nnumpy\npyyaml\n", ".gitignore": GITIGNORE,
             "fdl.yml.example": manifest_text(name, docker, with_hf),
             "README.md": f"# {name}\n\n```\npython -m flodl_b200.cli train        # or: cuda-train, cuda-train-ddp, test, check\n```\n\n"
                          + ("Commands run inside the `dev` / `cuda` docker compose services.\n" if docker else
                             "Commands run on the host: install the requirements, then `python -m flodl_b200.cli setup`.\n")}
    if docker:
        files["Dockerfile"] = DOCKERFILE.format(kind="CPU", name=name, base="python:3.12-slim")
        files["Dockerfile.cuda"] = DOCKERFILE.format(kind="CUDA", name=name, base="nvidia/cuda:12.8.0-cudnn-devel-ubuntu22.04")
        files["docker-compose.yml"] = COMPOSE.format()
    if with_hf:
        files.update({os.path.join("flodl-hf", k): v for k, v in hf_files(docker).items()})
    return files


def write_files(root: str, files: Dict[str, str]) -> List[str]:
    written = []
    for rel, text in files.items():
        path = os.path.join(root, rel)
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w") as f:
            f.write(text)
        written.append(rel)
    return written


# ---- the Hugging Face playground ---------------------------------------------------------------------------------
HF_CLASSIFY = '''"""Classify text with any supported encoder family (BERT, RoBERTa, XLM-R, DistilBERT, ALBERT, DeBERTa-v2)."""
import sys

from flodl_b200 import hf

repo = sys.argv[1] if len(sys.argv) > 1 else "distilbert/distilbert-base-uncased-finetuned-sst-2-english"
texts = sys.argv[2:] or ["this framework is a joy to use", "the build failed again"]
head = hf.AutoModelForSequenceClassification.from_pretrained(repo)        # config, weights and tokenizer from the hub cache
for text, dist in zip(texts, head.predict(texts)):
    label, p = dist[0]
    print(f"{label:<10} {p:.3f}  {text}")
'''

HF_README = '''# flodl-hf playground

A side directory for trying the Hugging Face integration; nothing in the parent project depends on it.

```
python -m flodl_b200.cli flodl-hf classify                       # DistilBERT sentiment on two sample sentences
python -m flodl_b200.cli flodl-hf bert                           # fill-mask with bert-base-uncased
python -m flodl_b200.cli flodl-hf convert -- <repo or .bin file>  # pytorch_model.bin -> model.safetensors
```

Weights are looked up in the repo directory itself, `$HF_HOME/flodl-converted/<repo>/` and the hub cache, then downloaded
(`HF_HUB_OFFLINE=1` forbids that). Repos that ship only `pytorch_model.bin` need the `convert` step once.
'''


def hf_manifest(docker: bool) -> str:
    tail = "    docker: dev\n" if docker else ""
    rows = [("classify", "Sentiment with a DistilBERT classifier", "python classify.py"),
            ("distilbert-sentiment", "Same, spelled out", "python classify.py distilbert/distilbert-base-uncased-finetuned-sst-2-english"),
            ("roberta-sentiment", "RoBERTa sentiment classifier", "python classify.py cardiffnlp/twitter-roberta-base-sentiment-latest"),
            ("bert", "Fill-mask with bert-base-uncased", "python fill_mask.py"),
            ("convert", "pytorch_model.bin -> model.safetensors", "python -m flodl_b200.hf.convert"),
            ("check", "Import the package", "python -m flodl_b200.cli diagnose")]
    out = "description: Hugging Face playground\n\ncommands:\n"
    for key, desc, run in rows:
        out += f"  {key}:\n    description: {desc}\n    run: {run}\n{tail}"
    return out


HF_FILL_MASK = '''"""Fill-mask with a masked-LM head: the top candidates for every [MASK] of the sentence."""
import sys

from flodl_b200 import hf

repo = sys.argv[1] if len(sys.argv) > 1 else "bert-base-uncased"
text = sys.argv[2] if len(sys.argv) > 2 else "paris is the [MASK] of france"
head = hf.AutoModelForMaskedLM.from_pretrained(repo)
for slot in head.fill_mask(text, 5):
    print("  ".join(f"{tok} ({p:.2f})" for tok, p in slot))
'''


def hf_files(docker: bool) -> Dict[str, str]:
    return {"classify.py": HF_CLASSIFY, "fill_mask.py": HF_FILL_MASK, "fdl.yml": hf_manifest(docker), "README.md": HF_README}


def add_flodl_hf(project_dir: str) -> List[str]:
    """Scaffold `./flodl-hf/` inside an initialised project. Docker mode is read off the project (a `docker-compose.yml`
    keeps `docker: dev` on the commands); an existing `./flodl-hf/` is never overwritten; the project's own files are
    left alone."""
    from .manifest import manifest_in
    if manifest_in(project_dir) is None:
        raise FileExistsError("`add flodl-hf` expects an initialised flodl project (no fdl.yml or fdl.yml.example here)")
    target = os.path.join(project_dir, "flodl-hf")
    if os.path.exists(target):
        raise FileExistsError(f"{target} already exists; delete it to regenerate")
    docker = os.path.isfile(os.path.join(project_dir, "docker-compose.yml"))
    return [os.path.join("flodl-hf", f) for f in write_files(target, hf_files(docker))]
