"""`python -m flodl_b200.hf.convert <repo-id | directory | pytorch_model.bin> [--out DIR]`

Turns a `pytorch_model.bin` checkpoint (a pickled state dict) into `model.safetensors` so `from_pretrained` can load
it (flodl-hf/scripts/convert_bin_to_safetensors.py). The result goes to `<HF_HOME>/flodl-converted/<repo>/` (the first
place `from_pretrained` looks) together with a copy of `config.json` / `tokenizer.json` when they sit beside the input.

The pickle is read with `torch.load(..., weights_only=True)`: tensors only, no code from the file is executed.
Shared tensors (tied embeddings) are written once per name, made contiguous, since safetensors has no aliasing.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
from typing import Dict, Optional

import torch

from . import hub
from .safetensors_io import write_safetensors


def load_state_dict(path: str) -> Dict[str, torch.Tensor]:
    sd = torch.load(path, map_location="cpu", weights_only=True)
    if isinstance(sd, dict) and "state_dict" in sd and isinstance(sd["state_dict"], dict):
        sd = sd["state_dict"]
    if not isinstance(sd, dict):
        raise ValueError(f"{path}: expected a state dict, got {type(sd).__name__}")
    out = {}
    for k, v in sd.items():
        if isinstance(v, torch.Tensor):
            out[str(k)] = v.detach().contiguous()
    if not out:
        raise ValueError(f"{path}: no tensors found")
    return out


def find_bin(src: str) -> str:
    if os.path.isfile(src):
        return src
    for d in ([src] if os.path.isdir(src) else []) + hub.candidate_dirs(src):
        p = os.path.join(d, "pytorch_model.bin")
        if os.path.isfile(p):
            return p
    if not os.path.isdir(src) and not hub.offline():
        return hub.fetch_file(src, "pytorch_model.bin")
    raise FileNotFoundError(f"no pytorch_model.bin for {src!r}")


def convert(src: str, out_dir: Optional[str] = None) -> str:
    """Returns the path of the written `model.safetensors`."""
    bin_path = find_bin(src)
    repo = src if not os.path.exists(src) else os.path.basename(os.path.dirname(os.path.abspath(bin_path)))
    out_dir = out_dir or os.path.join(hub.hf_home(), "flodl-converted", repo)
    os.makedirs(out_dir, exist_ok=True)
    tensors = load_state_dict(bin_path)
    dst = os.path.join(out_dir, "model.safetensors")
    with open(dst + ".part", "wb") as f:
        f.write(write_safetensors(tensors, {"format": "pt", "converted_from": os.path.basename(bin_path)}))
    os.replace(dst + ".part", dst)
    for side in ("config.json", "tokenizer.json", "vocab.txt", "tokenizer_config.json", "special_tokens_map.json"):
        p = os.path.join(os.path.dirname(bin_path), side)
        if os.path.isfile(p) and not os.path.exists(os.path.join(out_dir, side)):
            shutil.copyfile(p, os.path.join(out_dir, side))
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m flodl_b200.hf.convert", description=__doc__.split("\n\n")[1])
    ap.add_argument("source", help="hub repo id, a directory holding pytorch_model.bin, or the .bin file itself")
    ap.add_argument("--out", default=None, help="output directory (default: <HF_HOME>/flodl-converted/<repo>)")
    a = ap.parse_args(argv)
    try:
        dst = convert(a.source, a.out)
    except Exception as e:  # noqa: BLE001
        print(f"convert: {e}", file=sys.stderr)
        return 1
    print(dst)
    return 0


if __name__ == "__main__":
    sys.exit(main())
