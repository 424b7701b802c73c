"""`python -m flodl_b200.hf.export_tool (--hub <repo> | --checkpoint <file.fdl>) --out <dir> [--head KIND] [--config FILE]`:
write a Hugging Face directory (`model.safetensors` + `config.json`) with this library's own writer
(flodl-hf/examples/export_hf.rs).

* `--hub <repo_id>`: fetch the repo (or read it from the caches), rebuild the matching graph, write the export. The head
  follows `architectures[0]` unless `--head base|seqcls|tokcls|qa|mlm` overrides it (`--head base` re-exports a
  pretraining checkpoint as a plain encoder). The written config gets `flodl_source_repo: <repo_id>` so that
  `verify_export` can find the upstream to compare against.
* `--checkpoint <file.fdl>`: weights from a local checkpoint, architecture from its `<stem>.config.json` sidecar or an
  explicit `--config <file>`.
"""
from __future__ import annotations

import json
import os
import sys
from dataclasses import dataclass
from typing import Optional

from ..cli.args import ArgError, FdlArgs, arg
from ..tensor import TensorError


@dataclass
class ExportToolArgs(FdlArgs):
    """Export a hub repo or a local checkpoint as a Hugging Face directory (bert / roberta / distilbert / xlm-roberta /
    albert / deberta-v2, picked from `model_type`)."""
    hub: Optional[str] = arg(None, help="hub repo id (or local repo directory) to re-export")
    checkpoint: Optional[str] = arg(None, help=".fdl checkpoint to export")
    out: str = arg("hf_export", help="output directory")
    head: str = arg("auto", help="head to build", choices=["auto", "base", "seqcls", "tokcls", "qa", "mlm"])
    config: Optional[str] = arg(None, help="config.json to use with --checkpoint instead of the sidecar")
    device: str = arg("cpu", help="device to build on")


def stamp_source_repo(config_json: str, repo_id: str) -> str:
    cfg = json.loads(config_json)
    cfg["flodl_source_repo"] = repo_id
    return json.dumps(cfg, indent=2, sort_keys=True)


def export_from_hub(repo_id: str, out_dir: str, head: str = "auto", device=None) -> str:
    from .export import export_hf_dir
    from .models.auto import AutoModel
    g = (AutoModel.from_pretrained_for_export_on_device(repo_id, device) if head == "auto"
         else AutoModel.from_pretrained_for_export_with_head_on_device(repo_id, head, device))
    cfg_json = g.source_config()
    if cfg_json is None:
        raise TensorError(f"export: the graph built for {repo_id} carries no source config")
    export_hf_dir(g, stamp_source_repo(cfg_json, repo_id), out_dir)
    return out_dir


def export_from_checkpoint(path: str, out_dir: str, config_path: Optional[str] = None, device=None) -> str:
    from ..nn.checkpoint import checkpoint_keys
    from .export import build_for_export, export_checkpoint, export_hf_dir
    from .models.auto import AutoConfig
    from .safetensors_io import keys_have_pooler
    if config_path is None:
        export_checkpoint(path, out_dir, device)
        return out_dir
    cfg_json = open(config_path).read()
    g = build_for_export(AutoConfig.from_json_str(cfg_json), keys_have_pooler(checkpoint_keys(path)), device)
    g.load_checkpoint(path)
    export_hf_dir(g, cfg_json, out_dir)
    return out_dir


def main(argv=None) -> int:
    try:
        a = ExportToolArgs.parse(sys.argv[1:] if argv is None else argv, "flodl_b200.hf.export_tool")
        if (a.hub is None) == (a.checkpoint is None):
            raise ArgError("give exactly one of --hub <repo> and --checkpoint <file.fdl>")
        if a.hub is not None:
            export_from_hub(a.hub, a.out, a.head, a.device)
        else:
            if a.head != "auto":
                raise ArgError("--head applies to --hub; a checkpoint's head is the one named in its config")
            export_from_checkpoint(a.checkpoint, a.out, a.config, a.device)
    except (ArgError, TensorError, OSError) as e:
        print(f"export: {e}", file=sys.stderr)
        return 2
    print(f"wrote {os.path.join(a.out, 'model.safetensors')} and {os.path.join(a.out, 'config.json')}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
