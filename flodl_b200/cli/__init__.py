"""`fdl`-style command line: `python -m flodl_b200.cli <command>` (flodl-cli/src/main.rs).

Built-ins: `diagnose`, `build`, `bench`, `export-hf`, `api-ref`, `schema`, `completions`,
`config show`, `init`; anything else is looked up in the nearest `fdl.yml` manifest."""
from .args import REQUIRED, ArgError, FdlArgs, arg  # noqa: F401
from .main import main  # noqa: F401
from .args import answer_schema_probe, argparse_schema  # noqa: F401
from .manifest import (ManifestError, command_help, compose, config_to_args, deep_merge, find_manifest, load_manifest, resolve,  # noqa: F401
                       resolve_command, run_command)  # noqa: F401
