"""Multi-GPU training: process group and symmetric memory (`comm`), flat parameter buffers (`flat`), gradient
exchange (`grad_sync`), the whole-step engine (`engine`), synchronous DDP (`ddp`), El Che (`el_che`) and the
asynchronous coordinator / worker path (`ddp_run`).

The names most programs need are importable from here; they are resolved on first use so that importing the
package stays cheap and free of import cycles."""
from __future__ import annotations

_EXPORTS = {
    "TrainEngine": ("engine", "TrainEngine"),
    "Trainer": ("ddp", "Trainer"),
    "Ddp": ("ddp", "Ddp"),
    "DdpConfig": ("ddp", "DdpConfig"),
    "DistributedState": ("ddp", "DistributedState"),
    "ElChe": ("el_che", "ElChe"),
    "FlatParams": ("flat", "FlatParams"),
    "GradSync": ("grad_sync", "GradSync"),
    "SymmetricBuffer": ("comm", "SymmetricBuffer"),
    "init_process_group": ("comm", "init_process_group"),
    "destroy_process_group": ("comm", "destroy_process_group"),
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str):
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib
    value = getattr(importlib.import_module(f"{__name__}.{target[0]}"), target[1])
    globals()[name] = value
    return value
