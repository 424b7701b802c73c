"""Named-tensor checkpoints in the `.fdl` format (flodl/src/nn/checkpoint.rs).

Layout, little-endian: "FDLC" | u32 version (2; reader accepts 1..=2) | 32-byte structural hash
(zeros = unchecked) | u32 count | count x { u32 name_len, name, u32 ndim, i64 shape[ndim],
u8 dtype (1=f16 2=bf16 3=f32 4=f64 5=i32 6=i64), u64 nbytes, raw bytes }. Parameters come first,
then buffers. A path ending in ".gz" gzips the whole stream. The byte-level reader / writer is the
C++ runtime (`csrc/runtime/runtime.cpp`); this module holds the matching policy: by-name load with
a `LoadReport`, shape mismatch is an error, dtype is cast to the model's, hash mismatch is an
error only when both sides are non-zero; `migrate_checkpoint` re-keys an old file.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _ext
from ..tensor import TensorError
from .module import Buffer, Parameter

VERSION = 2
HASH_LEN = 32


@dataclass
class LoadReport:
    loaded: List[str] = field(default_factory=list)
    skipped: List[str] = field(default_factory=list)   # in the file, not in the model
    missing: List[str] = field(default_factory=list)   # in the model, not in the file


@dataclass
class MigrateReport:
    unchanged: List[str] = field(default_factory=list)
    remapped: List[Tuple[str, str]] = field(default_factory=list)
    dropped: List[str] = field(default_factory=list)
    missing: List[str] = field(default_factory=list)

    def is_complete(self) -> bool:
        return not self.dropped and not self.missing

    def __str__(self) -> str:
        out = []
        for title, items in (("unchanged", self.unchanged), ("remapped", [f"{a} -> {b}" for a, b in self.remapped]),
                             ("dropped", self.dropped), ("missing", self.missing)):
            if items:
                out.append(f"{title} ({len(items)}):")
                out.extend(f"  {i}" for i in items)
        return "\n".join(out)


def _hash_bytes(hex_hash: Optional[str]) -> bytes:
    if not hex_hash:
        return b"\0" * HASH_LEN
    try:
        b = bytes.fromhex(hex_hash)
    except ValueError as e:
        raise TensorError(f"invalid structural hash: {e}")
    if len(b) != HASH_LEN:
        raise TensorError("structural hash must be 32 bytes (64 hex chars)")
    return b


def _entries(params, buffers):
    out = [(n, p.variable.data() if isinstance(p, Parameter) else p) for n, p in params]
    out += [(n, b.get() if isinstance(b, Buffer) else b) for n, b in buffers]
    return out


def save_checkpoint(params: Sequence[Tuple[str, Parameter]], buffers: Sequence[Tuple[str, Buffer]],
                    structural_hash: Optional[str] = None) -> bytes:
    return _ext.require().fdl_save_bytes(_entries(params, buffers), _hash_bytes(structural_hash), VERSION)


def save_checkpoint_file(path: str, params, buffers, structural_hash: Optional[str] = None) -> None:
    _ext.require().fdl_save(path, _entries(params, buffers), _hash_bytes(structural_hash), VERSION)


def _apply(raw, params, buffers, structural_hash) -> LoadReport:
    version, file_hash, entries = raw
    expected = _hash_bytes(structural_hash)
    if any(file_hash) and any(expected) and bytes(file_hash) != expected:
        raise TensorError(f"checkpoint architecture mismatch: file={bytes(file_hash).hex()} model={structural_hash}")
    targets = {}
    for n, p in params:
        targets[n] = ("p", p)
    for n, b in buffers:
        targets[n] = ("b", b)
    report = LoadReport()
    seen = set()
    for name, t in entries:
        tgt = targets.get(name)
        if tgt is None:
            report.skipped.append(name)
            continue
        kind, obj = tgt
        cur = obj.variable.t if kind == "p" else obj.get()
        if list(cur.shape) != list(t.shape):
            raise TensorError(f"checkpoint shape mismatch for '{name}': file={list(t.shape)} model={list(cur.shape)}")
        val = t.to(device=cur.device, dtype=cur.dtype)
        if kind == "p":
            obj.variable.set_data(val)
        else:
            obj.set(val)
        seen.add(name)
        report.loaded.append(name)
    report.missing = [n for n in targets if n not in seen]
    return report


def load_checkpoint(data: bytes, params, buffers, structural_hash: Optional[str] = None) -> LoadReport:
    rep = _apply(_ext.require().fdl_load_bytes(data, False), params, buffers, structural_hash)
    _sync_shadows(params)
    return rep


def load_checkpoint_file(path: str, params, buffers, structural_hash: Optional[str] = None) -> LoadReport:
    try:
        raw = _ext.require().fdl_load(path, False)
    except RuntimeError as e:
        raise TensorError(str(e).split("\n")[0])
    rep = _apply(raw, params, buffers, structural_hash)
    _sync_shadows(params)
    return rep


def _sync_shadows(params) -> None:
    for _, p in params:
        t = p.variable.t if isinstance(p, Parameter) else p
        sh = getattr(t, "_fb_bf16", None)
        if sh is not None:
            sh.copy_(t.detach())


def checkpoint_keys(path: str) -> List[str]:
    return [n for n, _ in _ext.require().fdl_load(path, True)[2]]


def checkpoint_version(path: str) -> int:
    return int(_ext.require().fdl_load(path, True)[0])


def migrate_checkpoint(data: bytes, params, buffers) -> Tuple[bytes, MigrateReport]:
    """Re-key a checkpoint for a renamed model: exact name+shape matches first, then the first
    unused entry with the same shape and dtype, in file order. Writes a zero hash."""
    C = _ext.require()
    _, _, entries = C.fdl_load_bytes(data, False)
    targets = [(n, list(p.variable.t.shape), p.variable.t.dtype) for n, p in params]
    targets += [(n, list(b.get().shape), b.get().dtype) for n, b in buffers]
    rep = MigrateReport()
    used = [False] * len(entries)
    index = {n: i for i, (n, _) in enumerate(entries)}
    output, unmatched = [], []
    for name, shape, dt in targets:
        ci = index.get(name)
        if ci is not None and not used[ci] and list(entries[ci][1].shape) == shape:
            rep.unchanged.append(name)
            used[ci] = True
            output.append((name, entries[ci][1]))
        else:
            unmatched.append((name, shape, dt))
    for name, shape, dt in unmatched:
        found = next((i for i, (_, t) in enumerate(entries) if not used[i] and list(t.shape) == shape and t.dtype == dt), None)
        if found is None:
            rep.missing.append(name)
        else:
            rep.remapped.append((entries[found][0], name))
            used[found] = True
            output.append((name, entries[found][1]))
    rep.dropped = [n for i, (n, _) in enumerate(entries) if not used[i]]
    return C.fdl_save_bytes(output, b"\0" * HASH_LEN, VERSION), rep


def migrate_checkpoint_file(src: str, dst: str, params, buffers) -> MigrateReport:
    import gzip
    opener = gzip.open if src.endswith(".gz") else open
    with opener(src, "rb") as f:
        data = f.read()
    out, rep = migrate_checkpoint(data, params, buffers)
    opener = gzip.open if dst.endswith(".gz") else open
    with opener(dst, "wb") as f:
        f.write(out)
    return rep
