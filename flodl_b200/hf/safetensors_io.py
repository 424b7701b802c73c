"""safetensors <-> graph (flodl-hf/src/safetensors_io.rs).

The file format is parsed here directly: 8-byte little-endian header length, a JSON header mapping
tensor name -> {dtype, shape, data_offsets}, then the raw little-endian tensor bytes. Loading is
validate-then-commit: every expected key must be present with the right shape (and, unless allowed,
no extra keys) before a single parameter is touched. Only floating-point tensors are accepted.
Graph keys map to HuggingFace keys by replacing the last '/' with '.'.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..tensor import TensorError
from .path import hf_key_from_flodl_key

_DTYPES = {"F32": torch.float32, "F64": torch.float64, "F16": torch.float16, "BF16": torch.bfloat16}
_NAMES = {v: k for k, v in _DTYPES.items()}
_INT_DTYPES = {"I64", "I32", "I16", "I8", "U8", "BOOL", "U16", "U32", "U64"}


# ---- raw format ------------------------------------------------------------------------------------
def parse_header(data: bytes) -> Tuple[Dict[str, dict], int]:
    """(header without `__metadata__`, offset of the data section)."""
    if len(data) < 8:
        raise TensorError("safetensors parse error: file shorter than its 8-byte header length")
    (n,) = struct.unpack("<Q", data[:8])
    if n > len(data) - 8:
        raise TensorError(f"safetensors parse error: header length {n} exceeds file size {len(data)}")
    try:
        header = json.loads(data[8:8 + n].decode("utf-8"))
    except Exception as e:
        raise TensorError(f"safetensors parse error: {e}")
    if not isinstance(header, dict):
        raise TensorError("safetensors parse error: the header is not a JSON object")
    header.pop("__metadata__", None)
    base = 8 + n
    for name, info in header.items():
        offs = info.get("data_offsets") if isinstance(info, dict) else None
        shape = info.get("shape") if isinstance(info, dict) else None
        if (not isinstance(info.get("dtype") if isinstance(info, dict) else None, str) or not isinstance(offs, list) or len(offs) != 2
                or not all(isinstance(x, int) and not isinstance(x, bool) for x in offs) or not isinstance(shape, list)
                or not all(isinstance(x, int) and not isinstance(x, bool) and x >= 0 for x in shape)):
            raise TensorError(f"safetensors parse error: entry {name!r} needs a string `dtype`, a `shape` of non-negative integers and two integer `data_offsets`")
        a, b = offs
        if a < 0 or a > b or base + b > len(data):
            raise TensorError(f"safetensors parse error: tensor {name!r} data range [{a}, {b}) is outside the file")
    return header, base


def tensor_from_entry(data: bytes, base: int, name: str, info: dict, device=None) -> torch.Tensor:
    dt = info["dtype"]
    if dt not in _DTYPES:
        raise TensorError(f"unsupported safetensors dtype {dt} for {name!r} — floats (F32/F64/BF16/F16) only")
    a, b = info["data_offsets"]
    shape = [int(s) for s in info["shape"]]
    numel = 1
    for s in shape:
        numel *= s
    esz = torch.empty((), dtype=_DTYPES[dt]).element_size()
    if (b - a) != numel * esz:
        raise TensorError(f"safetensors tensor {name!r}: {b - a} bytes for shape {shape} of {dt}")
    if numel == 0:
        t = torch.empty(shape, dtype=_DTYPES[dt])
    else:
        t = torch.frombuffer(bytearray(data[base + a:base + b]), dtype=_DTYPES[dt]).view(shape)
    return t if device is None else t.to(device)


def read_safetensors(data: bytes) -> Dict[str, torch.Tensor]:
    header, base = parse_header(data)
    return {k: tensor_from_entry(data, base, k, v) for k, v in header.items()}


def write_safetensors(tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> bytes:
    """Keys in sorted order, data packed back to back, header padded with spaces to 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    blobs, off = [], 0
    for k in sorted(tensors):
        t = tensors[k].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise TensorError(f"save_safetensors: dtype {t.dtype} of {k!r} not supported — only floating-point parameters / buffers can be serialised")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""      # reshape: a 0-dim tensor cannot be viewed as bytes
        header[k] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    return struct.pack("<Q", len(hj)) + hj + b"".join(blobs)


# ---- validation ------------------------------------------------------------------------------------
@dataclass
class ExpectedParam:
    key: str
    shape: List[int]


@dataclass
class ShapeMismatch:
    key: str
    expected: List[int]
    found: List[int]


@dataclass
class LoadValidation:
    missing: List[str] = field(default_factory=list)
    unused: List[str] = field(default_factory=list)
    shape_mismatches: List[ShapeMismatch] = field(default_factory=list)

    def is_ok(self) -> bool:
        return not (self.missing or self.unused or self.shape_mismatches)

    def _message(self, with_unused: bool) -> str:
        msg = "safetensors checkpoint does not match the model:\n"

        def listing(title, items, fmt):
            nonlocal msg
            if not items:
                return
            msg += f"  {len(items)} {title}:\n"
            for it in items[:20]:
                msg += f"    - {fmt(it)}\n"
            if len(items) > 20:
                msg += f"    ... and {len(items) - 20} more\n"
        listing("missing key(s) (model expects, checkpoint lacks)", self.missing, str)
        if with_unused:
            listing("unused key(s) (checkpoint has, model lacks)", self.unused, str)
        listing("shape mismatch(es)", self.shape_mismatches, lambda m: f"{m.key}: expected {m.expected}, found {m.found}")
        return msg

    def into_result(self) -> None:
        if not self.is_ok():
            raise TensorError(self._message(True))

    def into_result_allow_unused(self) -> None:
        if self.missing or self.shape_mismatches:
            raise TensorError(self._message(False))


def validate_keys(expected: Sequence[ExpectedParam], actual: Dict[str, List[int]]) -> LoadValidation:
    v = LoadValidation()
    names = {p.key for p in expected}
    for p in expected:
        found = actual.get(p.key)
        if found is None:
            v.missing.append(p.key)
        elif list(found) != list(p.shape):
            v.shape_mismatches.append(ShapeMismatch(p.key, list(p.shape), list(found)))
    v.unused = sorted(k for k in actual if k not in names)
    v.missing.sort()
    v.shape_mismatches.sort(key=lambda m: m.key)
    return v


def expected_from_graph(graph) -> List[ExpectedParam]:
    out = [ExpectedParam(hf_key_from_flodl_key(k), list(p.t.shape)) for k, p in graph.named_parameters()]
    out += [ExpectedParam(hf_key_from_flodl_key(k), list(b.get().shape)) for k, b in graph.named_buffers()]
    return out


# ---- key renames -----------------------------------------------------------------------------------
def bert_legacy_layernorm_rename(key: str) -> str:
    if key.endswith("LayerNorm.gamma"):
        return key[:-len("gamma")] + "weight"
    if key.endswith("LayerNorm.beta"):
        return key[:-len("beta")] + "bias"
    return key


def bert_legacy_key_rename(key: str) -> str:
    """Old TF-style names (`LayerNorm.gamma/beta`) and the MLM decoder bias stored beside the
    decoder (`cls.predictions.bias`, `lm_head.bias`, ALBERT's `predictions.bias`)."""
    if key == "cls.predictions.bias":
        return "cls.predictions.decoder.bias"
    if key == "predictions.bias":
        return "predictions.decoder.bias"
    if key == "lm_head.bias":
        return "lm_head.decoder.bias"
    return bert_legacy_layernorm_rename(key)


def hf_canonical_save_key(key: str) -> str:
    if key == "cls.predictions.decoder.bias":
        return "cls.predictions.bias"
    if key == "lm_head.decoder.bias":
        return "lm_head.bias"
    return key


def _is_pooler_key(key: str) -> bool:
    k = key.replace("/", ".")
    return k.endswith(("pooler.dense.weight", "pooler.dense.bias", "pooler.weight", "pooler.bias"))


def keys_have_pooler(keys: Sequence[str]) -> bool:
    return any(_is_pooler_key(k) for k in keys)


def weights_have_pooler(weights: bytes) -> bool:
    header, _ = parse_header(weights)
    return keys_have_pooler(list(header))


# ---- load ------------------------------------------------------------------------------------------
def _load_core(graph, data: bytes, rename: Callable[[str], str], allow_unused: bool) -> List[str]:
    header, base = parse_header(data)
    canon: Dict[str, str] = {}
    shapes: Dict[str, List[int]] = {}
    for name, info in header.items():
        c = rename(name)
        if c in canon:
            raise TensorError(f"safetensors key rename collision: both {canon[c]!r} and {name!r} map to canonical key {c!r}")
        canon[c] = name
        shapes[c] = [int(s) for s in info["shape"]]
        if info["dtype"] in _INT_DTYPES and c in {e.key for e in expected_from_graph(graph)}:
            raise TensorError(f"unsupported safetensors dtype {info['dtype']} for {name!r} — floats (F32/F64/BF16/F16) only")
    v = validate_keys(expected_from_graph(graph), shapes)
    if allow_unused:
        v.into_result_allow_unused()
    else:
        v.into_result()
    staged = []
    for key, p in graph.named_parameters():
        name = canon[hf_key_from_flodl_key(key)]
        staged.append((p.variable, tensor_from_entry(data, base, name, header[name])))
    staged_b = []
    for key, b in graph.named_buffers():
        name = canon[hf_key_from_flodl_key(key)]
        staged_b.append((b, tensor_from_entry(data, base, name, header[name])))
    for var, src in staged:                                   # commit only after everything parsed
        var.set_data(src.to(device=var.t.device, dtype=var.t.dtype))
    for b, src in staged_b:
        b.set(src.to(device=b.get().device, dtype=b.get().dtype))
    return v.unused


def load_safetensors_into_graph(graph, data: bytes) -> None:
    _load_core(graph, data, lambda k: k, False)


def load_safetensors_into_graph_with_rename(graph, data: bytes, rename: Callable[[str], str]) -> None:
    _load_core(graph, data, rename, False)


def load_safetensors_into_graph_with_rename_allow_unused(graph, data: bytes, rename: Callable[[str], str]) -> List[str]:
    return _load_core(graph, data, rename, True)


def load_safetensors_file_into_graph(graph, path: str) -> None:
    with open(path, "rb") as f:
        load_safetensors_into_graph(graph, f.read())


def load_safetensors_file_into_graph_with_rename(graph, path: str, rename: Callable[[str], str]) -> None:
    with open(path, "rb") as f:
        load_safetensors_into_graph_with_rename(graph, f.read(), rename)


# ---- save ------------------------------------------------------------------------------------------
def save_safetensors_from_graph(graph) -> bytes:
    entries: Dict[str, torch.Tensor] = {}
    owner: Dict[str, int] = {}
    for key, p in graph.named_parameters():
        k = hf_canonical_save_key(hf_key_from_flodl_key(key))
        if k in entries and owner[k] != id(p.t):
            raise TensorError(f"save_safetensors: HF key {k!r} collision — multiple distinct tensors map to the same name; fix the conflicting `tag(...)` in the graph")
        entries[k], owner[k] = p.t.detach(), id(p.t)
    for key, b in graph.named_buffers():
        k = hf_canonical_save_key(hf_key_from_flodl_key(key))
        if k in entries:
            raise TensorError(f"save_safetensors: HF key {k!r} collision — buffer collides with a parameter or another buffer")
        if not b.get().is_floating_point():
            raise TensorError(f"save_safetensors: integer dtype {b.get().dtype} not supported — only floating-point parameters / buffers can be serialised")
        entries[k] = b.get().detach()
    return write_safetensors(entries)


def save_safetensors_file_from_graph(graph, path: str) -> None:
    with open(path, "wb") as f:
        f.write(save_safetensors_from_graph(graph))
