"""`HfTokenizer`: a `tokenizer.json` loaded through the `tokenizers` package, producing the tensors
the encoder graphs take (flodl-hf/src/tokenizer.rs). Padding to the longest sequence of the batch is
switched on if the file does not configure padding itself."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..tensor import TensorError


@dataclass
class EncodedBatch:
    input_ids: torch.Tensor        # [B, S] int64
    attention_mask: torch.Tensor   # [B, S] float32, 1 = token, 0 = padding
    token_type_ids: torch.Tensor   # [B, S] int64
    position_ids: torch.Tensor     # [B, S] int64, 0..S-1
    sequence_ids: Optional[torch.Tensor] = None   # [B, S] int64: 0 / 1 = first / second text of a pair, -1 = special token or padding

    def to(self, device) -> "EncodedBatch":
        return EncodedBatch(*(None if t is None else t.to(device)
                              for t in (self.input_ids, self.attention_mask, self.token_type_ids, self.position_ids, self.sequence_ids)))


class HfTokenizer:
    def __init__(self, inner):
        self._tok = inner
        if self._tok.padding is None:
            pad_id = self._tok.token_to_id("[PAD]")
            pad_tok = "[PAD]"
            if pad_id is None:
                pad_id, pad_tok = self._tok.token_to_id("<pad>"), "<pad>"
            self._tok.enable_padding(pad_id=pad_id if pad_id is not None else 0, pad_token=pad_tok)

    @classmethod
    def from_file(cls, path: str) -> "HfTokenizer":
        try:
            from tokenizers import Tokenizer
        except Exception as e:  # pragma: no cover - environment without the package
            raise TensorError(f"HfTokenizer needs the `tokenizers` package: {e}")
        try:
            return cls(Tokenizer.from_file(str(path)))
        except Exception as e:
            raise TensorError(f"tokenizer load {path}: {e}")

    @classmethod
    def from_pretrained(cls, repo_id: str) -> "HfTokenizer":
        """The `tokenizer.json` of a hub repo or local directory (looked up like the weights: the directory
        itself, the converted-models folder, the hub cache, then a download unless `HF_HUB_OFFLINE=1`)."""
        from . import hub
        path = hub.resolve_tokenizer(repo_id)
        if path is None:
            raise TensorError(f"HfTokenizer.from_pretrained({repo_id}): no tokenizer.json found (looked in {hub.candidate_dirs(repo_id)})")
        return cls.from_file(path)

    @classmethod
    def from_inner(cls, inner) -> "HfTokenizer":
        return cls(inner)

    def inner(self):
        return self._tok

    def save(self, path: str) -> None:
        self._tok.save(str(path))

    def token_to_id(self, token: str) -> Optional[int]:
        return self._tok.token_to_id(token)

    def id_to_token(self, idx: int) -> Optional[str]:
        return self._tok.id_to_token(int(idx))

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self._tok.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def _pack(self, encs, device) -> EncodedBatch:
        ids = torch.tensor([e.ids for e in encs], dtype=torch.long)
        mask = torch.tensor([e.attention_mask for e in encs], dtype=torch.float32)
        tt = torch.tensor([e.type_ids for e in encs], dtype=torch.long)
        pos = torch.arange(ids.shape[1]).unsqueeze(0).expand_as(ids).contiguous()
        seq = torch.tensor([[-1 if s is None else int(s) for s in e.sequence_ids] for e in encs], dtype=torch.long)
        b = EncodedBatch(ids, mask, tt, pos, seq)
        return b if device is None else b.to(device)

    def encode(self, texts: Sequence[str]) -> EncodedBatch:
        return self.encode_on_device(texts, None)

    def encode_on_device(self, texts: Sequence[str], device) -> EncodedBatch:
        if not texts:
            raise TensorError("encode: empty batch")
        return self._pack(self._tok.encode_batch(list(texts)), device)

    def encode_pairs(self, pairs: Sequence[Tuple[str, str]]) -> EncodedBatch:
        return self.encode_pairs_on_device(pairs, None)

    def encode_pairs_on_device(self, pairs: Sequence[Tuple[str, str]], device) -> EncodedBatch:
        if not pairs:
            raise TensorError("encode_pairs: empty batch")
        return self._pack(self._tok.encode_batch([tuple(p) for p in pairs]), device)
