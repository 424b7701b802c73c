"""Decoder-only transformer LM (scaled-up ddp-bench/src/models/gpt_nano.rs: pre-LayerNorm blocks,
GELU feed-forward, learned position embedding, untied vocabulary head).

    x = tok_emb[ids] + pos_emb
    per block:  x = x + dropout(attn(LN1(x)));  x = x + dropout(ffn(LN2(x)))
    logits = head(LN_f(x))

Kernel mapping on CUDA/bf16: each "add + dropout -> LayerNorm" is one fused kernel that returns
both the new residual stream and its normalised value; QKV is one GEMM (weights back to back in the
flat buffer), attention is the causal flash kernel, the FFN is two GEMMs with GELU / GELU' in the
epilogues, and `loss()` fuses the vocabulary projection with the softmax cross-entropy."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from .. import ops as _ops
from ..autograd import Variable
from ..hf.transformer_layer import fused_rows
from ..nn.layers import Embedding, LayerNorm, Linear
from ..nn.module import Module, Parameter


@dataclass
class DecoderLMConfig:
    vocab_size: int = 32000
    d_model: int = 512
    n_layers: int = 6
    n_heads: int = 8
    d_ff: int = 2048
    max_seq: int = 256
    dropout: float = 0.0
    layer_norm_eps: float = 1e-5


class DecoderBlock(Module):
    def __init__(self, cfg: DecoderLMConfig, device=None):
        d = cfg.d_model
        self.cfg = cfg
        self.ln1, self.ln2 = LayerNorm(d, cfg.layer_norm_eps, device), LayerNorm(d, cfg.layer_norm_eps, device)
        self.q, self.k, self.v, self.o = (Linear(d, d, True, device) for _ in range(4))
        self.up, self.down = Linear(d, cfg.d_ff, True, device), Linear(cfg.d_ff, d, True, device)
        self._fused = None

    def name(self): return "decoder_block"
    def sub_modules(self): return [self.ln1, self.q, self.k, self.v, self.o, self.ln2, self.up, self.down]
    def fuse_groups(self): return [[self.q.weight, self.k.weight, self.v.weight], [self.q.bias, self.k.bias, self.v.bias]]

    def _qkv(self, h: torch.Tensor) -> torch.Tensor:
        B, S, d = h.shape
        H, D = self.cfg.n_heads, d // self.cfg.n_heads
        ws = [m.weight.t for m in (self.q, self.k, self.v)]
        bs = [m.bias.t for m in (self.q, self.k, self.v)]
        if h.is_cuda and getattr(ws[0], "_fb_flat", None) is not None:
            if self._fused is None or self._fused[0].data_ptr() != ws[0].data_ptr():
                fw, fb = fused_rows(ws), fused_rows(bs)
                self._fused = (fw, fb) if fw is not None and fb is not None else (ws[0], None)
            if self._fused[1] is not None:
                return _ops.linear(h, self._fused[0], self._fused[1]).view(B, S, 3, H, D)
        return torch.stack([_ops.linear(h, w, b).view(B, S, H, D) for w, b in zip(ws, bs)], dim=2)

    def forward_pair(self, delta, stream):
        """`delta` is the previous sub-layer output not yet added to the residual `stream` (or None)."""
        c = self.cfg
        p = c.dropout
        if delta is None:
            h1, x = _ops.layer_norm(stream, self.ln1.weight.t, self.ln1.bias.t, c.layer_norm_eps), stream
        else:
            h1, x = _ops.layer_norm(delta, self.ln1.weight.t, self.ln1.bias.t, c.layer_norm_eps, residual=stream, p_drop=p,
                                    training=self.training, return_pre=True)
        B, S, d = x.shape
        ctx = _ops.attention(self._qkv(h1), causal=True, p_drop=0.0, training=self.training)
        a = _ops.linear(ctx.reshape(B, S, d), self.o.weight.t, self.o.bias.t)
        h2, x2 = _ops.layer_norm(a, self.ln2.weight.t, self.ln2.bias.t, c.layer_norm_eps, residual=x, p_drop=p, training=self.training,
                                 return_pre=True)
        f = _ops.feed_forward(h2, self.up.weight.t, self.up.bias.t, self.down.weight.t, self.down.bias.t, "gelu")
        return f, x2

    def forward(self, x: Variable) -> Variable:
        f, s = self.forward_pair(None, x.t)
        return Variable.wrap(s + _ops.dropout(f, self.cfg.dropout, self.training))


class DecoderLM(Module):
    def __init__(self, cfg: DecoderLMConfig, device=None):
        self.cfg = cfg
        self.tok = Embedding(cfg.vocab_size, cfg.d_model, None, device)
        self.pos = Embedding(cfg.max_seq, cfg.d_model, None, device)
        self.blocks: List[DecoderBlock] = [DecoderBlock(cfg, device) for _ in range(cfg.n_layers)]
        self.ln_f = LayerNorm(cfg.d_model, cfg.layer_norm_eps, device)
        self.head = Linear(cfg.d_model, cfg.vocab_size, False, device)

    def name(self): return "decoder_lm"
    def sub_modules(self): return [self.tok, self.pos, *self.blocks, self.ln_f, self.head]

    def hidden(self, ids: torch.Tensor) -> torch.Tensor:
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device)
        x = self.tok.forward(Variable.wrap(ids)).t + self.pos.forward(Variable.wrap(pos)).t
        if x.is_cuda and _ops.FLAGS.autocast == torch.bfloat16:
            x = x.to(torch.bfloat16)
        delta = None
        for blk in self.blocks:
            delta, x = blk.forward_pair(delta, x)
        c = self.cfg
        return _ops.layer_norm(delta, self.ln_f.weight.t, self.ln_f.bias.t, c.layer_norm_eps, residual=x, p_drop=c.dropout,
                               training=self.training)

    def forward(self, ids: Variable) -> Variable:
        return Variable.wrap(_ops.linear(self.hidden(ids.t), self.head.weight.t, None))

    def loss(self, ids: torch.Tensor, targets: torch.Tensor) -> Variable:
        """Mean next-token cross-entropy; projection + loss fused on CUDA."""
        h = self.hidden(ids)
        return Variable.wrap(_ops.linear_cross_entropy(h, self.head.weight.t, None, targets.reshape(-1), -100))
