"""Post-LN encoder block shared by BERT / RoBERTa / XLM-R / DistilBERT / ALBERT
(flodl-hf/src/models/transformer_layer.rs:224-263):

    Q,K,V = Linear(x) -> attention(mask, dropout) -> Linear -> dropout -> +x -> LayerNorm
          -> Linear -> GELU -> Linear -> dropout -> +residual -> LayerNorm

Kernel mapping on CUDA/bf16: one fused QKV GEMM (the three weights sit back to back in the flat
parameter buffer, so they are addressed as one [3H, H] operand), the flash-attention kernel on the
packed QKV, an output-projection GEMM, fused dropout+residual+LayerNorm, the two FFN GEMMs with
GELU in the first epilogue (and GELU' in the backward epilogue), fused dropout+residual+LayerNorm.
`LayerNaming` carries the per-family HuggingFace key suffixes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import ops as _ops
from ..autograd import Variable
from ..nn.activation import GeluApprox
from ..nn.layers import LayerNorm, Linear
from ..nn.module import Module, Parameter
from ..parallel import flat as _flat
from ..tensor import TensorError
from .path import prefix_params


@dataclass(frozen=True)
class LayerNaming:
    query: str
    key: str
    value: str
    attn_output: str
    attn_layer_norm: str
    ffn_up: str
    ffn_down: str
    ffn_layer_norm: str


LayerNaming.BERT = LayerNaming("attention.self.query", "attention.self.key", "attention.self.value", "attention.output.dense",
                               "attention.output.LayerNorm", "intermediate.dense", "output.dense", "output.LayerNorm")
LayerNaming.DISTILBERT = LayerNaming("attention.q_lin", "attention.k_lin", "attention.v_lin", "attention.out_lin", "sa_layer_norm",
                                     "ffn.lin1", "ffn.lin2", "output_layer_norm")
LayerNaming.ALBERT = LayerNaming("attention.query", "attention.key", "attention.value", "attention.dense", "attention.LayerNorm",
                                 "ffn", "ffn_output", "full_layer_layer_norm")


@dataclass
class TransformerLayerConfig:
    hidden_size: int
    num_attention_heads: int
    intermediate_size: int
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-12
    hidden_act: GeluApprox = GeluApprox.Exact


def fused_rows(tensors: List[torch.Tensor]) -> Optional[torch.Tensor]:
    """If `tensors` (same trailing shape) lie back to back in one FlatParams buffer, return a tensor
    that views them as one `[sum rows, ...]` operand and carries the matching bf16-shadow and
    gradient-slot views; else None."""
    first = getattr(tensors[0], "_fb_flat", None)
    if first is None:
        return None
    flat, off, _ = first
    expect = off
    for t in tensors:
        f = getattr(t, "_fb_flat", None)
        if f is None or f[0] is not flat or f[1] != expect or f[2] % _flat.ALIGN:
            return None
        expect += f[2]
    rows = sum(t.shape[0] for t in tensors)
    shape = (rows,) + tuple(tensors[0].shape[1:])
    fused = flat.params[off:expect].view(shape)
    fused.requires_grad_(any(t.requires_grad for t in tensors))
    fused._fb_grad = flat.grads[off:expect].view(shape)
    fused._fb_members = list(tensors)
    if flat.shadow is not None:
        fused._fb_bf16 = flat.shadow[off:expect].view(shape)
    return fused


class TransformerLayer(Module):
    def __init__(self, config: TransformerLayerConfig, naming: LayerNaming = LayerNaming.BERT, device=None):
        if config.hidden_size % config.num_attention_heads:
            raise TensorError(f"hidden_size ({config.hidden_size}) must be divisible by num_attention_heads ({config.num_attention_heads})")
        H, I = config.hidden_size, config.intermediate_size
        self.cfg, self.naming = config, naming
        self.num_heads, self.head_dim = config.num_attention_heads, H // config.num_attention_heads
        self.query, self.key, self.value = Linear(H, H, True, device), Linear(H, H, True, device), Linear(H, H, True, device)
        self.attn_output = Linear(H, H, True, device)
        self.attn_layer_norm = LayerNorm(H, config.layer_norm_eps, device)
        self.ffn_up, self.ffn_down = Linear(H, I, True, device), Linear(I, H, True, device)
        self.ffn_layer_norm = LayerNorm(H, config.layer_norm_eps, device)
        self.act = "gelu" if config.hidden_act == GeluApprox.Exact else "gelu_tanh"
        self._fused = None

    @classmethod
    def on_device(cls, config, naming, device):
        return cls(config, naming, device)

    def name(self):
        return "transformer_layer"

    def own_parameters(self) -> List[Parameter]:
        n = self.naming
        out = []
        for prefix, m in ((n.query, self.query), (n.key, self.key), (n.value, self.value), (n.attn_output, self.attn_output),
                          (n.attn_layer_norm, self.attn_layer_norm), (n.ffn_up, self.ffn_up), (n.ffn_down, self.ffn_down),
                          (n.ffn_layer_norm, self.ffn_layer_norm)):
            out.extend(prefix_params(prefix, m.own_parameters()))
        return out

    def fuse_groups(self):
        return [[self.query.weight, self.key.weight, self.value.weight], [self.query.bias, self.key.bias, self.value.bias]]

    def _qkv(self, x: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        Hn, D = self.num_heads, self.head_dim
        ws = [self.query.weight.t, self.key.weight.t, self.value.weight.t]
        bs = [self.query.bias.t, self.key.bias.t, self.value.bias.t]
        if x.is_cuda and getattr(ws[0], "_fb_flat", None) is not None:
            if self._fused is None or self._fused[0].data_ptr() != ws[0].data_ptr():
                fw, fb = fused_rows(ws), fused_rows(bs)
                self._fused = (fw, fb) if fw is not None and fb is not None else (ws[0], None)
            fw, fb = self._fused
            if fb is not None:
                return _ops.linear(x, fw, fb).view(B, S, 3, Hn, D)
        q, k, v = (_ops.linear(x, w, b).view(B, S, Hn, D) for w, b in zip(ws, bs))
        return torch.stack((q, k, v), dim=2)

    def forward_impl(self, x: Variable, attention_mask: Optional[Variable]) -> Variable:
        c = self.cfg
        t = x.t
        B, S, H = t.shape
        qkv = self._qkv(t)
        ctx = _ops.attention(qkv, mask=None if attention_mask is None else attention_mask.t, causal=False,
                             p_drop=c.attention_probs_dropout_prob, training=self.training)
        proj = _ops.linear(ctx.reshape(B, S, H), self.attn_output.weight.t, self.attn_output.bias.t)
        h1 = _ops.layer_norm(proj, self.attn_layer_norm.weight.t, self.attn_layer_norm.bias.t, c.layer_norm_eps, residual=t,
                             p_drop=c.hidden_dropout_prob, training=self.training)
        ffn = _ops.feed_forward(h1, self.ffn_up.weight.t, self.ffn_up.bias.t, self.ffn_down.weight.t, self.ffn_down.bias.t, self.act)
        out = _ops.layer_norm(ffn, self.ffn_layer_norm.weight.t, self.ffn_layer_norm.bias.t, c.layer_norm_eps, residual=h1,
                              p_drop=c.hidden_dropout_prob, training=self.training)
        return Variable.wrap(out)

    def forward(self, x: Variable) -> Variable:
        return self.forward_impl(x, None)

    def forward_named(self, x: Variable, refs: Dict[str, Variable]) -> Variable:
        return self.forward_impl(x, refs.get("attention_mask"))
