"""The eleven benchmark models (benchmarks/src/tier1/*.rs, tier2/*.rs), each built twice: with this
framework's modules / `FlowBuilder`, and as a plain `torch.nn` module with the same shapes. A model
entry returns `(forward, parameters, make_batch, loss)` for the requested implementation."""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Tuple

import torch
import torch.nn as tnn
import torch.nn.functional as F

from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder, LearnedHalt, SoftmaxRouter
from flodl_b200.nn.module import Module

from .harness import BenchConfig


# ------------------------------------------------------------------------------------ helpers
def _ln_block(dim, device):
    return FlowBuilder.from_(nn.Linear(dim, dim, True, device)).through(nn.GELU()).through(nn.LayerNorm(dim, device=device)).build()


class _TBlock(tnn.Module):
    def __init__(self, dim):
        super().__init__()
        self.l, self.n = tnn.Linear(dim, dim), tnn.LayerNorm(dim)

    def forward(self, x):
        return self.n(F.gelu(self.l(x)))


def _mse(pred, target):
    return nn.mse_loss(pred, target)


def _randn_pair(shape_x, shape_y):
    def make(device, gen):
        return (torch.randn(*shape_x, generator=gen).to(device), torch.randn(*shape_y, generator=gen).to(device))
    return make


# ------------------------------------------------------------------------------------ tier 1
def mlp(cfg: BenchConfig, impl, device, scale=1):
    D, Hd = 1024 // scale, 2048 // scale
    dims = [D, Hd, Hd, Hd, Hd]
    if impl == "flodl":
        b = FlowBuilder.from_(nn.Linear(D, Hd, True, device)).through(nn.GELU()).through(nn.LayerNorm(Hd, device=device))
        for _ in range(3):
            b = b.through(nn.Linear(Hd, Hd, True, device)).through(nn.GELU()).through(nn.LayerNorm(Hd, device=device))
        model = b.through(nn.Linear(Hd, D, True, device)).build()
    else:
        layers = []
        for i, o in zip(dims[:-1], dims[1:]):
            layers += [tnn.Linear(i, o), tnn.GELU(), tnn.LayerNorm(o)]
        model = tnn.Sequential(*layers, tnn.Linear(Hd, D)).to(device)
    return model, _randn_pair((cfg.batch_size, D), (cfg.batch_size, D)), "mse", 1e-3


class _ClassifyHead(Module):
    """Global average pool + Linear (benchmarks/src/tier1/convnet.rs:9-33)."""
    def __init__(self, c, n, device): self.linear = nn.Linear(c, n, True, device)
    def name(self): return "classify_head"
    def sub_modules(self): return [self.linear]
    def forward(self, x): return self.linear.forward(Variable.wrap(x.t.mean((2, 3))))


def convnet(cfg, impl, device, scale=1):
    ch = [3] + [c // scale for c in (64, 128, 256, 512, 512)]
    HW = 64 // (2 if scale > 1 else 1)
    if impl == "flodl":
        b = None
        for i in range(5):
            conv = nn.Conv2d.configure(ch[i], ch[i + 1], 3).with_padding(1).on_device(device).done()
            b = FlowBuilder.from_(conv) if b is None else b.through(conv)
            b = b.through(nn.BatchNorm2d(ch[i + 1], device)).through(nn.ReLU())
            if i < 4:
                b = b.through(nn.MaxPool2d(2))
        model = b.through(_ClassifyHead(ch[5], 100, device)).build()
    else:
        layers = []
        for i in range(5):
            layers += [tnn.Conv2d(ch[i], ch[i + 1], 3, padding=1), tnn.BatchNorm2d(ch[i + 1]), tnn.ReLU()]
            if i < 4:
                layers.append(tnn.MaxPool2d(2))
        model = tnn.Sequential(*layers, tnn.AdaptiveAvgPool2d(1), tnn.Flatten(), tnn.Linear(ch[5], 100)).to(device)
    return model, _randn_pair((cfg.batch_size, 3, HW, HW), (cfg.batch_size, 100)), "mse", 1e-3


def conv_autoencoder(cfg, impl, device, scale=1):
    ch = [3] + [c // scale for c in (64, 128, 256, 512)]
    HW = 64 // (2 if scale > 1 else 1)
    if impl == "flodl":
        b = None
        for i in range(4):
            conv = nn.Conv2d.configure(ch[i], ch[i + 1], 4).with_stride(2).with_padding(1).on_device(device).done()
            b = FlowBuilder.from_(conv) if b is None else b.through(conv)
            b = b.through(nn.BatchNorm2d(ch[i + 1], device)).through(nn.ReLU())
        for i in range(4, 0, -1):
            b = b.through(nn.ConvTranspose2d.build(ch[i], ch[i - 1], 4, True, 2, 1, 1, 1, device))
            b = b.through(nn.BatchNorm2d(ch[i - 1], device)).through(nn.ReLU()) if i > 1 else b.through(nn.Tanh())
        model = b.build()
    else:
        layers = []
        for i in range(4):
            layers += [tnn.Conv2d(ch[i], ch[i + 1], 4, 2, 1), tnn.BatchNorm2d(ch[i + 1]), tnn.ReLU()]
        for i in range(4, 0, -1):
            layers.append(tnn.ConvTranspose2d(ch[i], ch[i - 1], 4, 2, 1))
            layers += [tnn.BatchNorm2d(ch[i - 1]), tnn.ReLU()] if i > 1 else [tnn.Tanh()]
        model = tnn.Sequential(*layers).to(device)

    def make(dev, gen):
        x = torch.randn(cfg.batch_size, 3, HW, HW, generator=gen).to(dev)
        return x, x.clone()
    return model, make, "mse", 1e-3


class _GruSeq(Module):
    def __init__(self, i, h, steps, device):
        self.gru, self.out, self.steps = nn.GRUCell(i, h, device), nn.Linear(h, i, True, device), steps
    def name(self): return "gru_seq"
    def sub_modules(self): return [self.gru, self.out]
    def forward(self, x):
        h = None
        for t in range(self.steps):
            h = self.gru.forward_step(x.select(1, t), h)
        return self.out.forward(h)


class _TGruSeq(tnn.Module):
    def __init__(self, i, h, steps):
        super().__init__()
        self.gru, self.out, self.steps = tnn.GRUCell(i, h), tnn.Linear(h, i), steps

    def forward(self, x):
        h = None
        for t in range(self.steps):
            h = self.gru(x[:, t], h)
        return self.out(h)


def gru_seq(cfg, impl, device, scale=1):
    S, I, Hd = 50 // (5 if scale > 1 else 1), 256 // scale, 512 // scale
    model = _GruSeq(I, Hd, S, device) if impl == "flodl" else _TGruSeq(I, Hd, S).to(device)
    return model, _randn_pair((cfg.batch_size, S, I), (cfg.batch_size, I)), "mse", 1e-3


class _LstmSeq(Module):
    def __init__(self, i, h, layers, device):
        self.lstm, self.out = nn.LSTM(i, h, layers, device).batch_first(True), nn.Linear(h, i, True, device)
    def name(self): return "lstm_seq"
    def sub_modules(self): return [self.lstm, self.out]
    def forward(self, x):
        out, _ = self.lstm.forward_seq(x)
        return self.out.forward(out.select(1, out.t.shape[1] - 1))


class _TLstmSeq(tnn.Module):
    def __init__(self, i, h, layers):
        super().__init__()
        self.lstm, self.out = tnn.LSTM(i, h, layers, batch_first=True), tnn.Linear(h, i)

    def forward(self, x):
        return self.out(self.lstm(x)[0][:, -1])


def lstm_seq(cfg, impl, device, scale=1):
    S, I, Hd = 50 // (5 if scale > 1 else 1), 256 // scale, 512 // scale
    model = _LstmSeq(I, Hd, 2, device) if impl == "flodl" else _TLstmSeq(I, Hd, 2).to(device)
    return model, _randn_pair((cfg.batch_size, S, I), (cfg.batch_size, I)), "mse", 1e-3


class _EncoderLayer(Module):
    def __init__(self, d, ff, heads, device):
        self.mha = nn.MultiheadAttention(d, heads, device)
        self.n1, self.n2 = nn.LayerNorm(d, device=device), nn.LayerNorm(d, device=device)
        self.f1, self.f2 = nn.Linear(d, ff, True, device), nn.Linear(ff, d, True, device)
    def name(self): return "encoder_layer"
    def sub_modules(self): return [self.mha, self.n1, self.f1, self.f2, self.n2]
    def forward(self, x):
        x = self.n1.forward(x.add(self.mha.forward(x)))
        return self.n2.forward(x.add(self.f2.forward(self.f1.forward(x).gelu())))


class _Transformer(Module):
    def __init__(self, vocab, d, ff, heads, layers, seq, device):
        self.emb = nn.Embedding(vocab, d, device=device)
        self.pos = nn.Parameter(torch.randn(1, seq, d, device=device), "pos_embed")
        self.layers = [_EncoderLayer(d, ff, heads, device) for _ in range(layers)]
        self.out = nn.Linear(d, vocab, True, device)
    def name(self): return "transformer"
    def sub_modules(self): return [self.emb, *self.layers, self.out]
    def own_parameters(self): return [self.pos]
    def forward(self, ids):
        x = self.emb.forward(ids).add(self.pos.variable)
        for layer in self.layers:
            x = layer.forward(x)
        return self.out.forward(x)


class _TTransformer(tnn.Module):
    def __init__(self, vocab, d, ff, heads, layers, seq):
        super().__init__()
        self.emb, self.pos = tnn.Embedding(vocab, d), tnn.Parameter(torch.randn(1, seq, d))
        self.layers = tnn.ModuleList([tnn.TransformerEncoderLayer(d, heads, ff, 0.0, F.gelu, batch_first=True) for _ in range(layers)])
        self.out = tnn.Linear(d, vocab)

    def forward(self, ids):
        x = self.emb(ids) + self.pos
        for layer in self.layers:
            x = layer(x)
        return self.out(x)


def transformer(cfg, impl, device, scale=1):
    V, D, FF, Hh, L, S = 8192 // scale, 512 // scale, 2048 // scale, 8, 4 if scale == 1 else 2, 128 // (4 if scale > 1 else 1)
    model = _Transformer(V, D, FF, Hh, L, S, device) if impl == "flodl" else _TTransformer(V, D, FF, Hh, L, S).to(device)

    def make(dev, gen):
        return (torch.randint(0, V, (cfg.batch_size, S), generator=gen).to(dev), torch.randint(0, V, (cfg.batch_size, S), generator=gen).to(dev))
    return model, make, "ce", 1e-4


# ------------------------------------------------------------------------------------ tier 2
class _TResidualLoop(tnn.Module):
    """x = proj(x); n times x = x + block(x) (one shared block, or `blocks` distinct ones); out(x)."""
    def __init__(self, dim, n, shared, halt=False, pre_norm=True):
        super().__init__()
        self.inp = tnn.Linear(dim, dim)
        self.pre = tnn.LayerNorm(dim) if pre_norm else None
        self.blocks = tnn.ModuleList([_TBlock(dim) for _ in range(1 if shared else n)])
        self.n, self.shared = n, shared
        self.halt = tnn.Linear(dim, 1) if halt else None
        self.out = tnn.Linear(dim, dim)

    def forward(self, x):
        x = self.inp(x)
        if self.pre is not None:
            x = self.pre(F.gelu(x))
        for i in range(self.n):
            blk = self.blocks[0 if self.shared else i]
            x = x + blk(x)
            if self.halt is not None and float(self.halt(x).reshape(-1)[0]) > 0.0:
                break
        return self.out(x)


def residual_tower(cfg, impl, device, scale=1):
    D, n = 1024 // scale, 12
    if impl == "flodl":
        b = FlowBuilder.from_(nn.Linear(D, D, True, device))
        for _ in range(n):
            b = b.also(_ln_block(D, device))
        model = b.through(nn.Linear(D, D, True, device)).build()
    else:
        model = _TResidualLoop(D, n, shared=False, pre_norm=False).to(device)
    return model, _randn_pair((cfg.batch_size, D), (cfg.batch_size, D)), "mse", 1e-3


def _loop_model(D, device, finish: Callable):
    body = FlowBuilder.new().also(_ln_block(D, device)).build()
    b = FlowBuilder.from_(nn.Linear(D, D, True, device)).through(nn.GELU()).through(nn.LayerNorm(D, device=device)).loop_body(body)
    return finish(b).through(nn.Linear(D, D, True, device)).build()


def feedback_loop(cfg, impl, device, scale=1):
    D = 512 // scale
    if impl == "flodl":
        model = _loop_model(D, device, lambda b: b.until_cond(LearnedHalt(D, device), 10))
    else:
        model = _TResidualLoop(D, 10, shared=True, halt=True).to(device)
    return model, _randn_pair((cfg.batch_size, D), (cfg.batch_size, D)), "mse", 1e-3


def feedback_loop_fixed(cfg, impl, device, scale=1):
    D = 512 // scale
    model = _loop_model(D, device, lambda b: b.for_n(10)) if impl == "flodl" else _TResidualLoop(D, 10, shared=True).to(device)
    return model, _randn_pair((cfg.batch_size, D), (cfg.batch_size, D)), "mse", 1e-3


def iterative_refine(cfg, impl, device, scale=1):
    D = 1024 // scale
    model = _loop_model(D, device, lambda b: b.for_n(8)) if impl == "flodl" else _TResidualLoop(D, 8, shared=True).to(device)
    return model, _randn_pair((cfg.batch_size, D), (cfg.batch_size, D)), "mse", 1e-3


class _TGated(tnn.Module):
    def __init__(self, dim, experts):
        super().__init__()
        self.inp, self.router, self.out = tnn.Linear(dim, dim), tnn.Linear(dim, experts), tnn.Linear(dim, dim)
        self.experts = tnn.ModuleList([_TBlock(dim) for _ in range(experts)])

    def forward(self, x):
        x = F.gelu(self.inp(x))
        w = self.router(x).softmax(-1)
        y = torch.stack([e(x) for e in self.experts], -1)
        return self.out((y * w.unsqueeze(-2)).sum(-1))


def gated_routing(cfg, impl, device, scale=1):
    D, E = 512 // scale, 8
    if impl == "flodl":
        model = (FlowBuilder.from_(nn.Linear(D, D, True, device)).through(nn.GELU())
                 .gate(SoftmaxRouter(D, E, device), [_ln_block(D, device) for _ in range(E)])
                 .through(nn.Linear(D, D, True, device)).build())
    else:
        model = _TGated(D, E).to(device)
    return model, _randn_pair((cfg.batch_size, D), (cfg.batch_size, D)), "mse", 1e-3


MODELS: Dict[str, Tuple[Callable, BenchConfig]] = {
    "mlp": (mlp, BenchConfig("mlp", batch_size=256, batches_per_epoch=50)),
    "convnet": (convnet, BenchConfig("convnet", batch_size=128, batches_per_epoch=50)),
    "conv_autoencoder": (conv_autoencoder, BenchConfig("conv_autoencoder", batch_size=64, batches_per_epoch=50)),
    "gru_seq": (gru_seq, BenchConfig("gru_seq", batch_size=128, batches_per_epoch=50)),
    "lstm_seq": (lstm_seq, BenchConfig("lstm_seq", batch_size=128, batches_per_epoch=50)),
    "transformer": (transformer, BenchConfig("transformer", batch_size=32, batches_per_epoch=50)),
    "residual_tower": (residual_tower, BenchConfig("residual_tower", batch_size=256, batches_per_epoch=50)),
    "feedback_loop": (feedback_loop, BenchConfig("feedback_loop", batch_size=128, batches_per_epoch=50)),
    "feedback_loop_fixed": (feedback_loop_fixed, BenchConfig("feedback_loop_fixed", batch_size=128, batches_per_epoch=50)),
    "gated_routing": (gated_routing, BenchConfig("gated_routing", batch_size=256, batches_per_epoch=50)),
    "iterative_refine": (iterative_refine, BenchConfig("iterative_refine", batch_size=256, batches_per_epoch=50)),
}
TIER1 = ["mlp", "convnet", "conv_autoencoder", "gru_seq", "lstm_seq", "transformer"]
TIER2 = ["residual_tower", "feedback_loop", "feedback_loop_fixed", "gated_routing", "iterative_refine"]
