"""The eight validation models (ddp-bench/src/models/*.rs) on synthetic data of the right shape: there is no
network here, so each dataset is a fixed-seed teacher task (labels produced by a frozen random network of
the same family), which keeps "does the distributed run reach the solo loss" meaningful."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

import torch

from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder
from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
from flodl_b200.models.resnet import BasicBlock, ResNet20
from flodl_b200.nn.module import Module


@dataclass
class ModelDefaults:
    epochs: int = 5
    batches_per_epoch: int = 100
    batch_size: int = 64
    lr: float = 0.01
    momentum: float = 0.9
    optimizer: str = "sgd"


@dataclass
class ModelDef:
    name: str
    description: str
    build: Callable                                  # (device, tiny) -> Module
    dataset: Callable                                # (n, seed, tiny) -> (inputs, targets) CPU tensors
    train_fn: Callable                               # (model, batch) -> loss Variable
    eval_fn: Callable                                # (model, inputs, targets) -> float
    defaults: ModelDefaults = field(default_factory=ModelDefaults)
    reference: str = ""
    published_eval: Optional[float] = None
    eval_higher_is_better: bool = True
    graph: bool = False                              # built with FlowBuilder (the `sync` mode needs a graph)

    def optimizer(self, lr: float) -> Callable:
        d = self.defaults
        return (lambda ps: nn.Adam(ps, lr)) if d.optimizer == "adam" else (lambda ps: nn.SGD(ps, lr, d.momentum))


def _ce(m, batch):
    return nn.cross_entropy_loss(m.forward(Variable.wrap(batch[0])), Variable.wrap(batch[1]))


def _accuracy(m, x, y):
    with torch.no_grad():
        return float((m.forward(Variable.wrap(x)).t.argmax(-1) == y).float().mean())


def _teacher_labels(x: torch.Tensor, classes: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(x[0].numel(), classes, generator=g)
    return (x.reshape(x.shape[0], -1) @ w).argmax(-1)


def _image_task(shape, classes):
    def make(n, seed, tiny):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(n, *shape, generator=g)
        return x, _teacher_labels(x, classes, 1234)
    return make


# ---- logistic / mlp / lenet --------------------------------------------------------------------
def _logistic(device, tiny):
    return FlowBuilder.from_(nn.Flatten()).through(nn.Linear(784, 10, True, device)).build()


def _mlp(device, tiny):
    h1, h2 = (32, 16) if tiny else (256, 128)
    return (FlowBuilder.from_(nn.Flatten()).through(nn.Linear(784, h1, True, device)).through(nn.ReLU())
            .through(nn.Linear(h1, h2, True, device)).through(nn.ReLU()).through(nn.Linear(h2, 10, True, device)).build())


def _lenet(device, tiny):
    return (FlowBuilder.from_(nn.Conv2d(1, 6, 5, 1, 2, device=device)).through(nn.ReLU()).through(nn.MaxPool2d(2))
            .through(nn.Conv2d(6, 16, 5, device=device)).through(nn.ReLU()).through(nn.MaxPool2d(2)).through(nn.Flatten())
            .through(nn.Linear(400, 120, True, device)).through(nn.ReLU()).through(nn.Linear(120, 84, True, device)).through(nn.ReLU())
            .through(nn.Linear(84, 10, True, device)).build())


# ---- resnet (hand-written module) and resnet_graph (FlowBuilder) ----------------------------------
def _resnet(device, tiny):
    return ResNet20(10, device)


class _Shortcut(Module):
    def __init__(self, i, o, s, device):
        self.conv, self.bn = nn.Conv2d(i, o, 1, s, 0, bias=False, device=device), nn.BatchNorm2d(o, device)
    def name(self): return "shortcut"
    def sub_modules(self): return [self.conv, self.bn]
    def forward(self, x): return self.bn.forward(self.conv.forward(x))


def _resnet_graph(device, tiny):
    b = FlowBuilder.from_(nn.Conv2d(3, 16, 3, 1, 1, bias=False, device=device)).through(nn.BatchNorm2d(16, device)).through(nn.ReLU())
    in_c = 16
    for out_c, stride in ((16, 1), (32, 2), (64, 2)):
        for i in range(1 if tiny else 3):
            s = stride if i == 0 else 1
            main = (FlowBuilder.from_(nn.Conv2d(in_c, out_c, 3, s, 1, bias=False, device=device)).through(nn.BatchNorm2d(out_c, device))
                    .through(nn.ReLU()).through(nn.Conv2d(out_c, out_c, 3, 1, 1, bias=False, device=device))
                    .through(nn.BatchNorm2d(out_c, device)).build())
            b = b.also(main) if (s == 1 and in_c == out_c) else b.also_with(_Shortcut(in_c, out_c, s, device), main)
            b = b.through(nn.ReLU())
            in_c = out_c
    return b.through(nn.AdaptiveAvgPool2d(1)).through(nn.Flatten()).through(nn.Linear(64, 10, True, device)).build()


# ---- char_rnn / gpt_nano (next-token prediction on a synthetic Markov text) -------------------------
VOCAB = 65


def _markov_text(n, seq, seed):
    g = torch.Generator().manual_seed(seed)
    trans = torch.softmax(torch.randn(VOCAB, VOCAB, generator=torch.Generator().manual_seed(99)) * 2.0, -1)
    ids = torch.empty(n, seq + 1, dtype=torch.long)
    ids[:, 0] = torch.randint(0, VOCAB, (n,), generator=g)
    for t in range(seq):
        ids[:, t + 1] = torch.multinomial(trans[ids[:, t]], 1, generator=g).squeeze(1)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


class _CharRnn(Module):
    def __init__(self, hidden, device):
        self.emb = nn.Embedding(VOCAB, hidden, device=device)
        self.rnn = nn.GRU(hidden, hidden, 1, device).batch_first(True)
        self.out = nn.Linear(hidden, VOCAB, True, device)
    def name(self): return "char_rnn"
    def sub_modules(self): return [self.emb, self.rnn, self.out]
    def forward(self, ids):
        h, _ = self.rnn.forward_seq(self.emb.forward(ids))
        return self.out.forward(h)


def _seq_ce(m, batch):
    logits = m.forward(Variable.wrap(batch[0]))
    return nn.cross_entropy_loss(logits.reshape([-1, VOCAB]), Variable.wrap(batch[1].reshape(-1)))


def _seq_loss_eval(m, x, y):
    with torch.no_grad():
        return float(_seq_ce(m, (x, y)).t)


def _char_rnn(device, tiny):
    return _CharRnn(32 if tiny else 128, device)


def _gpt_nano(device, tiny):
    return DecoderLM(DecoderLMConfig(VOCAB, 32 if tiny else 128, 1 if tiny else 4, 4, 64 if tiny else 512, 64), device)


# ---- conv autoencoder -----------------------------------------------------------------------------
def _conv_ae(device, tiny):
    c = 4 if tiny else 16
    return (FlowBuilder.from_(nn.Conv2d(1, c, 3, 2, 1, device=device)).through(nn.ReLU()).through(nn.Conv2d(c, 2 * c, 3, 2, 1, device=device))
            .through(nn.ReLU()).through(nn.ConvTranspose2d(2 * c, c, 3, 2, 1, 1, 1, True, 1, device)).through(nn.ReLU())
            .through(nn.ConvTranspose2d(c, 1, 3, 2, 1, 1, 1, True, 1, device)).through(nn.Sigmoid()).build())


def _ae_data(n, seed, tiny):
    g = torch.Generator().manual_seed(seed)
    base = torch.rand(n, 1, 7, 7, generator=g)
    x = torch.nn.functional.interpolate(base, size=28, mode="bilinear", align_corners=False)
    return x, x.clone()


def _mse(m, batch):
    return nn.mse_loss(m.forward(Variable.wrap(batch[0])), Variable.wrap(batch[1]))


def _mse_eval(m, x, y):
    with torch.no_grad():
        return float(_mse(m, (x, y)).t)


def all_models() -> List[ModelDef]:
    img = _image_task((1, 28, 28), 10)
    cifar = _image_task((3, 32, 32), 10)
    text = lambda n, seed, tiny: _markov_text(n, 32 if tiny else 64, seed)
    return [
        ModelDef("logistic", "784 -> 10 linear classifier", _logistic, img, _ce, _accuracy, ModelDefaults(lr=0.05), "MNIST logistic regression", 0.92, graph=True),
        ModelDef("mlp", "784-256-128-10 ReLU MLP", _mlp, img, _ce, _accuracy, ModelDefaults(lr=0.05), "MNIST MLP", 0.98, graph=True),
        ModelDef("lenet", "LeNet-5", _lenet, img, _ce, _accuracy, ModelDefaults(lr=0.05), "MNIST LeNet-5", 0.99, graph=True),
        ModelDef("resnet", "ResNet-20 (hand-written blocks)", _resnet, cifar, _ce, _accuracy, ModelDefaults(batch_size=128, lr=0.1), "CIFAR-10 ResNet-20 (He et al.)", 0.9125),
        ModelDef("resnet_graph", "ResNet-20 as a FlowBuilder graph", _resnet_graph, cifar, _ce, _accuracy, ModelDefaults(batch_size=128, lr=0.1), "CIFAR-10 ResNet-20 (He et al.)", 0.9125, graph=True),
        ModelDef("char_rnn", "embedding + GRU + projection, next-character", _char_rnn, text, _seq_ce, _seq_loss_eval, ModelDefaults(optimizer="adam", lr=2e-3), "Shakespeare char-RNN", None, False),
        ModelDef("gpt_nano", "4-layer 128-wide decoder LM, next-character", _gpt_nano, text, _seq_ce, _seq_loss_eval, ModelDefaults(optimizer="adam", lr=1e-3), "nanoGPT Shakespeare-char", None, False),
        ModelDef("conv_ae", "convolutional autoencoder", _conv_ae, _ae_data, _mse, _mse_eval, ModelDefaults(optimizer="adam", lr=1e-3), "MNIST conv autoencoder", None, False, graph=True),
    ]


def find_model(name: str) -> Optional[ModelDef]:
    return next((m for m in all_models() if m.name == name), None)
